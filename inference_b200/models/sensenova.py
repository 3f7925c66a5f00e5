"""SenseNova-U1 (NEO-Unify) unified multimodal backbone, text-to-image path (parity: candle-gen-sensenova/src/{qwen3,fm,
vision,config,t2i,distill}.rs).

One dense Qwen3 decoder with two parameter sets per layer ("mixture of transformers"): an understanding path (plain key
names) and a generation path (`*_mot_gen`). There is no autoencoder and no separate text encoder: the prompt is
prefilled on the understanding path into a key / value cache; then, at every flow-matching step, the noisy RGB image is
patch-embedded (16 x 16 patches, GELU, 2-D adjacent-pair rotary on the two halves of the width, a 2 x 2 strided
convolution that merges four patches into one token), the timestep (and noise-scale) embeddings are added, the
generation path runs over those image tokens attending the cached prompt (the cache is read, never extended), and a
two-layer head predicts the clean 32 x 32 x 3 pixel cell of every token. The velocity is (x_pred - z) / max(1 - t, eps).

Attention splits every head in two: the first half carries the sequence position (theta 5e6), the second half a row
and a column position (theta 1e4, a quarter of the head each), each half with its own RMSNorm; rotation is the
rotate-half form. Tokens with equal sequence position (one image) see each other; otherwise attention is causal.

One implementation for both backends: projections go through nn_dual (tcgen05 GEMM in bf16 on a CUDA device); the
masked attention uses the framework's scaled-dot-product call."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import nn_dual as nd


@dataclass
class NeoLlmConfig:
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 42
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    vocab_size: int = 151936
    rope_theta: float = 5_000_000.0
    rope_theta_hw: float = 10_000.0


@dataclass
class NeoVisionConfig:
    hidden_size: int = 1024
    llm_hidden_size: int = 4096
    patch_size: int = 16
    downsample_ratio: float = 0.5
    rope_theta_vision: float = 10_000.0


@dataclass
class NeoChatConfig:
    tie_word_embeddings: bool = False
    downsample_ratio: float = 0.5
    patch_size: int = 16
    timestep_shift: float = 1.0
    timestep_shift_declared: bool = False
    noise_scale_mode: str = "resolution"
    noise_scale: float = 1.0
    noise_scale_max_value: float = 8.0
    noise_scale_base_image_seq_len: int = 64
    add_noise_scale_embedding: bool = True
    llm: NeoLlmConfig = field(default_factory=NeoLlmConfig)
    vision: NeoVisionConfig = field(default_factory=NeoVisionConfig)

    @staticmethod
    def from_json(j: dict) -> "NeoChatConfig":
        for key in ("llm_config", "vision_config"):
            if not isinstance(j.get(key), dict):
                raise ValueError(f"sensenova: config.json is missing the `{key}` object (corrupt or wrong snapshot); refusing to "
                                 "fall back to 8B defaults for generation-math scalars")
        pick = lambda cls, src: cls(**{k: src[k] for k in cls.__dataclass_fields__ if k in src and not isinstance(src[k], dict)})   # noqa: E731
        c = pick(NeoChatConfig, j)
        c.llm, c.vision = pick(NeoLlmConfig, j["llm_config"]), pick(NeoVisionConfig, j["vision_config"])
        if not c.llm.head_dim:
            c.llm.head_dim = c.llm.hidden_size // c.llm.num_attention_heads
        c.timestep_shift_declared = isinstance(j.get("timestep_shift"), (int, float))
        return c

    def inference_timestep_shift(self, product_default: float) -> float:
        """The checkpoint's own shift when it declares a non-identity one, else the product default."""
        return self.timestep_shift if self.timestep_shift_declared and self.timestep_shift != 1.0 else product_default


def rope_table(positions: torch.Tensor, dim: int, theta: float):
    """cos / sin [S, dim] in the rotate-half layout (frequencies repeated over the two halves)."""
    inv = 1.0 / theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)
    ang = positions.float()[:, None] * inv[None]
    ang = torch.cat([ang, ang], 1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, d]; rotate-half."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * cos[None, :, None].to(x) + rot * sin[None, :, None].to(x)


def block_mask(past: int, temporal: torch.Tensor) -> torch.Tensor:
    """Additive mask [1, 1, q, past + q]: the cached prefix is visible; among the new tokens, equal sequence positions
    (one image) are mutually visible, otherwise causal."""
    q = temporal.numel()
    same = temporal[:, None] == temporal[None, :]
    causal = torch.ones(q, q, dtype=torch.bool).tril()
    allowed = torch.cat([torch.ones(q, past, dtype=torch.bool), same | causal], 1)
    return torch.where(allowed, 0.0, -1e30)[None, None]


def text_indexes(n: int):
    z = torch.zeros(n, dtype=torch.int64)
    return torch.arange(n), z, z.clone()


def image_indexes(token_h: int, token_w: int, text_len: int):
    i = torch.arange(token_h * token_w)
    return torch.full_like(i, text_len), i // token_w, i % token_w


class KvCache:
    def __init__(self, layers: int):
        self.k, self.v, self.len = [None] * layers, [None] * layers, 0


class SenseNovaT2i:
    def __init__(self, cfg: NeoChatConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        if not cfg.noise_scale_max_value > 0:
            raise ValueError(f"sensenova: noise_scale_max_value must be > 0 (got {cfg.noise_scale_max_value})")
        w = dict(weights)
        for p in ("fm_modules.vision_model_mot_gen.embeddings", "vision_model.embeddings"):
            if p + ".patch_embedding.weight" in w and w[p + ".patch_embedding.weight"].dim() == 4:
                w[p + ".patch_embedding.weight"] = w[p + ".patch_embedding.weight"].flatten(1)
        self.w = nd.WeightBag(w, dtype, self.device)
        self.merge = round(1.0 / cfg.downsample_ratio)

    @property
    def cell(self) -> int:
        return self.cfg.patch_size * self.merge

    # ---- decoder --------------------------------------------------------------------------------------------------------
    def _rms(self, x, name):
        return nd.rms_norm(x, self.w[name], self.cfg.llm.rms_norm_eps)

    def _qk(self, x, heads, p, s, tables):
        hd = self.cfg.llm.head_dim
        B, S, _ = x.shape
        x = x.view(B, S, heads, hd)
        t = self._rms(x[..., :hd // 2].contiguous(), f"{p}_norm{s}.weight")
        hw = self._rms(x[..., hd // 2:].contiguous(), f"{p}_norm_hw{s}.weight")
        (ct, st), (ch, sh), (cw, sw) = tables
        return torch.cat([apply_rope(t, ct, st), apply_rope(hw[..., :hd // 4], ch, sh), apply_rope(hw[..., hd // 4:], cw, sw)], -1)

    def prepare(self, temporal, height, width, past: int):
        """Rotary tables and the mask for a chunk of tokens at (sequence, row, column) positions behind `past` cached ones."""
        hd, c = self.cfg.llm.head_dim, self.cfg.llm
        tables = (rope_table(temporal, hd // 2, c.rope_theta), rope_table(height, hd // 4, c.rope_theta_hw),
                  rope_table(width, hd // 4, c.rope_theta_hw))
        tables = tuple((a.to(self.device), b.to(self.device)) for a, b in tables)
        return tables, block_mask(past, temporal).to(self.device), temporal.numel()

    @torch.no_grad()
    def forward_chunk(self, embeds, prep, gen_path: bool, cache: KvCache, append: bool) -> torch.Tensor:
        """Run one chunk on the understanding (gen_path False) or generation path against the cache; `append` extends it."""
        c, w = self.cfg.llm, self.w
        tables, mask, n = prep
        s = "_mot_gen" if gen_path else ""
        H, K, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        x = embeds.to(self.device, self.dtype)
        B, S, _ = x.shape
        for i in range(c.num_hidden_layers):
            p = f"language_model.model.layers.{i}"
            a = p + ".self_attn"
            h = self._rms(x, f"{p}.input_layernorm{s}.weight")
            q = self._qk(w.lin(h, f"{a}.q_proj{s}"), H, a + ".q", s, tables)
            k = self._qk(w.lin(h, f"{a}.k_proj{s}"), K, a + ".k", s, tables)
            v = w.lin(h, f"{a}.v_proj{s}").view(B, S, K, hd)
            if cache.k[i] is not None:
                k_all, v_all = torch.cat([cache.k[i], k], 1), torch.cat([cache.v[i], v], 1)
            else:
                k_all, v_all = k, v
            if append:
                cache.k[i], cache.v[i] = k_all, v_all
            o = nd.attention(q, k_all, v_all, mask=mask.to(q.dtype))
            x = x + w.lin(o, f"{a}.o_proj{s}")
            h = self._rms(x, f"{p}.post_attention_layernorm{s}.weight")
            m = p + (".mlp_mot_gen" if gen_path else ".mlp")
            x = x + w.lin((F.silu(w.lin(h, m + ".gate_proj").float()) * w.lin(h, m + ".up_proj").float()).to(self.dtype), m + ".down_proj")
        if append:
            cache.len += n
        return self._rms(x, "language_model.model.norm_mot_gen.weight" if gen_path else "language_model.model.norm.weight")

    def prefill(self, ids: list[int]) -> tuple[KvCache, int]:
        cache = KvCache(self.cfg.llm.num_hidden_layers)
        emb = self.w["language_model.model.embed_tokens.weight"][torch.tensor(ids, device=self.device)][None]
        self.forward_chunk(emb, self.prepare(*text_indexes(len(ids)), 0), False, cache, True)
        return cache, len(ids)

    # ---- image side -------------------------------------------------------------------------------------------------------
    def vision_embed(self, patches: torch.Tensor, grid_h: int, grid_w: int, prefix: str = "fm_modules.vision_model_mot_gen.embeddings"):
        """[grid_h * grid_w, 3 * p * p] channel-first patches -> [grid_h / m * grid_w / m, llm hidden]."""
        w, theta = self.w, self.cfg.vision.rope_theta_vision
        pe = w.lin(patches.to(self.device, self.dtype), prefix + ".patch_embedding", act="gelu").float()
        E = pe.shape[1]
        idx = torch.arange(grid_h * grid_w)

        def rope1d(x, pos):
            part = x.shape[1]
            inv = 1.0 / theta ** (torch.arange(0, part, 2, dtype=torch.float32) / part)
            ang = (pos.float()[:, None] * inv[None]).to(x.device)
            a, b = x[:, 0::2], x[:, 1::2]
            return torch.stack([a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()], -1).reshape(x.shape)

        r = torch.cat([rope1d(pe[:, :E // 2], idx % grid_w), rope1d(pe[:, E // 2:], idx // grid_w)], 1)
        block = r.view(grid_h, grid_w, E).permute(2, 0, 1)[None]
        dw = w[prefix + ".dense_embedding.weight"]
        out = F.conv2d(block.to(dw.dtype), dw, w[prefix + ".dense_embedding.bias"], stride=self.merge)
        return out[0].permute(1, 2, 0).reshape(-1, out.shape[1])

    def _timestep_embed(self, t: torch.Tensor, prefix: str) -> torch.Tensor:
        freq = nd.sinusoidal_embedding(t.to(self.device), 256).to(self.dtype)
        return self.w.lin(self.w.lin(freq, prefix + ".mlp.0", act="silu"), prefix + ".mlp.2")

    def noise_scale_for(self, grid_h: int, grid_w: int) -> float:
        c = self.cfg
        scale = c.noise_scale
        if c.noise_scale_mode in ("resolution", "dynamic", "dynamic_sqrt"):
            seq = grid_h * grid_w / (self.merge * self.merge)
            scale = math.sqrt(seq / c.noise_scale_base_image_seq_len) * c.noise_scale
            if c.noise_scale_mode == "dynamic_sqrt":
                scale = math.sqrt(scale)
        return min(scale, c.noise_scale_max_value)

    def step_tokens(self, image: torch.Tensor, t: float, noise_embed):
        """image [1, 3, H, W] -> (z [1, L, cell * cell * 3] in (row, column, channel) order, conditioning tokens [1, L, hidden])."""
        ps = self.cfg.patch_size
        _, _, H, W = image.shape
        gh, gw = H // ps, W // ps
        z = patchify(image, self.cell)
        vis = self.vision_embed(patchify_channel_first(image, ps)[0], gh, gw)
        L = vis.shape[0]
        cond = vis.to(self.dtype) + self._timestep_embed(torch.full((L,), float(t)), "fm_modules.timestep_embedder")
        if noise_embed is not None:
            cond = cond + noise_embed
        return z, cond[None]

    def noise_scale_embed(self, noise_scale: float, L: int):
        if not self.cfg.add_noise_scale_embedding:
            return None
        return self._timestep_embed(torch.full((L,), noise_scale / self.cfg.noise_scale_max_value), "fm_modules.noise_scale_embedder")

    def predict_v(self, cond, prep, cache: KvCache, z: torch.Tensor, t: float, t_eps: float) -> torch.Tensor:
        hidden = self.forward_chunk(cond, prep, True, cache, False)
        x_pred = self.w.lin(self.w.lin(hidden, "fm_modules.fm_head.0", act="gelu"), "fm_modules.fm_head.2").float()
        return (x_pred - z.to(x_pred.device)) / max(1.0 - t, t_eps)


def patchify(img: torch.Tensor, p: int) -> torch.Tensor:
    n, _, H, W = img.shape
    return img.reshape(n, 3, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(n, (H // p) * (W // p), p * p * 3)


def patchify_channel_first(img: torch.Tensor, p: int) -> torch.Tensor:
    n, _, H, W = img.shape
    return img.reshape(n, 3, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(n, (H // p) * (W // p), 3 * p * p)


def unpatchify(x: torch.Tensor, p: int, h: int, w: int) -> torch.Tensor:
    n = x.shape[0]
    return x.reshape(n, h, w, p, p, 3).permute(0, 5, 1, 3, 2, 4).reshape(n, 3, h * p, w * p)


def time_schedule(steps: int, shift: float, enable: bool = True) -> list[float]:
    """steps + 1 times from 0 (noise) to 1 (data); the shift acts on sigma = 1 - t."""
    if steps < 1:
        raise ValueError("sensenova: num_steps must be >= 1")
    out = []
    for i in range(steps + 1):
        t = i / steps
        if enable:
            s = 1.0 - t
            t = 1.0 - shift * s / (1.0 + (shift - 1.0) * s)
        out.append(t)
    return out


def merge_distill_lora(weights: dict[str, torch.Tensor], lora: dict[str, torch.Tensor], layers: int) -> int:
    """Folds `<target>.lora_down / lora_up / alpha` into the generation path's projections and the flow head; returns the
    number of merged targets."""
    targets = ["fm_modules.fm_head.0", "fm_modules.fm_head.2"]
    for i in range(layers):
        p = f"language_model.model.layers.{i}"
        targets += [f"{p}.self_attn.{n}_proj_mot_gen" for n in "qkvo"] + [f"{p}.mlp_mot_gen.{n}_proj" for n in ("gate", "up", "down")]
    n = 0
    for t in targets:
        if t + ".lora_down.weight" not in lora:
            continue
        down, up = lora[t + ".lora_down.weight"].float(), lora[t + ".lora_up.weight"].float()
        if down.shape[0] == 0:
            raise ValueError(f"distill LoRA: zero-rank factor at '{t}'")
        alpha = float(lora[t + ".alpha"].float().reshape(-1)[0])
        wt = weights[t + ".weight"]
        weights[t + ".weight"] = (wt.float() + (up @ down) * (alpha / down.shape[0])).to(wt.dtype)
        n += 1
    return n


def random_sensenova_weights(cfg: NeoChatConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    c, v = cfg.llm, cfg.vision
    D, hd = c.hidden_size, c.head_dim
    w["language_model.model.embed_tokens.weight"] = rn(c.vocab_size, D) * 0.1
    lin(w, "language_model.lm_head", c.vocab_size, D, bias=False)
    for s in ("", "_mot_gen"):
        w[f"language_model.model.norm{s}.weight"] = 1 + rn(D) * 0.05
    for i in range(c.num_hidden_layers):
        p = f"language_model.model.layers.{i}"
        for s in ("", "_mot_gen"):
            w[f"{p}.input_layernorm{s}.weight"], w[f"{p}.post_attention_layernorm{s}.weight"] = 1 + rn(D) * 0.05, 1 + rn(D) * 0.05
            lin(w, f"{p}.self_attn.q_proj{s}", c.num_attention_heads * hd, D, bias=False)
            lin(w, f"{p}.self_attn.k_proj{s}", c.num_key_value_heads * hd, D, bias=False)
            lin(w, f"{p}.self_attn.v_proj{s}", c.num_key_value_heads * hd, D, bias=False)
            lin(w, f"{p}.self_attn.o_proj{s}", D, c.num_attention_heads * hd, bias=False)
            for n, d in (("q_norm", hd // 2), ("k_norm", hd // 2), ("q_norm_hw", hd // 2), ("k_norm_hw", hd // 2)):
                w[f"{p}.self_attn.{n}{s}.weight"] = 1 + rn(d) * 0.05
        for m in (".mlp", ".mlp_mot_gen"):
            lin(w, p + m + ".gate_proj", c.intermediate_size, D, bias=False)
            lin(w, p + m + ".up_proj", c.intermediate_size, D, bias=False)
            lin(w, p + m + ".down_proj", D, c.intermediate_size, bias=False)
    m = round(1.0 / cfg.downsample_ratio)
    for pre in ("fm_modules.vision_model_mot_gen.embeddings",):
        w[pre + ".patch_embedding.weight"], w[pre + ".patch_embedding.bias"] = rn(v.hidden_size, 3, v.patch_size, v.patch_size) * 0.05, rn(v.hidden_size) * 0.02
        w[pre + ".dense_embedding.weight"], w[pre + ".dense_embedding.bias"] = rn(D, v.hidden_size, m, m) * 0.05, rn(D) * 0.02
    cell = cfg.patch_size * m
    lin(w, "fm_modules.fm_head.0", D, D)
    lin(w, "fm_modules.fm_head.2", cell * cell * 3, D)
    for e in ("timestep_embedder", "noise_scale_embedder"):
        lin(w, f"fm_modules.{e}.mlp.0", D, 256)
        lin(w, f"fm_modules.{e}.mlp.2", D, D)
    return w
