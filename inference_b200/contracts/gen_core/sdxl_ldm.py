"""Key remapping for single-file SDXL checkpoints in the original latent-diffusion layout
(gen-core/src/sdxl_ldm.rs): each tensor key maps to a component (UNet, CLIP-L, OpenCLIP bigG, VAE) and a
diffusers-style key, possibly with a tensor operation (split a fused QKV into three, transpose the text projection,
squeeze the VAE attention's 1x1 convolutions to linear weights)."""
from __future__ import annotations

import enum
from dataclasses import dataclass


class SdxlComponent(enum.Enum):
    UNET = "unet"
    CLIP_L = "clip_l"
    CLIP_BIG_G = "clip_big_g"
    VAE = "vae"


@dataclass(frozen=True)
class TensorRemap:
    op: str                      # "rename" | "split_qkv" | "transpose" | "squeeze"
    component: SdxlComponent
    keys: tuple[str, ...]        # one key, or (q, k, v) for split_qkv

    @property
    def key(self) -> str:
        return self.keys[0]


def _index_after(key: str, prefix: str) -> int | None:
    if not key.startswith(prefix):
        return None
    head = key[len(prefix):].split(".", 1)[0]
    return int(head) if head.isdigit() else None


def _resnet(key: str) -> str:
    for a, b in (("in_layers.0", "norm1"), ("in_layers.2", "conv1"), ("out_layers.0", "norm2"),
                 ("out_layers.3", "conv2"), ("emb_layers.1", "time_emb_proj"), ("skip_connection", "conv_shortcut")):
        key = key.replace(a, b)
    return key


def _unet(key: str) -> str | None:
    for a, b in (("time_embed.0.", "time_embedding.linear_1."), ("time_embed.2.", "time_embedding.linear_2."),
                 ("input_blocks.0.0.", "conv_in."), ("out.0.", "conv_norm_out."), ("out.2.", "conv_out."),
                 ("label_emb.0.0.", "add_embedding.linear_1."), ("label_emb.0.2.", "add_embedding.linear_2.")):
        if key.startswith(a):
            return b + key[len(a):]
    i = _index_after(key, "input_blocks.")
    if i is not None:
        if i == 0:
            return None
        block, layer = (i - 1) // 3, (i - 1) % 3
        p = f"input_blocks.{i}."
        if key.startswith(p + "0.op."):
            return f"down_blocks.{block}.downsamplers.0.conv.{key[len(p) + 5:]}"
        if key.startswith(p + "0."):
            return _resnet(f"down_blocks.{block}.resnets.{layer}.{key[len(p) + 2:]}")
        if key.startswith(p + "1."):
            return f"down_blocks.{block}.attentions.{layer}.{key[len(p) + 2:]}"
    i = _index_after(key, "middle_block.")
    if i is not None:
        rest = key[len(f"middle_block.{i}."):]
        return _resnet(f"mid_block.resnets.{max(i - 1, 0)}.{rest}") if i % 2 == 0 else \
            f"mid_block.attentions.{i - 1}.{rest}"
    i = _index_after(key, "output_blocks.")
    if i is not None:
        block, layer = i // 3, i % 3
        p = f"output_blocks.{i}."
        if key.startswith(p + "0."):
            return _resnet(f"up_blocks.{block}.resnets.{layer}.{key[len(p) + 2:]}")
        for slot in (1, 2):
            q = f"{p}{slot}.conv."
            if key.startswith(q):
                return f"up_blocks.{block}.upsamplers.0.conv.{key[len(q):]}"
        if key.startswith(p + "1."):
            return f"up_blocks.{block}.attentions.{layer}.{key[len(p) + 2:]}"
    return None


def _vae_attn(key: str) -> str:
    for a, b in ((".norm.", ".group_norm."), (".q.", ".to_q."), (".k.", ".to_k."), (".v.", ".to_v."),
                 (".proj_out.", ".to_out.0.")):
        key = key.replace(a, b)
    return key


def _vae(key: str) -> str | None:
    for a, b in (("encoder.conv_in.", "encoder.conv_in."), ("encoder.conv_out.", "encoder.conv_out."),
                 ("encoder.norm_out.", "encoder.conv_norm_out."), ("decoder.conv_in.", "decoder.conv_in."),
                 ("decoder.conv_out.", "decoder.conv_out."), ("decoder.norm_out.", "decoder.conv_norm_out."),
                 ("quant_conv.", "quant_conv."), ("post_quant_conv.", "post_quant_conv.")):
        if key.startswith(a):
            return b + key[len(a):]
    for side in ("encoder", "decoder"):
        for block in (1, 2):
            p = f"{side}.mid.block_{block}."
            if key.startswith(p):
                return f"{side}.mid_block.resnets.{block - 1}.{key[len(p):]}".replace("nin_shortcut", "conv_shortcut")
        p = f"{side}.mid.attn_1."
        if key.startswith(p):
            return _vae_attn(f"{side}.mid_block.attentions.0.{key[len(p):]}")
    i = _index_after(key, "encoder.down.")
    if i is not None:
        p = f"encoder.down.{i}."
        if key.startswith(p + "downsample.conv."):
            return f"encoder.down_blocks.{i}.downsamplers.0.conv.{key[len(p) + 16:]}"
        if key.startswith(p + "block."):
            return f"encoder.down_blocks.{i}.resnets.{key[len(p) + 6:]}".replace("nin_shortcut", "conv_shortcut")
    i = _index_after(key, "decoder.up.")
    if i is not None and i <= 3:
        target = 3 - i                      # the original layout counts decoder levels from the output side
        p = f"decoder.up.{i}."
        if key.startswith(p + "upsample.conv."):
            return f"decoder.up_blocks.{target}.upsamplers.0.conv.{key[len(p) + 14:]}"
        if key.startswith(p + "block."):
            return f"decoder.up_blocks.{target}.resnets.{key[len(p) + 6:]}".replace("nin_shortcut", "conv_shortcut")
    return None


def _openclip(key: str) -> str | None:
    fixed = {"positional_embedding": "text_model.embeddings.position_embedding.weight",
             "token_embedding.weight": "text_model.embeddings.token_embedding.weight",
             "ln_final.weight": "text_model.final_layer_norm.weight", "ln_final.bias": "text_model.final_layer_norm.bias"}
    if key in fixed:
        return fixed[key]
    if not key.startswith("transformer."):
        return None
    rest = key[len("transformer."):]
    for a, b in (("resblocks.", "text_model.encoder.layers."), ("ln_1", "layer_norm1"), ("ln_2", "layer_norm2"),
                 (".mlp.c_fc.", ".mlp.fc1."), (".mlp.c_proj.", ".mlp.fc2."), (".attn", ".self_attn")):
        rest = rest.replace(a, b)
    return rest


def remap_sdxl_ldm_key(key: str) -> TensorRemap | None:
    C = SdxlComponent
    if key.startswith("model.diffusion_model."):
        k = _unet(key[len("model.diffusion_model."):])
        return TensorRemap("rename", C.UNET, (k,)) if k else None
    p = "conditioner.embedders.0.transformer."
    if key.startswith(p):
        return TensorRemap("rename", C.CLIP_L, (key[len(p):],))
    p = "conditioner.embedders.1.model."
    if key.startswith(p):
        inner = key[len(p):]
        if inner == "text_projection":
            return TensorRemap("transpose", C.CLIP_BIG_G, ("text_projection.weight",))
        for suffix in (".in_proj_weight", ".in_proj_bias"):
            if inner.endswith(suffix):
                base = _openclip(inner[: -len(suffix)])
                if base is None:
                    return None
                leaf = "weight" if suffix.endswith("weight") else "bias"
                return TensorRemap("split_qkv", C.CLIP_BIG_G, tuple(f"{base}.{n}_proj.{leaf}" for n in "qkv"))
        k = _openclip(inner)
        return TensorRemap("rename", C.CLIP_BIG_G, (k,)) if k else None
    if key.startswith("first_stage_model."):
        k = _vae(key[len("first_stage_model."):])
        if k is None:
            return None
        return TensorRemap("squeeze" if ".attentions." in k and k.endswith(".weight") else "rename", C.VAE, (k,))
    return None


def apply_remap(tensors: dict) -> dict[SdxlComponent, dict]:
    """Splits a single-file checkpoint into per-component dictionaries with diffusers keys (torch tensors)."""
    out = {c: {} for c in SdxlComponent}
    for key, t in tensors.items():
        r = remap_sdxl_ldm_key(key)
        if r is None:
            continue
        d = out[r.component]
        if r.op == "rename":
            d[r.key] = t
        elif r.op == "transpose":
            d[r.key] = t.t().contiguous()
        elif r.op == "squeeze":
            d[r.key] = t.reshape(t.shape[0], t.shape[1]) if t.dim() == 4 else t
        else:
            n = t.shape[0] // 3
            for i, k in enumerate(r.keys):
                d[k] = t[i * n:(i + 1) * n].contiguous()
    return out
