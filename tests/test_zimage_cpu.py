"""Z-Image DiT oracle against an independent restatement (complex-number RoPE, explicit softmax attention, padded
caption with a key mask), plus the token-layout helpers."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_zimage as Z

CFG = Z.ZImageConfig(dim=48, n_layers=2, n_refiner_layers=1, n_heads=3, in_channels=4, cap_feat_dim=20,
                     axes_dims=(4, 6, 6))


def _rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def _direct(w, cfg, z, t, cap, pad_to):
    """One sample; the caption is zero-padded to `pad_to` rows and masked as attention keys, as the padded pipeline
    does it; image positions start one past the padded length."""
    D, nh, hd = cfg.dim, cfg.n_heads, cfg.head_dim
    L = cap.shape[0]
    capp = torch.cat([cap, torch.zeros(pad_to - L, cap.shape[1])], 0)
    keep = torch.arange(pad_to) < L

    def freqs(ids):
        out = []
        for a, d in enumerate(cfg.axes_dims):
            inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2).double() / d))
            out.append(torch.polar(torch.ones(ids.shape[0], d // 2, dtype=torch.float64), ids[:, a:a + 1].double() * inv))
        return torch.cat(out, -1)

    def rope(x, fr):                                  # x [S, nh, hd]
        xc = torch.view_as_complex(x.double().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * fr[:, None, :]).flatten(-2).float()

    def attn(x, p, fr, mask):
        S = x.shape[0]
        q, k, v = (x @ w[f"{p}.attention.{n}.weight"].t() for n in ("to_q", "to_k", "to_v"))
        q = rope(_rms(q.view(S, nh, hd), w[f"{p}.attention.norm_q.weight"], 1e-5), fr)
        k = rope(_rms(k.view(S, nh, hd), w[f"{p}.attention.norm_k.weight"], 1e-5), fr)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        s = s.masked_fill(~mask[None, None, :], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v.view(S, nh, hd)).reshape(S, D)
        return o @ w[f"{p}.attention.to_out.0.weight"].t()

    def block(x, p, fr, mask, ada):
        if ada is not None:
            m = ada @ w[f"{p}.adaLN_modulation.0.weight"].t() + w[f"{p}.adaLN_modulation.0.bias"]
            sa, ga, sm, gm = m.chunk(4)
            sa, sm, ga, gm = 1 + sa, 1 + sm, torch.tanh(ga), torch.tanh(gm)
        else:
            sa = sm = ga = gm = torch.ones(D)
        a = attn(_rms(x, w[f"{p}.attention_norm1.weight"], cfg.norm_eps) * sa, p, fr, mask)
        x = x + ga * _rms(a, w[f"{p}.attention_norm2.weight"], cfg.norm_eps)
        h = _rms(x, w[f"{p}.ffn_norm1.weight"], cfg.norm_eps) * sm
        f = (F.silu(h @ w[f"{p}.feed_forward.w1.weight"].t()) * (h @ w[f"{p}.feed_forward.w3.weight"].t())) \
            @ w[f"{p}.feed_forward.w2.weight"].t()
        return x + gm * _rms(f, w[f"{p}.ffn_norm2.weight"], cfg.norm_eps)

    C, H, W = z.shape
    ht, wt = H // 2, W // 2
    half = 128
    fq = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    te = torch.cat([torch.cos(t * 1000.0 * fq), torch.sin(t * 1000.0 * fq)])
    ada = F.silu(te @ w["t_embedder.mlp.0.weight"].t() + w["t_embedder.mlp.0.bias"]) @ w["t_embedder.mlp.2.weight"].t() \
        + w["t_embedder.mlp.2.bias"]
    patches = torch.stack([torch.stack([z[:, 2 * i + a, 2 * j + b] for a in range(2) for b in range(2)], 0).reshape(-1)
                           for i in range(ht) for j in range(wt)], 0)          # (a, b, c) with c fastest
    x = patches @ w["all_x_embedder.2-1.weight"].t() + w["all_x_embedder.2-1.bias"]
    img_ids = torch.tensor([[pad_to + 1, i, j] for i in range(ht) for j in range(wt)], dtype=torch.float64)
    cap_ids = torch.tensor([[1 + i, 0, 0] for i in range(pad_to)], dtype=torch.float64)
    c = _rms(capp, w["cap_embedder.0.weight"], cfg.norm_eps) @ w["cap_embedder.1.weight"].t() + w["cap_embedder.1.bias"]
    for i in range(cfg.n_refiner_layers):
        x = block(x, f"noise_refiner.{i}", freqs(img_ids), torch.ones(x.shape[0], dtype=torch.bool), ada)
        c = block(c, f"context_refiner.{i}", freqs(cap_ids), keep, None)
    u = torch.cat([x, c], 0)
    fr = freqs(torch.cat([img_ids, cap_ids], 0))
    mask = torch.cat([torch.ones(x.shape[0], dtype=torch.bool), keep])
    for i in range(cfg.n_layers):
        u = block(u, f"layers.{i}", fr, mask, ada)
    sc = 1 + F.silu(ada) @ w["all_final_layer.2-1.adaLN_modulation.1.weight"].t() + w["all_final_layer.2-1.adaLN_modulation.1.bias"]
    o = (F.layer_norm(u[: x.shape[0]], (D,), eps=1e-6) * sc) @ w["all_final_layer.2-1.linear.weight"].t() \
        + w["all_final_layer.2-1.linear.bias"]
    out = torch.zeros(C, H, W)
    for n, (i, j) in enumerate((i, j) for i in range(ht) for j in range(wt)):
        out[:, 2 * i:2 * i + 2, 2 * j:2 * j + 2] = o[n].view(2, 2, C).permute(2, 0, 1)
    return out


def test_oracle_matches_direct_restatement():
    w = Z.random_zimage_weights(CFG, seed=1, std=0.15)
    g = torch.Generator().manual_seed(2)
    z = torch.randn(1, 4, 6, 8, generator=g)
    cap = torch.randn(1, 37, 20, generator=g)
    t = torch.tensor([0.35])
    out = Z.OracleZImageDiT(CFG, w).forward(z, t, cap)
    ref = _direct(w, CFG, z[0], t[0], cap[0], pad_to=64)
    assert out.shape == z.shape and ref.abs().max() > 0.05
    assert (out[0] - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_token_layout_helpers():
    z = torch.arange(2 * 4 * 6 * 8, dtype=torch.float32).view(2, 4, 6, 8)
    p = Z.patchify(z)
    assert p.shape == (2, 12, 16)
    assert torch.equal(p[0, 5].view(2, 2, 4)[1, 0], z[0, :, 2 * 1 + 1, 2 * 1 + 0])          # token 5 = (row 1, column 1)
    assert torch.equal(Z.unpatchify(p, 6, 8), z)
    img, cap = Z.position_ids(3, 4, 33)
    assert cap[:, 0].tolist() == list(range(1, 34)) and cap[:, 1:].abs().sum() == 0
    assert img[:, 0].unique().tolist() == [65.0] and img[5].tolist() == [65.0, 1.0, 1.0]
    assert Z.ZImageConfig().ffn_dim == 10240 and Z.ZImageConfig().head_dim == 128


# ---- providers ---------------------------------------------------------------------------------------------------------------
def test_sigma_tables():
    from inference_b200.media.z_image import ZImageVariant, z_image_sigmas

    t = z_image_sigmas(ZImageVariant.TURBO, 4)
    lo = 3.0 * 0.001 / 1.002
    assert len(t) == 5 and t[0] == 1.0 and t[-1] == 0.0 and abs(t[3] - lo) < 1e-12
    assert abs((t[0] - t[1]) - (t[1] - t[2])) < 1e-12                       # a linear ramp: conditioning 1 - sigma matches it
    b = z_image_sigmas(ZImageVariant.BASE, 50)
    assert len(b) == 51 and b[0] == 1.0 and b[-1] == 0.0 and all(x > y for x, y in zip(b, b[1:]))
    lin = [1.0 + (6.0 * 0.001 / 1.005 - 1.0) * i / 49 for i in range(50)]
    assert all(bs > ls for bs, ls in zip(b[1:50], lin[1:]))                 # the static shift lifts every interior value


def test_z_image_providers_conform(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.z_image import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "zi", text="qwen3")
    reg = provider_registry("cpu")
    assert [i for i in reg.ids() if "z_image" in i] == ["cpu_z_image", "cpu_z_image_turbo"]
    assert reg.descriptor_conformance_errors() == []
    turbo = reg.load("cpu_z_image_turbo", LoadSpec.from_dir(snap))
    kit.conformance(turbo, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_z_image_turbo", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    with pytest.raises(InferenceError):
        turbo.generate(GenerationRequest(**req, negative_prompt="blurry"))     # distilled: no negative prompt
    base = reg.load("cpu_z_image", LoadSpec.from_dir(snap))
    a = base.generate(GenerationRequest(**req, guidance=1.0)).images[0].pixels
    b = base.generate(GenerationRequest(**req)).images[0].pixels                # default guidance 4, empty negative
    c = base.generate(GenerationRequest(**req, guidance=4.0, negative_prompt="")).images[0].pixels
    d = base.generate(GenerationRequest(**req, sampler="heun", scheduler="simple")).images[0].pixels
    assert b == c and a != b and d != b and len(a) == 256 * 256 * 3


# ---- trainer and adapters ----------------------------------------------------------------------------------------------------
def test_z_image_trainer_and_adapter_round_trip(tmp_path):
    from inference_b200.contracts.gen_core import (AdapterKind, AdapterSpec, GenerationRequest, LoadSpec, TrainingConfig,
                                                   WeightsSource)
    from inference_b200.io.safetensors_io import load_file, save_file
    from inference_b200.media import provider_registry
    from inference_b200.media.train import Z_IMAGE_TARGETS, merge_lora
    from inference_b200.media.z_image import write_synthetic_snapshot
    from inference_b200.testkit.aux_suites import TrainerProfile, trainer_conformance

    snap = write_synthetic_snapshot(tmp_path / "zi")
    ds = tmp_path / "ds"
    ds.mkdir()
    g = torch.Generator().manual_seed(0)
    for i in range(2):
        save_file({"latent": torch.randn(16, 8, 8, generator=g), "txt": torch.randn(9, 64, generator=g)},
                  ds / f"item{i}.safetensors")
    reg = provider_registry("cpu")
    tr = reg.load_kind("trainer", "cpu_z_image_lora_trainer", LoadSpec.from_dir(snap))
    assert tr.descriptor().id == "cpu_z_image_lora_trainer"
    items = tr._items(ds)
    noise = torch.randn(16, 8, 8, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    cfg = TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "run", steps=10, learning_rate=5e-3, rank=4, alpha=4.0, seed=3)
    final = tr.train(cfg, lambda p: None)
    ad = load_file(final)
    assert all(k.split(".lora_")[0].endswith(Z_IMAGE_TARGETS) for k in ad) and len(ad) == 2 * 4 * 4     # 4 blocks x 4 targets
    base_w = {k: v.float() for k, v in load_file(snap / "transformer" / "diffusion_pytorch_model.safetensors").items()}
    tr.model.w.update({k: v for k, v in merge_lora(base_w, ad).items() if k in tr.model.w})
    assert float(tr.loss_on(items[0], 0.5, noise)) < before
    # the generator merges the same file at load
    req = lambda: GenerationRequest(prompt="a fox", width=256, height=256, steps=1, seed=2)      # noqa: E731
    big = {k: v * (30.0 if "lora_B" in k else 1.0) for k, v in ad.items()}
    save_file(big, tmp_path / "big.safetensors")

    def run(scale):
        spec = LoadSpec(weights=WeightsSource.dir(snap),
                        adapters=[] if scale is None else [AdapterSpec(path=tmp_path / "big.safetensors", scale=scale,
                                                                       kind=AdapterKind.LORA)])
        return reg.load("cpu_z_image_turbo", spec).generate(req(), lambda e: None).images[0].pixels
    plain = run(None)
    assert run(0.0) == plain and run(1.0) != plain
    trainer_conformance(reg.load_kind("trainer", "cpu_z_image_lora_trainer", LoadSpec.from_dir(snap)),
                        TrainerProfile(ds, tmp_path / "out", steps=3, rank=2))


def test_reference_guided_generation(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media import provider_registry
    from inference_b200.media.chroma import convert_diffusers_vae_encoder
    from inference_b200.media.z_image import init_time_step, native_vae_encoder_to_diffusers, write_synthetic_snapshot
    from inference_b200.models.vae import VaeConfig, random_vae_encoder_weights

    assert [init_time_step(28, s) for s in (None, 0.0, -1.0, 0.5, 0.01, 1.0)] == [0, 0, 0, 14, 1, 27]
    cfg = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    native = random_vae_encoder_weights(cfg, 1)
    back = convert_diffusers_vae_encoder(native_vae_encoder_to_diffusers(native))
    assert back.keys() == native.keys() and all(torch.equal(back[k], native[k]) for k in native)
    snap = write_synthetic_snapshot(tmp_path / "zi")
    gen = provider_registry("cpu").load("cpu_z_image_turbo", LoadSpec.from_dir(snap))
    g = torch.Generator().manual_seed(3)
    ref = Image(width=200, height=120, pixels=bytes(torch.randint(0, 256, (120 * 200 * 3,), generator=g, dtype=torch.uint8).tolist()))
    base = dict(prompt="a red fox", width=256, height=256, steps=4, seed=5)
    events = []
    plain = gen.generate(GenerationRequest(**base)).images[0].pixels
    guided = gen.generate(GenerationRequest(**base, conditioning=[Conditioning(ConditioningKind.REFERENCE, image=ref, strength=0.5)]),
                          events.append).images[0].pixels
    again = gen.generate(GenerationRequest(**base, conditioning=[Conditioning(ConditioningKind.REFERENCE, image=ref, strength=0.5)])
                         ).images[0].pixels
    zero = gen.generate(GenerationRequest(**base, conditioning=[Conditioning(ConditioningKind.REFERENCE, image=ref, strength=0.0)])
                        ).images[0].pixels
    assert guided == again and guided != plain and zero == plain
    steps = [e.current for e in events if hasattr(e, "current")]
    assert steps == [1, 2, 3, 4]                     # the skipped head of the schedule is still reported
