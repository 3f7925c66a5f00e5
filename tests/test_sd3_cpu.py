"""SD3.5 MMDiT against an independent restatement (strided-convolution patch embedding, per-head loops, einsum
unpatchify), for a Large-style and a Medium-style (dual attention) configuration."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.models import dit_sd3 as S


def _direct(w, cfg, z, timestep, ctx, pooled):
    D, nh, hd = cfg.dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda x, n: x @ w[n + ".weight"].t() + w[n + ".bias"]       # noqa: E731
    ln = lambda x: F.layer_norm(x, (D,), eps=1e-6)                       # noqa: E731

    def rms(x, key):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w[key] if key in w else x

    def attend(qs, ks, vs):                     # lists of ([S_i, D], norm key)
        q = torch.cat([rms(x.view(-1, nh, hd), k) for x, k in qs], 0)
        k = torch.cat([rms(x.view(-1, nh, hd), kk) for x, kk in ks], 0)
        v = torch.cat([x.view(-1, nh, hd) for x in vs], 0)
        out = torch.zeros(q.shape[0], nh, hd)
        for h in range(nh):
            s = (q[:, h] @ k[:, h].t()) / math.sqrt(hd)
            out[:, h] = s.softmax(-1) @ v[:, h]
        return out.reshape(-1, D)

    def ff(x, p):
        return lin(F.gelu(lin(x, p + ".net.0.proj"), approximate="tanh"), p + ".net.2")

    C, H, W = z.shape
    h, ww = H // 2, W // 2
    x = F.conv2d(z[None], w["pos_embed.proj.weight"], w["pos_embed.proj.bias"], stride=2)[0].flatten(1).t()
    m = cfg.pos_embed_max_size
    pe = w["pos_embed.pos_embed"].view(m, m, D)
    x = x + pe[(m - h) // 2:(m - h) // 2 + h, (m - ww) // 2:(m - ww) // 2 + ww].reshape(-1, D)
    half = 128
    fr = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half) * timestep
    te = torch.cat([fr.cos(), fr.sin()])
    t = "time_text_embed."
    vec = lin(F.silu(lin(te, t + "timestep_embedder.linear_1")), t + "timestep_embedder.linear_2") \
        + lin(F.silu(lin(pooled, t + "text_embedder.linear_1")), t + "text_embedder.linear_2")
    sv = F.silu(vec)
    c = lin(ctx, "context_embedder")
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        last, dual = i == cfg.num_layers - 1, i in cfg.dual_attention_layers
        mm = lin(sv, p + ".norm1.linear").chunk(9 if dual else 6)
        hx = ln(x) * (1 + mm[1]) + mm[0]
        if last:
            sc, sh = lin(sv, p + ".norm1_context.linear").chunk(2)
            hc = ln(c) * (1 + sc) + sh
        else:
            mc = lin(sv, p + ".norm1_context.linear").chunk(6)
            hc = ln(c) * (1 + mc[1]) + mc[0]
        a = p + ".attn."
        o = attend([(lin(hx, a + "to_q"), a + "norm_q.weight"), (lin(hc, a + "add_q_proj"), a + "norm_added_q.weight")],
                   [(lin(hx, a + "to_k"), a + "norm_k.weight"), (lin(hc, a + "add_k_proj"), a + "norm_added_k.weight")],
                   [lin(hx, a + "to_v"), lin(hc, a + "add_v_proj")])
        n = x.shape[0]
        x_attn = mm[2] * lin(o[:n], a + "to_out.0")
        if dual:
            h2 = ln(x) * (1 + mm[7]) + mm[6]
            a2 = p + ".attn2."
            o2 = attend([(lin(h2, a2 + "to_q"), a2 + "norm_q.weight")], [(lin(h2, a2 + "to_k"), a2 + "norm_k.weight")],
                        [lin(h2, a2 + "to_v")])
            x_attn = x_attn + mm[8] * lin(o2, a2 + "to_out.0")
        x = x + x_attn
        x = x + mm[5] * ff(ln(x) * (1 + mm[4]) + mm[3], p + ".ff")
        if not last:
            c = c + mc[2] * lin(o[n:], a + "to_add_out")
            c = c + mc[5] * ff(ln(c) * (1 + mc[4]) + mc[3], p + ".ff_context")
    sc, sh = lin(sv, "norm_out.linear").chunk(2)
    out = lin(ln(x) * (1 + sc) + sh, "proj_out").view(1, h, ww, 2, 2, C)
    return torch.einsum("nhwpqc->nchpwq", out).reshape(C, H, W)


@pytest.mark.parametrize("dual", [(), (0, 1)])
def test_mmdit_matches_direct_restatement(dual):
    cfg = S.Sd3Config(in_channels=4, pos_embed_max_size=12, num_attention_heads=3, attention_head_dim=8, num_layers=3,
                      joint_attention_dim=20, pooled_projection_dim=10, dual_attention_layers=dual)
    w = S.random_sd3_weights(cfg, seed=1, std=0.15)
    g = torch.Generator().manual_seed(2)
    z = torch.randn(1, 4, 8, 6, generator=g)
    ctx, pooled = torch.randn(1, 7, 20, generator=g), torch.randn(1, 10, generator=g)
    t = torch.tensor([430.0])
    out = S.Sd3DiT(cfg, w).forward(z, t, ctx, pooled)
    ref = _direct(w, cfg, z[0], t[0], ctx[0], pooled[0])
    assert out.shape == z.shape and ref.abs().max() > 0.05
    assert (out[0] - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_presets():
    L, M = S.Sd3Config.large(), S.Sd3Config.medium()
    assert (L.dim, L.num_layers, L.pos_embed_max_size, L.dual_attention_layers) == (2432, 38, 192, ())
    assert (M.dim, M.num_layers, M.pos_embed_max_size, M.dual_attention_layers) == (1536, 24, 384, tuple(range(13)))
    j = S.Sd3Config.from_json({"num_attention_heads": 24, "num_layers": 24, "pos_embed_max_size": 384,
                               "dual_attention_layers": list(range(13)), "qk_norm": "rms_norm"})
    assert j == M


def test_sd3_providers_conform(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.sd3 import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "sd3", dual=True)
    reg = provider_registry("cpu")
    assert [i for i in reg.ids() if "sd3" in i] == ["cpu_sd3_5_large", "cpu_sd3_5_large_turbo", "cpu_sd3_5_medium"]
    assert reg.descriptor_conformance_errors() == []
    turbo = reg.load("cpu_sd3_5_large_turbo", LoadSpec.from_dir(snap))
    kit.conformance(turbo, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_sd3_5_large_turbo", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    with pytest.raises(InferenceError):
        turbo.generate(GenerationRequest(**req, guidance=5.0))                 # distilled: no guidance
    with pytest.raises(InferenceError):
        turbo.generate(GenerationRequest(**{**req, "width": 1024}))           # beyond this snapshot's position table
    med = reg.load("cpu_sd3_5_medium", LoadSpec.from_dir(snap))
    a = med.generate(GenerationRequest(**req, guidance=1.0)).images[0].pixels
    b = med.generate(GenerationRequest(**req)).images[0].pixels                # default guidance 4.5, empty negative
    c = med.generate(GenerationRequest(**req, guidance=4.5, negative_prompt="")).images[0].pixels
    assert b == c and a != b and len(a) == 256 * 256 * 3


def test_triple_text_conditioning_shapes():
    """CLIP-L + CLIP-G second-to-last states side by side, zero-padded to the T5 width, then T5; pooled = both projections."""
    from inference_b200.media.sd3 import TripleTextEncoders

    class Clip:
        def __init__(self, d, p):
            self.d, self.p = d, p

        def encode_all(self, ids):
            return {"penultimate": torch.ones(1, ids.shape[1], self.d), "pooled": torch.zeros(1, self.d),
                    "projected": torch.full((1, self.p), 2.0)}

    class Tok:
        def encode(self, prompt, *a, **k):
            return [1] * (a[0] if a else 77)

    class T5:
        def encode(self, ids):
            return torch.full((1, ids.shape[1], 40), 3.0)

    enc = TripleTextEncoders(Clip(8, 6), Tok(), Clip(12, 10), Tok(), T5(), Tok(), width=40, t5_tokens=16)
    c = enc.encode("x")
    assert c.context.shape == (1, 77 + 16, 40) and c.pooled.shape == (1, 16)
    assert c.context[0, 0, :20].eq(1).all() and c.context[0, 0, 20:].eq(0).all() and c.context[0, 77:].eq(3).all()


def test_sigma_table_golden():
    from inference_b200.media.sd3 import sd3_sigmas

    got = sd3_sigmas(4)
    for a, b in zip(got, [1.0, 0.8573265, 0.6007194, 0.002994012, 0.0]):
        assert abs(a - b) < 1e-6
    s = sd3_sigmas(28)
    assert len(s) == 29 and all(x > y for x, y in zip(s, s[1:]))


def test_sd3_reference_guided_generation(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media import provider_registry
    from inference_b200.media.reference import init_time_step
    from inference_b200.media.sd3 import write_synthetic_snapshot

    assert init_time_step(28, 0.5) == 14 and init_time_step(28, 0.01) == 1 and init_time_step(28, None) == 0
    gen = provider_registry("cpu").load("cpu_sd3_5_large_turbo", LoadSpec.from_dir(write_synthetic_snapshot(tmp_path / "s")))
    g = torch.Generator().manual_seed(3)
    ref = Image(width=128, height=128, pixels=bytes(torch.randint(0, 256, (128 * 128 * 3,), generator=g, dtype=torch.uint8).tolist()))
    base = dict(prompt="a red fox", width=256, height=256, steps=4, seed=5)
    cond = lambda s: [Conditioning(ConditioningKind.REFERENCE, image=ref, strength=s)]      # noqa: E731
    plain = gen.generate(GenerationRequest(**base)).images[0].pixels
    guided = gen.generate(GenerationRequest(**base, conditioning=cond(0.5))).images[0].pixels
    assert guided != plain and gen.generate(GenerationRequest(**base, conditioning=cond(0.5))).images[0].pixels == guided
    assert gen.generate(GenerationRequest(**base, conditioning=cond(0.0))).images[0].pixels == plain
