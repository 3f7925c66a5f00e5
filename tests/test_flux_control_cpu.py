"""FLUX ControlNet branch: the injection interval, the converted branch against a restatement in the checkpoint's own
(diffusers) layout, residual injection into the base model, and the bespoke provider end to end on a synthetic snapshot."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.media import flux_control as C
from inference_b200.models.dit_flux import FluxConfig, OracleFluxDiT, make_ids, random_flux_weights, rope_table, timestep_embedding


def test_interval_and_kinds():
    assert C.control_residual_interval(19, 6) == 4 and C.control_residual_interval(19, 1) == 19
    assert C.control_residual_interval(19, 19) == 1 and C.control_residual_interval(19, 0) == 19
    assert all(min(i // 4, 5) < 6 for i in range(19))
    assert all(C.accepts_control_kind(k) for k in ("pose", "canny", "depth")) and not C.accepts_control_kind("scribble")
    assert C.DEFAULT_CONTROL_SCALE == 0.7


def _restated_branch(cfg: FluxConfig, sd, img, cond, img_ids, txt, txt_ids, t, y, g):
    """The branch in the checkpoint's own layout: separate q / k / v projections, AdaLayerNormZero, explicit softmax."""
    lin = lambda x, p: F.linear(x, sd[p + ".weight"], sd[p + ".bias"])                       # noqa: E731
    H, NH, D = cfg.hidden_size, cfg.num_heads, cfg.head_dim
    hidden = lin(img, "x_embedder") + lin(cond, "controlnet_x_embedder")
    enc = lin(txt, "context_embedder")
    mlp = lambda x, p: lin(F.silu(lin(x, p + ".linear_1")), p + ".linear_2")                 # noqa: E731
    emb = mlp(timestep_embedding(t), "time_text_embed.timestep_embedder") + mlp(timestep_embedding(g), "time_text_embed.guidance_embedder") \
        + mlp(y, "time_text_embed.text_embedder")
    cos, sin = rope_table(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.theta)
    ln = lambda x: F.layer_norm(x, (H,), eps=1e-6)                                           # noqa: E731
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w           # noqa: E731

    def rope(x):                                   # [B, S, NH, D], adjacent pairs
        xr = x.reshape(*x.shape[:-1], D // 2, 2)
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack([xr[..., 0] * c - xr[..., 1] * s, xr[..., 0] * s + xr[..., 1] * c], -1).flatten(-2)

    out = []
    T = enc.shape[1]
    for i in range(cfg.depth):
        b = f"transformer_blocks.{i}"
        m = lin(F.silu(emb), b + ".norm1.linear")[:, None].chunk(6, -1)
        mc = lin(F.silu(emb), b + ".norm1_context.linear")[:, None].chunk(6, -1)
        nh, ne = ln(hidden) * (1 + m[1]) + m[0], ln(enc) * (1 + mc[1]) + mc[0]
        hd = lambda x: x.view(1, -1, NH, D)                                                  # noqa: E731
        q = torch.cat([rms(hd(lin(ne, b + ".attn.add_q_proj")), sd[b + ".attn.norm_added_q.weight"]),
                       rms(hd(lin(nh, b + ".attn.to_q")), sd[b + ".attn.norm_q.weight"])], 1)
        k = torch.cat([rms(hd(lin(ne, b + ".attn.add_k_proj")), sd[b + ".attn.norm_added_k.weight"]),
                       rms(hd(lin(nh, b + ".attn.to_k")), sd[b + ".attn.norm_k.weight"])], 1)
        v = torch.cat([hd(lin(ne, b + ".attn.add_v_proj")), hd(lin(nh, b + ".attn.to_v"))], 1)
        q, k = rope(q).transpose(1, 2), rope(k).transpose(1, 2)
        a = (torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(D), -1) @ v.transpose(1, 2)).transpose(1, 2).reshape(1, -1, H)
        hidden = hidden + m[2] * lin(a[:, T:], b + ".attn.to_out.0")
        enc = enc + mc[2] * lin(a[:, :T], b + ".attn.to_add_out")
        hidden = hidden + m[5] * lin(F.gelu(lin(ln(hidden) * (1 + m[4]) + m[3], b + ".ff.net.0.proj"), approximate="tanh"), b + ".ff.net.2")
        enc = enc + mc[5] * lin(F.gelu(lin(ln(enc) * (1 + mc[4]) + mc[3], b + ".ff_context.net.0.proj"), approximate="tanh"),
                                b + ".ff_context.net.2")
        out.append(lin(hidden, f"controlnet_blocks.{i}"))
    return out


def _inputs(cfg, seed=0, ht=2, wt=3, St=5):
    g = torch.Generator().manual_seed(seed)
    img = torch.randn(1, ht * wt, cfg.in_channels, generator=g)
    cond = torch.randn(1, ht * wt, cfg.in_channels, generator=g)
    txt = torch.randn(1, St, cfg.context_in_dim, generator=g)
    y = torch.randn(1, cfg.vec_in_dim, generator=g)
    txt_ids, img_ids = make_ids(ht, wt, St)
    return img, cond, img_ids, txt, txt_ids, torch.tensor([0.7]), y, torch.tensor([3.5])


def test_branch_matches_restatement_and_injects_into_the_base():
    base_cfg = FluxConfig.tiny()
    sd = C.random_control_weights(base_cfg, layers=2, seed=1)
    branch = C.FluxControlNet(base_cfg, sd)
    assert branch.num_residuals == 2 and branch.cfg.in_channels == 2 * base_cfg.in_channels and branch.cfg.depth_single == 0
    img, cond, img_ids, txt, txt_ids, t, y, g = _inputs(base_cfg)
    got = branch.forward(img, cond, img_ids, txt, txt_ids, t, y, g)
    want = _restated_branch(branch.cfg, sd, img, cond, img_ids, txt, txt_ids, t, y, g)
    assert len(got) == 2
    for a, b in zip(got, want):
        assert a.shape == (1, 6, base_cfg.hidden_size) and torch.allclose(a, b, atol=2e-5, rtol=1e-4)
    # base with residuals: block i receives residual floor(i / interval) * scale after the block
    base = OracleFluxDiT(base_cfg, random_flux_weights(base_cfg, 2, std=0.05))
    plain = base.forward(img, img_ids, txt, txt_ids, t, y, g)
    ctl = C.ControlledDit(base, branch, cond, 0.7)
    assert ctl.interval == 1 and ctl.cfg is base.cfg
    out = ctl.forward(img, img_ids, txt, txt_ids, t, y, g)
    assert out.shape == plain.shape and not torch.allclose(out, plain, atol=1e-4) and base.injector is None
    assert torch.allclose(C.ControlledDit(base, branch, cond, 0.0).forward(img, img_ids, txt, txt_ids, t, y, g), plain, atol=1e-6)
    # the published initialisation (zero control embedder and output projections) leaves the base untouched
    zero = C.FluxControlNet(base_cfg, C.random_control_weights(base_cfg, 2, 1, zero_init=True))
    assert torch.allclose(C.ControlledDit(base, zero, cond, 1.0).forward(img, img_ids, txt, txt_ids, t, y, g), plain, atol=1e-6)
    # explicit restatement of the seam order: inner injector residual first, then the control residual
    class Inner:
        def after_double(self, i, im):
            return torch.full_like(im, 0.01 * (i + 1))

        def after_single(self, i, im):
            return None
    seam = C._Residuals(want, 0.5, 2, Inner())
    r = seam.after_double(1, torch.zeros(1, 6, base_cfg.hidden_size))
    assert torch.allclose(r, 0.02 + 0.5 * want[0]) and seam.after_single(0, None) is None
    one = C._Residuals(want[:1], 1.0, C.control_residual_interval(2, 1))
    assert torch.equal(one.after_double(1, None), want[0])
    from inference_b200.contracts.errors import LoadError
    with pytest.raises(LoadError):
        C.FluxControlNet(base_cfg, {k: v for k, v in sd.items() if not k.startswith("controlnet_blocks.")})
    with pytest.raises(LoadError):
        C.FluxControlNet(base_cfg, {k: v for k, v in sd.items() if k != "transformer_blocks.1.attn.to_k.weight"})


def test_provider_end_to_end(tmp_path):
    from inference_b200.contracts.errors import Canceled, InferenceError, LoadError
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressDecoding, ProgressStep
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media import flux

    snap = flux.write_synthetic_snapshot(tmp_path / "flux", flux.Variant.DEV)
    ctrl_dir = tmp_path / "ctrl"
    ctrl_dir.mkdir()
    with pytest.raises(LoadError):
        C.Flux1DevControl.load(C.Flux1ControlPaths(snap, ctrl_dir), "cpu")
    from inference_b200.contracts.gen_core.runtime import LoadSpec
    from inference_b200.media.catalog import provider_registry
    base_cfg = provider_registry("cpu").load("cpu_flux1_dev", LoadSpec.from_dir(snap)).pipe.dit_cfg
    save_file(C.random_control_weights(base_cfg, layers=1, seed=3, std=0.1), ctrl_dir / C.CONTROL_FILE)
    prov = C.Flux1DevControl.load(C.Flux1ControlPaths(snap, ctrl_dir), "cpu")
    assert prov.num_residuals == 1 and prov.residual_interval == base_cfg.depth
    g = torch.Generator().manual_seed(0)
    pose = Image(40, 24, bytes(torch.randint(0, 256, (24 * 40 * 3,), generator=g, dtype=torch.uint8).tolist()))
    lat = prov.encode_control_latent(pose, 256, 256)
    assert lat.shape == (1, 16 * 16, 64) and torch.isfinite(lat).all()
    events = []
    req = C.Flux1ControlRequest(prompt="a dancer on a stage", width=256, height=256, steps=2, seed=5)
    img = prov.generate(req, pose, events.append)
    assert (img.width, img.height) == (256, 256) and len(img.pixels) == 256 * 256 * 3
    assert [e.current for e in events if isinstance(e, ProgressStep)] == [1, 2] and isinstance(events[-1], ProgressDecoding)
    assert prov.generate(req, pose).pixels == img.pixels                               # reproducible
    off = prov.generate(C.Flux1ControlRequest(prompt="a dancer on a stage", width=256, height=256, steps=2, seed=5, control_scale=0.0), pose)
    from inference_b200.contracts.gen_core import GenerationRequest
    plain = prov.flux.generate(GenerationRequest(prompt="a dancer on a stage", width=256, height=256, steps=2, seed=5,
                                                 guidance=3.5)).images[0]
    assert off.pixels == plain.pixels and off.pixels != img.pixels                     # scale 0 is the base model; the default steers
    other = Image(40, 24, bytes(torch.randint(0, 256, (24 * 40 * 3,), generator=g, dtype=torch.uint8).tolist()))
    assert prov.generate(req, other).pixels != img.pixels
    for bad in (dict(prompt=" "), dict(control_kind="scribble"), dict(width=250), dict(steps=0), dict(control_scale=float("nan"))):
        with pytest.raises(InferenceError):
            prov.generate(C.Flux1ControlRequest(**{**dict(prompt="x", width=256, height=256, steps=2), **bad}), pose)
    with pytest.raises(InferenceError):
        prov.generate(req, _short_image())
    done = C.Flux1ControlRequest(prompt="x", width=256, height=256, steps=2)
    done.cancel.cancel()
    with pytest.raises(Canceled):
        prov.generate(done, pose)


def _short_image():
    from inference_b200.contracts.gen_core.media import Image

    im = Image(4, 4, bytes(48))
    im.pixels = bytes(10)
    return im
