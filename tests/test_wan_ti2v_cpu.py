"""Wan2.2 TI2V-5B: the parameter-free shortcut of the z48 autoencoder, its decode geometry (and causality in time), the 5B
configuration, and the provider on a synthetic snapshot."""
import pytest
import torch

from inference_b200.media import wan_ti2v as W
from inference_b200.models.vae_qwen import Wan22VaeConfig, Wan22VaeDecoder, random_wan22_vae_weights


def test_dup_shortcut_layout():
    x = torch.arange(2 * 8 * 2 * 1 * 1, dtype=torch.float32).view(2, 8, 2, 1, 1)
    y = Wan22VaeDecoder.dup_shortcut(x, 4, 1, 2)                      # space only: 8 -> 4 channels, 2 x 2 fold
    assert y.shape == (2, 4, 2, 2, 2)
    # repeats = 4 * 4 / 8 = 2: output channel o, offsets (dy, dx) read input channel (o * 4 + dy * 2 + dx) // 2
    for o in range(4):
        for dy in range(2):
            for dx in range(2):
                assert y[0, o, 1, dy, dx] == x[0, (o * 4 + dy * 2 + dx) // 2, 1, 0, 0]
    t = Wan22VaeDecoder.dup_shortcut(x, 4, 2, 2)                       # time and space: the leading frame is dropped
    assert t.shape == (2, 4, 3, 2, 2)
    assert t[0, 0, 0, 0, 0] == x[0, (0 * 8 + 1 * 4) // 4, 0, 0, 0]    # first kept frame is time offset 1 of latent frame 0


def test_decode_geometry_and_causality():
    cfg = Wan22VaeConfig(z_dim=8, base_dim=8, num_res_blocks=1)
    dec = Wan22VaeDecoder(cfg, random_wan22_vae_weights(cfg, 1))
    z = torch.randn(1, 8, 3, 2, 3, generator=torch.Generator().manual_seed(0))
    v = dec.decode(z)
    assert v.shape == (1, 3, 9, 32, 48) and torch.isfinite(v).all()
    assert dec.decode(z[:, :, :1]).shape == (1, 3, 1, 32, 48)
    # causal in time: the frames of the first two latent frames do not depend on the third
    z2 = z.clone()
    z2[:, :, 2] += 1.0
    assert torch.allclose(dec.decode(z2)[:, :, :5], v[:, :, :5], atol=1e-5) and not torch.allclose(dec.decode(z2)[:, :, 5:], v[:, :, 5:], atol=1e-3)
    assert Wan22VaeConfig().dims == (1024, 1024, 1024, 512, 256)


def test_provider(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressStep
    from inference_b200.media.catalog import provider_registry

    c = W.ti2v_dit_config()
    assert (c.dim, c.num_layers, c.in_channels, c.out_channels, c.ffn_dim) == (3072, 30, 48, 48, 14336)
    snap = W.write_synthetic_snapshot(tmp_path / "ti2v")
    reg = provider_registry("cpu")
    assert "cpu_wan2_2_ti2v_5b" in reg.ids()
    gen = reg.load("cpu_wan2_2_ti2v_5b", LoadSpec.from_dir(snap))
    d = gen.descriptor()
    assert d.family == "wan" and d.capabilities.supports_lora and d.capabilities.supports_lokr and d.capabilities.min_size == 480
    req = GenerationRequest(prompt="a kite over dunes", width=480, height=512, frames=5, steps=2, seed=4, guidance=2.0, sampler="euler")
    for bad in (dict(width=496), dict(frames=6), dict(width=1280, height=736), dict(prompt="")):
        with pytest.raises(InferenceError):
            gen.validate(GenerationRequest(**{**req.__dict__, **bad}))
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(**{**req.__dict__, "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=Image(8, 8, bytes(192)))]}))
    ev = []
    out = gen.generate(req, ev.append)
    assert len(out.video_frames) == 5 and out.fps == 24 and (out.video_frames[0].width, out.video_frames[0].height) == (480, 512)
    assert [(e.current, e.total) for e in ev if isinstance(e, ProgressStep)] == [(1, 2), (2, 2)]
    assert gen.generate(req).video_frames[3].pixels == out.video_frames[3].pixels
