"""SDXL: the UNet's block plan against the published model's geometry, building blocks against torch.nn modules, and
provider conformance on a synthetic snapshot."""
import pytest
import torch
import torch.nn as nn

from inference_b200.models import unet_sdxl as U


def test_plan_matches_the_published_geometry(monkeypatch):
    cfg = U.SdxlUnetConfig()
    down, up = U.unet_plan(cfg)
    assert [(lvl, res, d, s) for lvl, res, d, s in down] == [
        (0, [(320, 320), (320, 320)], 0, True), (1, [(320, 640), (640, 640)], 2, True),
        (2, [(640, 1280), (1280, 1280)], 10, False)]
    assert [res for _, res, _, _ in up] == [[(2560, 1280), (2560, 1280), (1920, 1280)], [(1920, 640), (1280, 640), (960, 640)],
                                            [(960, 320), (640, 320), (640, 320)]]
    count = {"n": 0}

    def fake(*shape, generator=None, device=None):
        count["n"] += int(torch.tensor(shape).prod())
        return torch.zeros(1)
    monkeypatch.setattr(torch, "randn", fake)
    w = U.random_sdxl_unet_weights(cfg)
    assert len(w) == 1680 and count["n"] == 2_567_463_684          # tensors and parameters of the SDXL base UNet
    j = {"block_out_channels": [320, 640, 1280], "transformer_layers_per_block": [1, 2, 10], "attention_head_dim": [5, 10, 20],
         "down_block_types": ["DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"]}
    assert U.SdxlUnetConfig.from_json(j) == cfg


def test_blocks_match_torch_modules():
    cfg = U.SdxlUnetConfig(block_out_channels=(16, 32), transformer_layers_per_block=(0, 1), attention_head_dim=8,
                           cross_attention_dim=12, addition_time_embed_dim=4, projection_class_embeddings_input_dim=24 + 10,
                           norm_groups=4)
    w = U.random_sdxl_unet_weights(cfg, seed=2, std=0.2)
    net = U.SdxlUnet(cfg, w)
    g = torch.Generator().manual_seed(0)
    # residual block
    x, emb = torch.randn(2, 16, 6, 5, generator=g), torch.randn(2, 64, generator=g)
    p = "down_blocks.1.resnets.0"
    n1, n2 = nn.GroupNorm(4, 16, eps=1e-5), nn.GroupNorm(4, 32, eps=1e-5)
    c1, c2, sc, tp = nn.Conv2d(16, 32, 3, padding=1), nn.Conv2d(32, 32, 3, padding=1), nn.Conv2d(16, 32, 1), nn.Linear(64, 32)
    for m, k in ((n1, "norm1"), (n2, "norm2"), (c1, "conv1"), (c2, "conv2"), (sc, "conv_shortcut"), (tp, "time_emb_proj")):
        m.load_state_dict({"weight": w[f"{p}.{k}.weight"], "bias": w[f"{p}.{k}.bias"]})
    act = nn.SiLU()
    with torch.no_grad():
        h = c1(act(n1(x))) + tp(act(emb))[:, :, None, None]
        ref = sc(x) + c2(act(n2(h)))
    torch.testing.assert_close(net._resnet(x, p, torch.nn.functional.silu(emb)), ref, atol=1e-5, rtol=1e-5)
    # cross-attention against nn.MultiheadAttention (separate projection weights, no input bias)
    b = "down_blocks.1.attentions.0.transformer_blocks.0.attn2"
    mha = nn.MultiheadAttention(32, 4, bias=True, kdim=12, vdim=12, batch_first=True)
    mha.load_state_dict({"q_proj_weight": w[b + ".to_q.weight"], "k_proj_weight": w[b + ".to_k.weight"],
                         "v_proj_weight": w[b + ".to_v.weight"], "in_proj_bias": torch.zeros(96),
                         "out_proj.weight": w[b + ".to_out.0.weight"], "out_proj.bias": w[b + ".to_out.0.bias"]})
    q, ctx = torch.randn(2, 9, 32, generator=g), torch.randn(2, 7, 12, generator=g)
    with torch.no_grad():
        ref = mha(q, ctx, ctx, need_weights=False)[0]
    torch.testing.assert_close(net._attention(q, ctx, b), ref, atol=1e-5, rtol=1e-5)
    # the whole network: shape, and dependence on timestep, context and the size numbers
    args = dict(x=torch.randn(1, 4, 8, 12, generator=g), timestep=torch.tensor([400.0]), context=torch.randn(1, 7, 12, generator=g),
                pooled=torch.randn(1, 10, generator=g), time_ids=torch.tensor([[64.0, 96, 0, 0, 64, 96]]))
    base = net.forward(**args)
    assert base.shape == (1, 4, 8, 12)
    for k, v in (("timestep", torch.tensor([10.0])), ("context", args["context"] * 0.5),
                 ("time_ids", torch.tensor([[512.0, 512, 0, 0, 64, 96]]))):
        assert (net.forward(**{**args, k: v}) - base).abs().max() > 1e-5


def test_sdxl_provider_conforms(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.sdxl import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "sdxl")
    reg = provider_registry("cpu")
    assert "cpu_sdxl" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_sdxl", LoadSpec.from_dir(snap))
    kit.conformance(gen, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_sdxl", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = gen.generate(GenerationRequest(**req, guidance=1.0)).images[0].pixels
    b = gen.generate(GenerationRequest(**req)).images[0].pixels
    c = gen.generate(GenerationRequest(**req, guidance=7.0, negative_prompt="", sampler="ddim", scheduler="normal")).images[0].pixels
    d = gen.generate(GenerationRequest(**req, sampler="euler_ancestral", scheduler="karras")).images[0].pixels
    assert b == c and a != b and d != b and len(a) == 256 * 256 * 3
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(**{**req, "width": 264}))


def test_sdxl_trainer_and_adapter_round_trip(tmp_path):
    from inference_b200.contracts.gen_core import (AdapterKind, AdapterSpec, GenerationRequest, LoadSpec, TrainingConfig,
                                                   WeightsSource)
    from inference_b200.io.safetensors_io import load_file, save_file
    from inference_b200.media import provider_registry
    from inference_b200.media.sdxl import write_synthetic_snapshot
    from inference_b200.media.train import SDXL_TARGETS
    from inference_b200.testkit.aux_suites import TrainerProfile, trainer_conformance

    snap = write_synthetic_snapshot(tmp_path / "sdxl")
    ds = tmp_path / "ds"
    ds.mkdir()
    g = torch.Generator().manual_seed(0)
    for i in range(2):
        save_file({"latent": torch.randn(4, 8, 8, generator=g), "txt": torch.randn(9, 64, generator=g),
                   "pooled": torch.randn(32, generator=g)}, ds / f"item{i}.safetensors")
    reg = provider_registry("cpu")
    tr = reg.load_kind("trainer", "cpu_sdxl_lora_trainer", LoadSpec.from_dir(snap))
    items = tr._items(ds)
    noise = torch.randn(4, 8, 8, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    cfg = TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "run", steps=10, learning_rate=5e-3, rank=4, alpha=4.0, seed=3,
                         save_every=5)
    final = tr.train(cfg, lambda p: None)
    ad = load_file(final)
    assert all(k.startswith("unet.") and k.split(".lora_")[0].endswith(SDXL_TARGETS) for k in ad)
    # resume from the step-5 checkpoint reproduces the straight run
    tr2 = reg.load_kind("trainer", "cpu_sdxl_lora_trainer", LoadSpec.from_dir(snap))
    final2 = tr2.train(TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "run2", steps=10, learning_rate=5e-3, rank=4,
                                      alpha=4.0, seed=3, resume=tmp_path / "run" / "adapter-step000005.safetensors"),
                       lambda p: None)
    ad2 = load_file(final2)
    assert all(torch.equal(ad[k], ad2[k]) for k in ad)
    tr.model.lora = {k[len("unet."):-len(".lora_A.weight")]: (ad[k], ad[k.replace("lora_A", "lora_B")], 1.0)
                     for k in ad if k.endswith("lora_A.weight")}
    assert float(tr.loss_on(items[0], 0.5, noise)) < before
    tr.model.lora = None
    big = {k: v * (30.0 if "lora_B" in k else 1.0) for k, v in ad.items()}
    save_file(big, tmp_path / "big.safetensors")
    req = lambda: GenerationRequest(prompt="a fox", width=256, height=256, steps=1, seed=2)      # noqa: E731

    def run(scale):
        spec = LoadSpec(weights=WeightsSource.dir(snap),
                        adapters=[] if scale is None else [AdapterSpec(path=tmp_path / "big.safetensors", scale=scale,
                                                                       kind=AdapterKind.LORA)])
        return reg.load("cpu_sdxl", spec).generate(req(), lambda e: None).images[0].pixels
    plain = run(None)
    assert run(0.0) == plain and run(1.0) != plain
    trainer_conformance(reg.load_kind("trainer", "cpu_sdxl_lora_trainer", LoadSpec.from_dir(snap)),
                        TrainerProfile(ds, tmp_path / "out", steps=3, rank=2))


def test_post_quant_convolution_is_applied_in_front_of_the_decoder():
    from inference_b200.media.sdxl import VAE_SCALE, apply_post_quant
    from inference_b200.models.vae import VaeConfig

    cfg = VaeConfig(z_channels=4, scale_factor=VAE_SCALE, shift_factor=0.25)
    g = torch.Generator().manual_seed(0)
    w, b, z = torch.randn(4, 4, 1, 1, generator=g), torch.randn(4, generator=g), torch.randn(1, 4, 5, 6, generator=g)
    out = apply_post_quant(z, (w, b), cfg)
    want = torch.nn.functional.conv2d(z / VAE_SCALE + 0.25, w, b)
    torch.testing.assert_close(out / VAE_SCALE + 0.25, want, atol=1e-5, rtol=1e-5)
    assert apply_post_quant(z, None, cfg) is z


def test_sdxl_reference_guided_generation(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media import provider_registry
    from inference_b200.media.sdxl import write_synthetic_snapshot

    gen = provider_registry("cpu").load("cpu_sdxl", LoadSpec.from_dir(write_synthetic_snapshot(tmp_path / "s")))
    g = torch.Generator().manual_seed(3)
    ref = Image(width=128, height=128, pixels=bytes(torch.randint(0, 256, (128 * 128 * 3,), generator=g, dtype=torch.uint8).tolist()))
    base = dict(prompt="a red fox", width=256, height=256, steps=4, seed=5)
    cond = lambda s: [Conditioning(ConditioningKind.REFERENCE, image=ref, strength=s)]      # noqa: E731
    plain = gen.generate(GenerationRequest(**base)).images[0].pixels
    guided = gen.generate(GenerationRequest(**base, conditioning=cond(0.5))).images[0].pixels
    assert guided != plain and gen.generate(GenerationRequest(**base, conditioning=cond(0.5))).images[0].pixels == guided
    assert gen.generate(GenerationRequest(**base, conditioning=cond(0.0))).images[0].pixels == plain
