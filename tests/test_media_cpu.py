"""Media engine on the CPU oracle backend: generator conformance, registry laws, seed and residency behaviour."""
import pytest
import torch

from inference_b200.contracts.errors import Canceled, InferenceError, Unsupported
from inference_b200.contracts.gen_core import (GenerationRequest, LoadSpec, OffloadPolicy, ProgressLoading, Quant,
                                               WeightsSource)
from inference_b200.media import image_seed, provider_registry, seeded_noise_nchw
from inference_b200.media.flux import (Variant, flux_schedule, patchify, unpatchify, write_synthetic_snapshot)
from inference_b200.testkit import generator as kit


@pytest.fixture(scope="module")
def snapshot(tmp_path_factory):
    return write_synthetic_snapshot(tmp_path_factory.mktemp("flux_dev"), Variant.DEV)


@pytest.fixture(scope="module")
def registry():
    return provider_registry("cpu")


def test_registry_lists_both_variants(registry):
    assert registry.ids()[:2] == ["cpu_flux1_schnell", "cpu_flux1_dev"]
    assert registry.descriptor_conformance_errors() == []
    dev = registry.find("generator", "cpu_flux1_dev").descriptor()
    sch = registry.find("generator", "cpu_flux1_schnell").descriptor()
    assert dev.capabilities.supports_guidance and not sch.capabilities.supports_guidance
    assert (dev.capabilities.min_size, dev.capabilities.max_size, dev.capabilities.max_count) == (256, 2048, 8)
    assert provider_registry("b200").ids() == ["flux1_schnell", "flux1_dev", "chroma1_hd", "chroma1_base", "chroma1_flash",
                                             "z_image", "z_image_turbo", "sd3_5_large", "sd3_5_large_turbo",
                                             "sd3_5_medium", "qwen_image", "sdxl", "kolors", "wan2_2_t2v_14b", "wan2_2_i2v_14b",
                                             "wan2_2_ti2v_5b", "wan_vace", "bernini_renderer", "scail2_14b", "boogu_image", "boogu_image_turbo", "boogu_image_edit", "sensenova_u1_8b", "sensenova_u1_8b_fast",
                                             "krea_2_turbo", "krea_2_raw", "flux2_klein_9b", "flux2_dev", "sana_1600m",
                                             "sana_sprint_1600m", "ideogram_4", "ideogram_4_turbo", "mochi_1", "anima_base",
                                             "anima_aesthetic", "anima_turbo", "svd_xt"]


def test_generator_conformance(registry, snapshot):
    g = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot))
    kit.conformance(g, kit.Profile(steps=2, cancel_steps=5))
    kit.check_batch_seed_law(g, kit.Profile(steps=1))
    kit.registry_conformance(registry, "cpu_flux1_dev", LoadSpec.from_dir(snapshot))


def test_load_rejections(registry, snapshot):
    with pytest.raises(Unsupported):
        registry.load("cpu_flux1_dev", LoadSpec(weights=WeightsSource.file(snapshot / "flux1-dev.safetensors")))
    with pytest.raises(Unsupported):
        registry.load("cpu_flux1_dev", LoadSpec(weights=WeightsSource.dir(snapshot), quantize=Quant.Q4))
    with pytest.raises(InferenceError):
        registry.load("nope", LoadSpec.from_dir(snapshot))
    g = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot / "missing"))     # lazy: paths only
    with pytest.raises(InferenceError):
        g.generate(GenerationRequest(prompt="x", width=256, height=256, steps=1, seed=1), lambda e: None)


def test_validate_rules(registry, snapshot):
    g = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot))
    ok = dict(prompt="a", width=256, height=256)
    g.validate(GenerationRequest(**ok, guidance=2.0))
    for bad in (dict(ok, prompt=""), dict(ok, width=264), dict(ok, steps=0), dict(ok, negative_prompt="n"),
                dict(ok, guidance=float("nan")), dict(ok, sampler="nope"), dict(ok, count=9)):
        with pytest.raises(InferenceError):
            g.validate(GenerationRequest(**bad))
    s = registry.load("cpu_flux1_schnell", LoadSpec.from_dir(snapshot))
    with pytest.raises(Unsupported):
        s.validate(GenerationRequest(**ok, guidance=3.5))


def test_sequential_policy_drops_components(registry, snapshot):
    spec = LoadSpec(weights=WeightsSource.dir(snapshot), offload_policy=OffloadPolicy.SEQUENTIAL)
    g = registry.load("cpu_flux1_dev", spec)
    ev = []
    req = GenerationRequest(prompt="a", width=256, height=256, steps=1, seed=3)
    a = g.generate(req, ev.append)
    assert g.residency.loaded_phases() == (False, False)
    assert [e.phase.value for e in ev if isinstance(e, ProgressLoading)] == ["text_encoder", "transformer"]
    r = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot))
    b = r.generate(GenerationRequest(prompt="a", width=256, height=256, steps=1, seed=3), lambda e: None)
    assert r.residency.loaded_phases() == (True, True)
    assert a.images[0].pixels == b.images[0].pixels
    ev2 = []
    r.generate(GenerationRequest(prompt="a", width=256, height=256, steps=1, seed=3), ev2.append)
    assert not any(isinstance(e, ProgressLoading) for e in ev2)


def test_samplers_and_schedulers_run(registry, snapshot):
    g = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot))
    base = g.generate(GenerationRequest(prompt="a", width=256, height=256, steps=3, seed=5), lambda e: None)
    for sampler, sched in (("heun", None), ("dpmpp_2m", "simple"), ("euler_ancestral", "karras")):
        ev = []
        out = g.generate(GenerationRequest(prompt="a", width=256, height=256, steps=3, seed=5, sampler=sampler,
                                           scheduler=sched), ev.append)
        kinds = [type(e).__name__ for e in ev]
        assert kinds.count("ProgressStep") == 3 and kinds.count("ProgressDecoding") == 1
        assert len(out.images[0].pixels) == len(base.images[0].pixels)


def test_seed_and_patch_helpers():
    assert image_seed(5, 2) == 7 and image_seed((1 << 64) - 1, 1) == 0
    a, b = seeded_noise_nchw(9, 16, 4, 6), seeded_noise_nchw(9, 16, 4, 6)
    assert torch.equal(a, b) and a.shape == (1, 16, 4, 6) and not torch.equal(a, seeded_noise_nchw(10, 16, 4, 6))
    z = torch.randn(1, 16, 8, 6)
    p = patchify(z)
    assert p.shape == (1, 12, 64) and torch.equal(unpatchify(p, 8, 6), z)
    assert torch.equal(p[0, 1, :4], torch.tensor([z[0, 0, 0, 2], z[0, 0, 0, 3], z[0, 0, 1, 2], z[0, 0, 1, 3]]))
    s = flux_schedule(Variant.DEV, 4, 1024, 1024)
    assert len(s) == 5 and s[0] == 1.0 and s[-1] == 0.0 and all(x > y for x, y in zip(s, s[1:]))
    assert s[2] > 0.5                                # the dev shift pushes time toward the noisy end
    assert flux_schedule(Variant.SCHNELL, 4, 512, 512) == [1.0, 0.75, 0.5, 0.25, 0.0]


def test_flux_with_t5_and_clip_text_encoders(tmp_path):
    """The full pipeline with real (tiny, random) T5 + CLIP encoders and tokenizer files."""
    from inference_b200.media.text_models import ClipBpeTokenizer, T5ClipEncoders

    snap = write_synthetic_snapshot(tmp_path / "flux_te", Variant.SCHNELL, text="t5_clip")
    tok = ClipBpeTokenizer.from_dir(snap / "tokenizer", 24)
    ids = tok.encode("A  Fox, a cat")
    assert len(ids) == 24 and ids[0] == tok.bos and ids[-1] == tok.eos
    assert tok.vocab["fox</w>"] in ids and tok.vocab["cat</w>"] in ids            # merges applied, lower-cased
    enc = T5ClipEncoders.from_snapshot(snap, "cpu", "cpu")
    a, b = enc.encode("a fox", 32), enc.encode("a dog", 32)
    assert a.txt.shape == (1, 32, 64) and a.pooled.shape == (1, 32)
    assert not torch.allclose(a.txt, b.txt) and not torch.allclose(a.pooled, b.pooled)
    g = provider_registry("cpu").load("cpu_flux1_schnell", LoadSpec.from_dir(snap))
    req = dict(width=256, height=256, steps=1, seed=4)
    x = g.generate(GenerationRequest(prompt="a fox", **req), lambda e: None)
    y = g.generate(GenerationRequest(prompt="a fox", **req), lambda e: None)
    z = g.generate(GenerationRequest(prompt="a big red dog", **req), lambda e: None)
    assert x.images[0].pixels == y.images[0].pixels and x.images[0].pixels != z.images[0].pixels
    fp = provider_registry("cpu").footprint("cpu_flux1_schnell", LoadSpec.from_dir(snap))
    assert fp.components["text_encoder"] > 0 and fp.components["text_encoder_2"] > 0


def test_flux_reference_guided_generation(registry, snapshot):
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image

    gen = registry.load("cpu_flux1_dev", LoadSpec.from_dir(snapshot))
    g = torch.Generator().manual_seed(3)
    ref = Image(width=96, height=160, pixels=bytes(torch.randint(0, 256, (160 * 96 * 3,), generator=g, dtype=torch.uint8).tolist()))
    base = dict(prompt="a red fox", width=256, height=256, steps=4, seed=5)
    cond = lambda s: [Conditioning(ConditioningKind.REFERENCE, image=ref, strength=s)]      # noqa: E731
    plain = gen.generate(GenerationRequest(**base)).images[0].pixels
    events = []
    guided = gen.generate(GenerationRequest(**base, conditioning=cond(0.5)), events.append).images[0].pixels
    assert guided != plain and gen.generate(GenerationRequest(**base, conditioning=cond(0.5))).images[0].pixels == guided
    assert gen.generate(GenerationRequest(**base, conditioning=cond(0.0))).images[0].pixels == plain
    assert [e.current for e in events if hasattr(e, "current")] == [1, 2, 3, 4]
