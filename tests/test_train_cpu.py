"""LoRA flow-matching trainer on the tiny CPU DiT: the loss drops, checkpoints resume bit-exactly, cancellation is
typed, and a trained adapter merged into the weights reproduces the adapted model."""
import math

import pytest
import torch

from inference_b200.contracts.errors import Canceled, InferenceError
from inference_b200.contracts.gen_core import TrainingConfig
from inference_b200.io.safetensors_io import load_file, save_file
from inference_b200.media.train import FluxLoraTrainer, lora_targets, lr_at, merge_lora
from inference_b200.models.dit_flux import FluxConfig, random_flux_weights

CFG = FluxConfig(in_channels=64, vec_in_dim=16, context_in_dim=32, hidden_size=128, num_heads=1, depth=1,
                 depth_single=1, guidance_embed=True)


@pytest.fixture(scope="module")
def dataset(tmp_path_factory):
    d = tmp_path_factory.mktemp("ds")
    g = torch.Generator().manual_seed(0)
    for i in range(2):
        save_file({"latent": torch.randn(16, 8, 8, generator=g), "txt": torch.randn(6, 32, generator=g),
                   "pooled": torch.randn(16, generator=g)}, d / f"item{i}.safetensors")
    return d


def test_lr_schedules():
    assert lr_at("constant", 5, 10, 0, 1.0) == 1.0
    assert lr_at("linear", 0, 10, 4, 1.0) == pytest.approx(0.25) and lr_at("linear", 7, 10, 4, 1.0) == pytest.approx(0.5)
    assert lr_at("cosine", 10, 10, 0, 2.0) == pytest.approx(0.0, abs=1e-9) and lr_at("cosine", 5, 10, 0, 2.0) == pytest.approx(1.0)
    with pytest.raises(InferenceError):
        lr_at("nope", 0, 1, 0, 1.0)


def test_training_reduces_loss_resumes_and_merges(dataset, tmp_path):
    w = random_flux_weights(CFG, seed=1, std=0.05)
    assert any(t.endswith("img_attn.qkv") for t in lora_targets(w)) and any(t.endswith("linear2") for t in lora_targets(w))
    tr = FluxLoraTrainer(CFG, w)
    items = tr._items(dataset)
    noise = torch.randn(16, 8, 8, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    prog = []
    cfg = TrainingConfig(dataset_dir=dataset, output_dir=tmp_path / "run", steps=12, learning_rate=5e-3, rank=4,
                         alpha=4.0, seed=3, save_every=6, lr_schedule="cosine", warmup_steps=2)
    final = tr.train(cfg, prog.append)
    assert [p.step for p in prog] == list(range(1, 13)) and prog[5].checkpoint is not None and all(
        math.isfinite(p.loss) for p in prog)
    ad = load_file(final)
    # the adapted model (base + merged adapter) must beat the base on the fixed probe
    tr2 = FluxLoraTrainer(CFG, merge_lora(w, {**ad, **{k.replace("lora_A.weight", "alpha"): torch.tensor(cfg.alpha)
                                                       for k in ad if k.endswith("lora_A.weight")}}))
    after = float(tr2.loss_on(items[0], 0.5, noise))
    assert after < before, (before, after)
    # resume from the step-6 checkpoint reproduces the straight run exactly
    tr3 = FluxLoraTrainer(CFG, w)
    cfg2 = TrainingConfig(dataset_dir=dataset, output_dir=tmp_path / "run2", steps=12, learning_rate=5e-3, rank=4,
                          alpha=4.0, seed=3, lr_schedule="cosine", warmup_steps=2,
                          resume=tmp_path / "run" / "adapter-step000006.safetensors")
    prog2 = []
    final2 = tr3.train(cfg2, prog2.append)
    assert [p.step for p in prog2] == list(range(7, 13))
    ad2 = load_file(final2)
    assert all(torch.equal(ad[k], ad2[k]) for k in ad)


def test_lokr_training_reduces_loss_and_its_file_folds_like_any_lokr(dataset, tmp_path):
    """adapter="lokr": Kronecker-factored deltas (w1 (x) w2_a w2_b) train through the same loop; the saved LyCORIS-style
    file, folded into the base by the generic adapter loader, reproduces the adapted model."""
    from inference_b200.contracts.gen_core import AdapterKind, AdapterSpec
    from inference_b200.media.family import fold_adapters
    from inference_b200.media.train import kron_split
    from inference_b200.models.nn_dual import adapter_residual

    assert kron_split(128) == (8, 16) and kron_split(384) == (16, 24) and kron_split(13) == (1, 13)
    g = torch.Generator().manual_seed(4)
    w1, w2a, w2b, x = torch.randn(3, 2, generator=g), torch.randn(4, 2, generator=g), torch.randn(2, 5, generator=g), torch.randn(7, 10, generator=g)
    dense = torch.kron(w1, w2a @ w2b)
    assert torch.allclose(adapter_residual((w1, w2a, w2b, 0.5), x), x @ dense.t() * 0.5, atol=1e-5)
    w = random_flux_weights(CFG, seed=1, std=0.05)
    tr = FluxLoraTrainer(CFG, w)
    items = tr._items(dataset)
    noise = torch.randn(16, 8, 8, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    cfg = TrainingConfig(dataset_dir=dataset, output_dir=tmp_path / "lokr", steps=14, learning_rate=5e-3, rank=4, alpha=4.0,
                         seed=3, adapter="lokr", save_every=7)
    prog = []
    final = tr.train(cfg, prog.append)
    ad = load_file(final)
    assert any(k.endswith(".lokr_w1") for k in ad) and any(k.endswith(".lokr_w2_b") for k in ad) and not any("lora_A" in k for k in ad)
    merged = fold_adapters(w, [AdapterSpec(path=str(final), scale=1.0, kind=AdapterKind.LOKR)], "test")
    after = float(FluxLoraTrainer(CFG, merged).loss_on(items[0], 0.5, noise))
    assert after < before, (before, after)
    # resume is exact for this adapter kind too
    cfg2 = TrainingConfig(dataset_dir=dataset, output_dir=tmp_path / "lokr2", steps=14, learning_rate=5e-3, rank=4, alpha=4.0,
                          seed=3, adapter="lokr", resume=tmp_path / "lokr" / "adapter-step000007.safetensors")
    ad2 = load_file(FluxLoraTrainer(CFG, w).train(cfg2))
    assert all(torch.equal(ad[k], ad2[k]) for k in ad)


def test_validation_and_cancellation(dataset, tmp_path):
    tr = FluxLoraTrainer(CFG, random_flux_weights(CFG, seed=2, std=0.05))
    for bad in (dict(adapter="loha"), dict(steps=0), dict(dataset_dir=tmp_path / "missing"), dict(lr_schedule="zigzag"),
                dict(batch_size=2)):
        kw = dict(dataset_dir=dataset, output_dir=tmp_path / "o", steps=2)
        kw.update(bad)
        with pytest.raises(InferenceError):
            tr.validate(TrainingConfig(**kw))
    cfg = TrainingConfig(dataset_dir=dataset, output_dir=tmp_path / "o", steps=5, rank=2)

    def cancel_after_one(p):
        cfg.cancel.cancel()
    with pytest.raises(Canceled):
        tr.train(cfg, cancel_after_one)
    assert tr.model.lora is None


def test_adapter_is_applied_by_the_generator(tmp_path):
    """An adapter file named in LoadSpec.adapters changes the generated image; scale 0 leaves it unchanged."""
    from inference_b200.contracts.gen_core import AdapterKind, AdapterSpec, GenerationRequest, LoadSpec, WeightsSource
    from inference_b200.media import provider_registry
    from inference_b200.media.flux import Variant, write_synthetic_snapshot

    snap = write_synthetic_snapshot(tmp_path / "snap", Variant.SCHNELL)
    base_w = load_file(snap / Variant.SCHNELL.transformer_file)
    g = torch.Generator().manual_seed(0)
    ad = {}
    for name in lora_targets(base_w)[:3]:
        w = base_w[name + ".weight"]
        ad[f"transformer.{name}.lora_A.weight"] = torch.randn(4, w.shape[1], generator=g) * 0.3
        ad[f"transformer.{name}.lora_B.weight"] = torch.randn(w.shape[0], 4, generator=g) * 0.3
    save_file(ad, tmp_path / "ad.safetensors")
    reg = provider_registry("cpu")
    req = lambda: GenerationRequest(prompt="a fox", width=256, height=256, steps=1, seed=2)   # noqa: E731

    def run(scale):
        spec = LoadSpec(weights=WeightsSource.dir(snap),
                        adapters=[] if scale is None else [AdapterSpec(path=tmp_path / "ad.safetensors", scale=scale,
                                                                       kind=AdapterKind.LORA)])
        return reg.load("cpu_flux1_schnell", spec).generate(req(), lambda e: None).images[0].pixels
    plain = run(None)
    assert run(0.0) == plain and run(1.0) != plain
    with pytest.raises(InferenceError):
        bad = LoadSpec(weights=WeightsSource.dir(snap), adapters=[AdapterSpec(path=tmp_path / "nope.safetensors", scale=1.0,
                                                                              kind=AdapterKind.LORA)])
        reg.load("cpu_flux1_schnell", bad).generate(req(), lambda e: None)


def test_trainer_conformance_suite(dataset, tmp_path):
    from inference_b200.testkit.aux_suites import TrainerProfile, trainer_conformance

    tr = FluxLoraTrainer(CFG, random_flux_weights(CFG, seed=3, std=0.05))
    trainer_conformance(tr, TrainerProfile(dataset, tmp_path / "out", steps=3, rank=2))
