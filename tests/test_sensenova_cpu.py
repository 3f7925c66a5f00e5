"""SenseNova-U1: chat queries, position indexes and the block mask, the time grid, patch layouts, the two-path decoder
(cache is read-only on the generation path; paths use disjoint weights), the vision embedder's merge, the distillation LoRA
merge, and the two providers on a synthetic snapshot."""
import pytest
import torch

from inference_b200.media import sensenova as M
from inference_b200.models import sensenova as S


def test_queries_indexes_and_mask():
    assert M.build_neo1_query("a fox", "") == "<|im_start|>user\na fox<|im_end|>\n<|im_start|>assistant\n"
    assert M.build_neo1_query("a fox", "SYS") == "<|im_start|>system\nSYS<|im_end|>\n<|im_start|>user\na fox<|im_end|>\n<|im_start|>assistant\n"
    assert M.cond_query("x").endswith("<think>\n\n</think>\n\n<img>") and M.uncond_query() == "<|im_start|>user\n<|im_end|>\n<|im_start|>assistant\n<img>"
    t, h, w = S.text_indexes(4)
    assert t.tolist() == [0, 1, 2, 3] and h.tolist() == [0] * 4 and w.tolist() == [0] * 4
    t, h, w = S.image_indexes(2, 3, 5)
    assert t.tolist() == [5] * 6 and h.tolist() == [0, 0, 0, 1, 1, 1] and w.tolist() == [0, 1, 2, 0, 1, 2]
    m = S.block_mask(0, torch.tensor([0, 1, 2]))[0, 0]
    assert m[0, 1] < -1e29 and m[1, 0] == 0 and m[2, 2] == 0                      # text is causal
    m = S.block_mask(1, torch.tensor([5, 5, 5]))[0, 0]
    assert (m == 0).all() and m.shape == (3, 4)                                   # one image sees the prefix and itself


def test_time_grid_and_patch_layouts():
    assert S.time_schedule(4, 1.0, enable=False) == [0.0, 0.25, 0.5, 0.75, 1.0]
    g = S.time_schedule(4, 3.0)
    assert g[0] == 0.0 and g[-1] == 1.0
    for got, t in zip(g, (0.0, 0.25, 0.5, 0.75, 1.0)):
        s = 1.0 - t
        assert got == pytest.approx(1.0 - 3.0 * s / (1.0 + 2.0 * s))
    with pytest.raises(ValueError):
        S.time_schedule(0, 3.0)
    img = torch.arange(48.0).view(1, 3, 4, 4)
    p = S.patchify(img, 2)
    assert p.shape == (1, 4, 12) and torch.equal(S.unpatchify(p, 2, 2, 2), img)
    assert p[0, 0, :3].tolist() == img[0, :, 0, 0].tolist()                       # channel fastest
    cf = S.patchify_channel_first(img, 2)
    assert cf[0, 0, :4].tolist() == img[0, 0, :2, :2].flatten().tolist()          # channel slowest


def _tiny():
    cfg = S.NeoChatConfig(patch_size=4, llm=S.NeoLlmConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                                                          num_key_value_heads=1, head_dim=16, vocab_size=50),
                          vision=S.NeoVisionConfig(hidden_size=16, llm_hidden_size=32, patch_size=4))
    w = S.random_sensenova_weights(cfg, 1)
    return cfg, w, S.SenseNovaT2i(cfg, w)


def test_two_path_decoder_and_cache():
    cfg, w, m = _tiny()
    cache, n = m.prefill([1, 2, 3, 4, 5])
    assert (n, cache.len) == (5, 5) and cache.k[0].shape == (1, 5, 1, 16)
    img = torch.randn(1, 3, 16, 24, generator=torch.Generator().manual_seed(0))
    z, cond = m.step_tokens(img, 0.3, m.noise_scale_embed(1.0, 6))
    assert z.shape == (1, 6, 192) and cond.shape == (1, 6, 32)
    prep = m.prepare(*S.image_indexes(2, 3, n), cache.len)
    v = m.predict_v(cond, prep, cache, z, 0.3, 0.02)
    assert v.shape == (1, 6, 192) and cache.len == 5 and cache.k[0].shape[1] == 5       # generation reads the cache only
    assert torch.equal(m.predict_v(cond, prep, cache, z, 0.3, 0.02), v)
    # prefix incrementality on the understanding path: 3 + 2 tokens leave the same cache as 5 at once
    c2 = S.KvCache(2)
    emb = m.w["language_model.model.embed_tokens.weight"][torch.tensor([1, 2, 3, 4, 5])][None]
    t, h, wd = S.text_indexes(5)
    m.forward_chunk(emb[:, :3], m.prepare(t[:3], h[:3], wd[:3], 0), False, c2, True)
    m.forward_chunk(emb[:, 3:], m.prepare(t[3:], h[3:], wd[3:], 3), False, c2, True)
    assert torch.allclose(c2.k[1], cache.k[1], atol=1e-5) and c2.len == 5
    # the two paths use disjoint parameters
    w2 = dict(w)
    w2["language_model.model.layers.0.mlp_mot_gen.up_proj.weight"] = w2["language_model.model.layers.0.mlp_mot_gen.up_proj.weight"] * 2
    m2 = S.SenseNovaT2i(cfg, w2)
    cb, _ = m2.prefill([1, 2, 3, 4, 5])
    assert torch.equal(cb.k[1], cache.k[1]) and not torch.allclose(m2.predict_v(cond, prep, cb, z, 0.3, 0.02), v)
    # velocity clamps its denominator near t = 1
    assert torch.isfinite(m.predict_v(cond, prep, cache, z, 0.999, 0.02)).all()
    assert m.noise_scale_for(16, 16) == pytest.approx(1.0) and m.noise_scale_for(64, 64) == pytest.approx(4.0) and m.noise_scale_for(512, 512) == 8.0


def test_vision_embedder_merges_four_patches():
    cfg, w, m = _tiny()
    patches = torch.randn(4 * 6, 48, generator=torch.Generator().manual_seed(2))
    out = m.vision_embed(patches, 4, 6)
    assert out.shape == (2 * 3, 32)
    p2 = patches.clone()
    p2[0] += 1.0                                       # patch (0, 0) feeds merged token 0 only
    d = (m.vision_embed(p2, 4, 6) - out).abs().amax(1)
    assert d[0] > 1e-4 and float(d[1:].max()) == 0.0


def test_distill_lora_merge():
    cfg, w, _ = _tiny()
    t = "language_model.model.layers.1.self_attn.q_proj_mot_gen"
    before = w[t + ".weight"].clone()
    down, up = torch.randn(2, 32), torch.randn(32, 2)
    n = S.merge_distill_lora(w, {t + ".lora_down.weight": down, t + ".lora_up.weight": up, t + ".alpha": torch.tensor(4.0)}, 2)
    assert n == 1 and torch.allclose(w[t + ".weight"], before + (up @ down) * 2.0, atol=1e-5)
    with pytest.raises(ValueError):
        S.merge_distill_lora(w, {t + ".lora_down.weight": torch.zeros(0, 32), t + ".lora_up.weight": torch.zeros(32, 0), t + ".alpha": torch.tensor(1.0)}, 2)
    with pytest.raises(ValueError, match="llm_config"):
        S.NeoChatConfig.from_json({"vision_config": {}})
    c = S.NeoChatConfig.from_json({"llm_config": {}, "vision_config": {}, "timestep_shift": 1.0})
    assert c.inference_timestep_shift(3.0) == 3.0
    assert S.NeoChatConfig.from_json({"llm_config": {}, "vision_config": {}, "timestep_shift": 7.0}).inference_timestep_shift(3.0) == 7.0


def test_providers(tmp_path):
    from inference_b200.contracts.errors import InferenceError, LoadError, Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.runtime import ProgressStep, WeightsSource
    from inference_b200.media.catalog import provider_registry

    snap = M.write_synthetic_snapshot(tmp_path / "u1")
    reg = provider_registry("cpu")
    assert {"cpu_sensenova_u1_8b", "cpu_sensenova_u1_8b_fast"} <= set(reg.ids())
    base = reg.load("cpu_sensenova_u1_8b", LoadSpec.from_dir(snap))
    d = base.descriptor()
    assert d.family == "sensenova" and d.capabilities.supports_guidance and not d.capabilities.supports_negative_prompt and d.capabilities.supports_kv_cache
    req = GenerationRequest(prompt="a red fox", width=256, height=288, steps=2, seed=4, guidance=2.0)
    for bad in (dict(prompt=" "), dict(steps=0), dict(width=272)):
        with pytest.raises(InferenceError):
            base.validate(GenerationRequest(**{**req.__dict__, **bad}))
    ev = []
    out = base.generate(req, ev.append)
    assert (out.images[0].width, out.images[0].height) == (256, 288) and [(e.current, e.total) for e in ev if isinstance(e, ProgressStep)] == [(1, 2), (2, 2)]
    assert base.generate(req).images[0].pixels == out.images[0].pixels
    assert base.generate(GenerationRequest(**{**req.__dict__, "guidance": 1.0})).images[0].pixels != out.images[0].pixels
    cfg = base.model()[2]
    assert base.options(req, cfg)["timestep_shift"] == 3.0 and base.options(GenerationRequest(**{**req.__dict__, "scheduler_shift": 2.5}), cfg)["timestep_shift"] == 2.5
    fast = reg.load("cpu_sensenova_u1_8b_fast", LoadSpec.from_dir(snap))
    o = fast.options(GenerationRequest(prompt="x", width=256, height=256), cfg)
    assert (o["num_steps"], o["cfg_scale"]) == (8, 1.0)
    f = fast.generate(GenerationRequest(**{**req.__dict__, "guidance": None}))
    assert f.images[0].pixels != base.generate(GenerationRequest(**{**req.__dict__, "guidance": 1.0})).images[0].pixels      # the LoRA moved the weights
    bare = M.write_synthetic_snapshot(tmp_path / "bare", lora=False)
    with pytest.raises(LoadError, match="distill LoRA"):
        reg.load("cpu_sensenova_u1_8b_fast", LoadSpec.from_dir(bare))
    ok = reg.load("cpu_sensenova_u1_8b_fast", LoadSpec(weights=WeightsSource.dir(bare), components={"distill_lora": WeightsSource.file(snap / M.DISTILL_LORA_FILE)}))
    assert ok.distill_lora == snap / M.DISTILL_LORA_FILE
    (bare / M.DISTILL_MERGED_MARKER).write_text("{}")
    assert reg.load("cpu_sensenova_u1_8b_fast", LoadSpec.from_dir(bare)).distill_lora is None
    with pytest.raises(LoadError, match="not a directory"):
        reg.load("cpu_sensenova_u1_8b_fast", LoadSpec(weights=WeightsSource.dir(tmp_path / "bare2"), components={"distill_lora": WeightsSource.dir(snap)}))
    from inference_b200.contracts.gen_core.runtime import Quant
    with pytest.raises(Unsupported):
        reg.load("cpu_sensenova_u1_8b", LoadSpec(weights=WeightsSource.dir(snap), quantize=list(Quant)[0]))
