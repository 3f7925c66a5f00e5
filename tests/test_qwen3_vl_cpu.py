"""Qwen3-VL pieces against Hugging Face transformers on a random tiny configuration: vision tower output and DeepStack
taps, image -> patch layout, three-axis position ids, the interleaved M-RoPE table, and the whole multimodal forward
(embedding splice + DeepStack injection) through the oracle decoder."""
import pytest
import torch

from inference_b200.models import qwen3_vl as V

transformers = pytest.importorskip("transformers")


def _hf(seed=0, head_dim=32, mrope_section=(6, 5, 5)):
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    cfg = Qwen3VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=head_dim, vocab_size=200, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                          "mrope_section": list(mrope_section), "mrope_interleaved": True},
                         tie_word_embeddings=False),
        vision_config=dict(depth=4, hidden_size=48, num_heads=4, intermediate_size=96, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1, 2]),
        image_token_id=150, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153)
    torch.manual_seed(seed)
    return cfg, Qwen3VLForConditionalGeneration(cfg).eval()


def test_vision_tower_matches_hugging_face():
    cfg, model = _hf()
    vc = V.Qwen3VlVisionConfig.from_json(cfg.to_dict())
    assert (vc.depth, vc.hidden_size, vc.patch_dim, vc.grid_side) == (4, 48, 96, 6)
    tower = V.Qwen3VlVisionTower(vc, dict(model.state_dict()))
    g = torch.Generator().manual_seed(1)
    grids = [(1, 4, 6), (1, 2, 2), (2, 2, 4)]                       # two stills and a two-patch video
    patches = torch.randn(4 * 6 + 2 * 2 + 2 * 2 * 4, vc.patch_dim, generator=g)
    with torch.no_grad():
        ref = model.model.visual(patches, grid_thw=torch.tensor(grids))
    out, taps = tower.forward(patches, grids)
    assert out.shape == (7 + 4, 64) and len(taps) == 3
    torch.testing.assert_close(out, ref.pooler_output, atol=2e-5, rtol=1e-4)
    for a, b in zip(taps, ref.deepstack_features):
        torch.testing.assert_close(a, b, atol=2e-5, rtol=1e-4)


def test_patch_layout_and_smart_resize():
    vc = V.Qwen3VlVisionConfig(patch_size=4, hidden_size=48, num_heads=4)
    assert V.smart_resize(100, 37, 8, min_pixels=64, max_pixels=10 ** 6) == (96, 40)          # round-half-even, as Python rounds 12.5
    assert V.smart_resize(1000, 1000, 32, max_pixels=256 * 256)[0] <= 256
    img = torch.arange(16 * 24 * 3, dtype=torch.float32).remainder(251).view(16, 24, 3).to(torch.uint8)
    patches, grid = V.image_to_patches(img, vc, min_pixels=16, max_pixels=10 ** 6)
    assert grid == (1, 4, 6) and patches.shape == (24, 3 * 2 * 4 * 4)
    # merge order: patch 1 is (row 0, col 1), patch 2 is (row 1, col 0); channel-major, frame repeated
    norm = (img.float() / 255 - 0.5) / 0.5
    p2 = patches[2].view(3, 2, 4, 4)
    torch.testing.assert_close(p2[:, 0], norm[4:8, 0:4].permute(2, 0, 1))
    torch.testing.assert_close(p2[:, 1], p2[:, 0])
    torch.testing.assert_close(patches[4].view(3, 2, 4, 4)[:, 0], norm[0:4, 8:12].permute(2, 0, 1))


def test_position_ids_and_interleaved_table_match_hugging_face():
    cfg, model = _hf()
    ids = [5, 6, 152] + [150] * 6 + [153, 7, 8, 152] + [150] * 1 + [153, 9]
    grids = [(1, 4, 6), (1, 2, 2)]
    pos, nxt = V.mrope_positions(ids, grids, 150)
    mm = torch.zeros(1, len(ids), dtype=torch.int32)
    mm[0, [i for i, t in enumerate(ids) if t == 150]] = 1
    ref, delta = model.model.get_rope_index(torch.tensor([ids]), mm_token_type_ids=mm, image_grid_thw=torch.tensor(grids))
    assert torch.equal(pos, ref[:, 0]) and nxt == int(ref.max()) + 1 and int(delta) == nxt - len(ids)
    rot = model.model.language_model.rotary_emb
    cos_ref, sin_ref = rot(torch.zeros(1, 1, 32), ref)
    cos, sin = V.interleaved_mrope_table(pos, rot.inv_freq, (6, 5, 5))
    torch.testing.assert_close(cos, cos_ref[0, :, :16], atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(sin, sin_ref[0, :, :16], atol=1e-6, rtol=1e-6)


def test_multimodal_forward_matches_hugging_face():
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import OracleLlama

    cfg, model = _hf(seed=3)
    sd = dict(model.state_dict())
    mc = ModelConfig.from_json(cfg.to_dict() | {"architectures": ["Qwen3VLForConditionalGeneration"]})
    assert mc.mrope_section == (6, 5, 5)
    text = {k.replace("model.language_model.", "model."): v for k, v in sd.items() if not k.startswith("model.visual.")}
    oracle = OracleLlama(mc, text)
    vc = V.Qwen3VlVisionConfig.from_json(cfg.to_dict())
    tower = V.Qwen3VlVisionTower(vc, sd)
    ids = [5, 6, 152] + [150] * 6 + [153, 7, 8]
    grids = [(1, 4, 6)]
    patches = torch.randn(24, vc.patch_dim, generator=torch.Generator().manual_seed(4))
    tokens, taps = tower.forward(patches, grids)
    rows = torch.tensor([i for i, t in enumerate(ids) if t == 150])
    emb = oracle.embed(torch.tensor([ids]))
    emb[0, rows] = tokens
    pos, nxt = V.mrope_positions(ids, grids, 150)
    h = oracle.hidden_states(None, None, embeds=emb, mrope_positions=pos, deepstack=(rows, taps))
    logits = oracle.project_logits(h)
    mm = torch.zeros(1, len(ids), dtype=torch.int32)
    mm[0, rows] = 1
    with torch.no_grad():
        ref = model(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor(grids),
                    mm_token_type_ids=mm).logits
    torch.testing.assert_close(logits, ref, atol=3e-5, rtol=1e-4)


def test_text_provider_answers_about_an_image(tmp_path):
    """A Qwen3-VL snapshot loads model-first through the text registry; greedy decoding with an image in the prompt
    matches Hugging Face generate() on the same token ids and patches (so the positions of the decode steps continue
    after the image block as the library's do)."""
    import json

    from inference_b200.bundles import runtime_cpu
    from inference_b200.contracts.core_llm import LoadSpec, Message, Role, TextLlmRequest
    from inference_b200.contracts.core_llm.message import ImageRef, Text
    from inference_b200.contracts.core_llm.request import Sampling
    from inference_b200.contracts.core_llm.template import RenderOptions
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json

    cfg, hf = _hf(seed=5)
    top = cfg.to_dict()
    top["model_type"] = "qwen3_vl"
    top["architectures"] = ["Qwen3VLForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(top))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    tok = json.loads(wordlevel_tokenizer_json(200))
    special = {150: "<|image_pad|>", 152: "<|vision_start|>", 153: "<|vision_end|>"}
    tok["model"]["vocab"] = {special.get(i, w): i for w, i in tok["model"]["vocab"].items()}
    tok["added_tokens"] = tok.get("added_tokens", []) + [
        {"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True}
        for i, c in special.items()]
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))
    llm = runtime_cpu.catalog().text().load_for_model(LoadSpec.dense(str(tmp_path)))
    d = llm.descriptor()
    assert d.id == "cpu-qwen3-vl" and d.capabilities.supports_vision
    g = torch.Generator().manual_seed(5)
    raw = bytes(torch.randint(0, 256, (16 * 24 * 3,), generator=g, dtype=torch.uint8).tolist())
    msg = Message(Role.USER, [ImageRef(24, 16, raw), Text("the cat sat")])
    req = TextLlmRequest(messages=[msg], max_new_tokens=5, seed=0, sampling=Sampling(temperature=0.0))
    # this tiny tower has 4-pixel patches: keep the test image at its own size
    import inference_b200.models.qwen3_vl as Q3

    orig = Q3.image_to_patches
    Q3.image_to_patches = lambda rgb, vc, **kw: orig(rgb, vc, min_pixels=16, max_pixels=10 ** 6)
    try:
        ids, seq = llm._splice_media(req, llm.tokenizer.encode(
            llm.template.render_with(llm._render_messages(req), RenderOptions(True, None, [])), add_special_tokens=False))
        assert ids.count(150) == (16 // 8) * (24 // 8) and seq is not None
        llm.backend.release(seq)
        out = llm.generate(req, on_event=lambda e: None)
    finally:
        Q3.image_to_patches = orig
    patches, grid = orig(torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(16, 24, 3),
                         Q3.Qwen3VlVisionConfig.from_json(top), min_pixels=16, max_pixels=10 ** 6)
    mm = torch.tensor([[1 if t == 150 else 0 for t in ids]], dtype=torch.int32)
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([grid]),
                          mm_token_type_ids=mm, attention_mask=torch.ones(1, len(ids), dtype=torch.long), max_new_tokens=5,
                          do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    stops = set(llm.stop_tokens)
    want = []
    for t in ref:
        if t in stops:
            break
        want.append(t)
    words = {i: w for w, i in tok["model"]["vocab"].items()}
    got = out.text.split()
    assert len(got) >= 1 and got == [words[t] for t in want][: len(got)]


def test_video_patches_placeholders_and_positions():
    vc = V.Qwen3VlVisionConfig(patch_size=4, hidden_size=48, num_heads=4)
    g = torch.Generator().manual_seed(0)
    frames = [torch.randint(0, 256, (16, 16, 3), generator=g, dtype=torch.uint8) for _ in range(3)]
    patches, grid, stamps = V.video_to_patches(frames, [0.0, 0.5, 1.0], vc, min_pixels=16, max_pixels=10 ** 6)
    assert grid == (2, 4, 4) and patches.shape == (2 * 16, 3 * 2 * 4 * 4) and stamps == [0.25, 1.0]
    norm = lambda f: (f.float() / 255 - 0.5) / 0.5                                    # noqa: E731
    p0 = patches[0].view(3, 2, 4, 4)
    torch.testing.assert_close(p0[:, 0], norm(frames[0])[:4, :4].permute(2, 0, 1))
    torch.testing.assert_close(p0[:, 1], norm(frames[1])[:4, :4].permute(2, 0, 1))
    last = patches[16].view(3, 2, 4, 4)                                              # second temporal patch: frame 2 twice
    torch.testing.assert_close(last[:, 0], last[:, 1])
    # the timestamp text of the published alignment case: frames at 0, 0.5, 1.0, 1.5 s
    assert V.video_placeholder_text([0.25, 1.25]) == ("<0.2 seconds><|vision_start|><|video_pad|><|vision_end|>"
                                                      "<1.2 seconds><|vision_start|><|video_pad|><|vision_end|>")
    # positions: every temporal patch is its own run with its own (1, h, w) grid
    ids = [27, 15, 152] + [151] * 4 + [153, 27, 16, 152] + [151] * 4 + [153, 9]
    pos, nxt = V.mrope_positions(ids, [(1, 4, 4), (1, 4, 4)], {150, 151})
    assert pos[0, 3:7].tolist() == [3] * 4 and pos[1, 3:7].tolist() == [3, 3, 4, 4] and pos[2, 3:7].tolist() == [3, 4, 3, 4]
    assert pos[:, 7].tolist() == [5, 5, 5] and nxt == int(pos.max()) + 1
    cfg, model = _hf()
    mm = torch.tensor([[2 if t == 151 else 0 for t in ids]], dtype=torch.int32)
    ref, _ = model.model.get_rope_index(torch.tensor([ids]), mm_token_type_ids=mm, video_grid_thw=torch.tensor([[2, 4, 4]]))
    assert torch.equal(pos, ref[:, 0])


def test_text_provider_answers_about_a_video(tmp_path):
    import json

    from inference_b200.bundles import runtime_cpu
    from inference_b200.contracts.core_llm import LoadSpec, Message, Role, TextLlmRequest
    from inference_b200.contracts.core_llm.message import ImageRef, Text, VideoRef
    from inference_b200.contracts.core_llm.request import Sampling
    from inference_b200.contracts.core_llm.template import RenderOptions
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json
    import inference_b200.models.qwen3_vl as Q3

    cfg, hf = _hf(seed=6)
    top = cfg.to_dict()
    top["model_type"], top["architectures"] = "qwen3_vl", ["Qwen3VLForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(top))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    tok = json.loads(wordlevel_tokenizer_json(200))
    special = {150: "<|image_pad|>", 151: "<|video_pad|>", 152: "<|vision_start|>", 153: "<|vision_end|>"}
    tok["model"]["vocab"] = {special.get(i, w): i for w, i in tok["model"]["vocab"].items()}
    tok["added_tokens"] = tok.get("added_tokens", []) + [
        {"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True}
        for i, c in special.items()]
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))
    llm = runtime_cpu.catalog().text().load_for_model(LoadSpec.dense(str(tmp_path)))
    assert llm.descriptor().capabilities.supports_video
    g = torch.Generator().manual_seed(5)
    frames = [torch.randint(0, 256, (16, 16, 3), generator=g, dtype=torch.uint8) for _ in range(4)]
    video = VideoRef(tuple(ImageRef(16, 16, bytes(f.flatten().tolist())) for f in frames), (0.0, 0.5, 1.0, 1.5))
    req = TextLlmRequest(messages=[Message(Role.USER, [video, Text("the cat sat")])], max_new_tokens=4, seed=0,
                         sampling=Sampling(temperature=0.0))
    lim = dict(min_pixels=16, max_pixels=10 ** 6)
    orig_v = Q3.video_to_patches
    Q3.video_to_patches = lambda fr, ts, vc, **kw: orig_v(fr, ts, vc, **lim)
    try:
        ids, seq = llm._splice_media(req, llm.tokenizer.encode(
            llm.template.render_with(llm._render_messages(req), RenderOptions(True, None, [])), add_special_tokens=False))
        assert ids.count(151) == 2 * 4 and ids.count(152) == 2                 # two temporal patches, four merged tokens each
        llm.backend.release(seq)
        out = llm.generate(req, on_event=lambda e: None)
    finally:
        Q3.video_to_patches = orig_v
    patches, grid, _ = orig_v(frames, [0.0, 0.5, 1.0, 1.5], Q3.Qwen3VlVisionConfig.from_json(top), **lim)
    mm = torch.tensor([[2 if t == 151 else 0 for t in ids]], dtype=torch.int32)
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values_videos=patches, video_grid_thw=torch.tensor([grid]),
                          mm_token_type_ids=mm, attention_mask=torch.ones(1, len(ids), dtype=torch.long), max_new_tokens=4,
                          do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    want = []
    for t in ref:
        if t in set(llm.stop_tokens):
            break
        want.append(t)
    words = {i: w for w, i in tok["model"]["vocab"].items()}
    got = out.text.split()
    assert len(got) >= 1 and got == [words[t] for t in want][: len(got)]
