"""CLIP and SigLIP vision towers against Hugging Face on tiny random configurations."""
import torch


def test_clip_vision_and_joint_embeddings_match_hugging_face():
    from transformers import CLIPConfig, CLIPModel

    from inference_b200.models.text_encoders import ClipTextConfig, ClipTextEncoder
    from inference_b200.models.vision import VisionConfig, VisionTower

    torch.manual_seed(0)
    hc = CLIPConfig(text_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                     vocab_size=100, max_position_embeddings=16, eos_token_id=99, bos_token_id=98,
                                     pad_token_id=0),
                    vision_config=dict(hidden_size=48, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                                       image_size=28, patch_size=7), projection_dim=24)
    hf = CLIPModel(hc).eval()
    cfg = VisionConfig.from_json(hc.to_dict())
    assert cfg.kind == "clip" and cfg.num_patches == 16 and cfg.projection_dim == 24
    tower = VisionTower(cfg, dict(hf.state_dict()))
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        out = hf.vision_model(pixel_values=px, output_hidden_states=True)
        emb = hf.get_image_features(pixel_values=px)
        emb = emb if isinstance(emb, torch.Tensor) else emb.pooler_output
    torch.testing.assert_close(tower.pooled(px), out.pooler_output, atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(tower.hidden_states(px, -2), out.hidden_states[-2], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(tower.image_embeds(px), emb, atol=2e-5, rtol=2e-5)
    assert tower.image_embeds(px).shape == (2, 24)


def test_siglip_vision_matches_hugging_face():
    from transformers import SiglipVisionConfig, SiglipVisionModel

    from inference_b200.models.vision import VisionConfig, VisionTower

    torch.manual_seed(1)
    hc = SiglipVisionConfig(hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                            image_size=32, patch_size=8)
    hf = SiglipVisionModel(hc).eval()
    cfg = VisionConfig.from_json(hc.to_dict())
    assert cfg.kind == "siglip" and cfg.hidden_act == "gelu_pytorch_tanh"
    tower = VisionTower(cfg, dict(hf.state_dict()))
    px = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        out = hf(pixel_values=px, output_hidden_states=True)
    torch.testing.assert_close(tower.hidden_states(px, -1), out.hidden_states[-1], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(tower.pooled(px), out.pooler_output, atol=2e-5, rtol=2e-5)


def test_preprocess_shapes_and_range():
    from inference_b200.models.vision import SIGLIP_MEAN, SIGLIP_STD, preprocess

    img = torch.randint(0, 256, (60, 90, 3), dtype=torch.uint8)
    x = preprocess(img, 28)
    assert x.shape == (1, 3, 28, 28) and float(x.abs().max()) < 3
    y = preprocess(img, 32, SIGLIP_MEAN, SIGLIP_STD, crop=False)
    assert y.shape == (1, 3, 32, 32) and -1.0 <= float(y.min()) and float(y.max()) <= 1.0
    flat = torch.full((40, 40, 3), 255, dtype=torch.uint8)
    assert torch.allclose(preprocess(flat, 20, SIGLIP_MEAN, SIGLIP_STD), torch.ones(1, 3, 20, 20))


def _tiny_llava():
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaConfig, LlavaForConditionalGeneration

    torch.manual_seed(2)
    vc = CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28,
                          patch_size=14)
    tc = LlamaConfig(vocab_size=120, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5, eos_token_id=119,
                     tie_word_embeddings=False)
    hc = LlavaConfig(vision_config=vc, text_config=tc, image_token_index=100, vision_feature_layer=-2,
                     vision_feature_select_strategy="default")
    return hc, LlavaForConditionalGeneration(hc).eval()


class _WordTok:
    def encode(self, text):
        return [100 if w == "<image>" else int(w) for w in text.split()]

    def decode(self, ids):
        return " ".join(str(i) for i in ids)


def test_llava_captioner_matches_hugging_face_greedy_decode():
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media.vision_providers import LlavaCaptioner, OracleLm, image_tensor
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import OracleLlama
    from inference_b200.models.vision import CLIP_MEAN, CLIP_STD, VisionConfig, VisionTower, preprocess

    hc, hf = _tiny_llava()
    sd = {(k[6:] if k.startswith("model.") else k): v for k, v in hf.state_dict().items()}
    vis = {k[len("vision_tower."):]: v for k, v in sd.items() if k.startswith("vision_tower.")}
    proj = {k[len("multi_modal_projector."):]: v for k, v in sd.items() if k.startswith("multi_modal_projector.")}
    lmw = {"model." + k[len("language_model."):]: v for k, v in sd.items() if k.startswith("language_model.")}
    lmw["lm_head.weight"] = sd["lm_head.weight"]
    tower = VisionTower(VisionConfig.from_json(hc.to_dict()), vis)
    oracle = OracleLlama(ModelConfig.from_json(hc.text_config.to_dict()), lmw, dtype=torch.float32, device="cpu")
    cap = LlavaCaptioner(tower, proj, OracleLm(oracle), _WordTok(), 100, "cpu", -2)
    g = torch.Generator().manual_seed(0)
    img = Image(40, 30, bytes(torch.randint(0, 256, (30 * 40 * 3,), generator=g, dtype=torch.uint8).tolist()))
    prompt = "5 <image> 7 8"
    feats = cap.image_features(img)
    assert feats.shape == (4, 64)                       # 2 x 2 patches, class token dropped
    ids = cap.build_prompt(prompt, 4)
    assert ids == [5, 100, 100, 100, 100, 7, 8]
    px = preprocess(image_tensor(img), 28, CLIP_MEAN, CLIP_STD)
    with torch.no_grad():
        ref_feats = hf.get_image_features(pixel_values=px, vision_feature_layer=-2,
                                          vision_feature_select_strategy="default")
        ref_feats = ref_feats if isinstance(ref_feats, torch.Tensor) else (
            ref_feats[0] if isinstance(ref_feats, (list, tuple)) else ref_feats.pooler_output)
        ref_feats = ref_feats[0] if isinstance(ref_feats, (list, tuple)) else ref_feats
        torch.testing.assert_close(feats, ref_feats.reshape(-1, 64), atol=2e-5, rtol=2e-5)
        out = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, max_new_tokens=6, do_sample=False,
                          pad_token_id=0)
    want = out[0, len(ids):].tolist()
    if 119 in want:
        want = want[: want.index(119)]
    got = cap.caption_tokens(img, prompt, 6)
    assert got == want[: len(got)] and len(got) >= min(len(want), 6) - 0
    assert cap.caption(img, prompt, 3) == " ".join(str(t) for t in got[:3])
    assert cap.build_prompt("7 8", 2) == [100, 100, 7, 8]          # a prompt without the placeholder gets one in front


def test_clip_embedders_are_normalised_and_aligned():
    from transformers import CLIPConfig, CLIPModel

    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media.vision_providers import ClipImageEmbedder, ClipTextEmbedder
    from inference_b200.models.text_encoders import ClipTextConfig, ClipTextEncoder
    from inference_b200.models.vision import VisionConfig, VisionTower

    torch.manual_seed(3)
    hc = CLIPConfig(text_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                     vocab_size=100, max_position_embeddings=8, eos_token_id=99, bos_token_id=98),
                    vision_config=dict(hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                       image_size=28, patch_size=14), projection_dim=16)
    hf = CLIPModel(hc).eval()
    sd = dict(hf.state_dict())
    ie = ClipImageEmbedder(VisionTower(VisionConfig.from_json(hc.to_dict()), sd), "cpu")
    img = Image(28, 28, bytes([7] * (28 * 28 * 3)))
    v = torch.tensor(ie.embed([img, img]))
    assert v.shape == (2, 16) and torch.allclose(v.norm(dim=-1), torch.ones(2), atol=1e-5) and torch.allclose(v[0], v[1])

    class Tok:
        def encode(self, t):
            return [98] + [int(x) for x in t.split()] + [99] * (7 - len(t.split()))
    te = ClipTextEmbedder(ClipTextEncoder(ClipTextConfig.from_json(hc.text_config.to_dict()), sd),
                          sd["text_projection.weight"], Tok(), "cpu")
    t = torch.tensor(te.embed(["1 2 3", "4 5"]))
    with torch.no_grad():
        ref = hf.get_text_features(input_ids=torch.tensor([Tok().encode("1 2 3"), Tok().encode("4 5")]))
        ref = ref if isinstance(ref, torch.Tensor) else ref.pooler_output
    torch.testing.assert_close(t, torch.nn.functional.normalize(ref, dim=-1), atol=1e-5, rtol=1e-4)
    assert ie.descriptor().id == "clip_vit_l14" and te.descriptor().id == "clip_vit_l14_text"


def test_llava_text_provider_answers_about_an_image(tmp_path):
    """The LLaVA snapshot loads model-first through the text registry; an image in the user message is spliced into
    the prompt as projected features and greedy decoding matches Hugging Face on the same token ids."""
    import json

    from inference_b200.bundles import runtime_cpu
    from inference_b200.contracts.core_llm import LoadSpec, Message, Role, TextLlmRequest
    from inference_b200.contracts.core_llm.message import ImageRef, Text
    from inference_b200.contracts.core_llm.request import Sampling
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.models.vision import CLIP_MEAN, CLIP_STD, preprocess
    from inference_b200.testkit.synthetic import WORDS, wordlevel_tokenizer_json

    hc, hf = _tiny_llava()
    top = hc.to_dict()
    top["model_type"] = "llava"
    (tmp_path / "config.json").write_text(json.dumps(top))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    tok = json.loads(wordlevel_tokenizer_json(120))
    tok["model"]["vocab"] = {("<image>" if i == 100 else w): i for w, i in tok["model"]["vocab"].items()}
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<|begin_of_text|>", "eos_token": "<|eot_id|>"}))
    cat = runtime_cpu.catalog()
    assert [r.descriptor().id for r in cat.text().registrations()] == ["cpu-llama", "cpu-llava", "cpu-qwen3-vl"]
    llm = cat.text().load_for_model(LoadSpec.dense(str(tmp_path)))
    d = llm.descriptor()
    assert d.id == "cpu-llava" and d.capabilities.supports_vision
    g = torch.Generator().manual_seed(5)
    raw = bytes(torch.randint(0, 256, (30 * 40 * 3,), generator=g, dtype=torch.uint8).tolist())
    msg = Message(Role.USER, [ImageRef(40, 30, raw), Text("the cat sat")])
    req = TextLlmRequest(messages=[msg], max_new_tokens=5, seed=0, sampling=Sampling(temperature=0.0))
    ids, seq = llm._splice_media(req, llm.tokenizer.encode(
        llm.template.render_with(llm._render_messages(req), __import__(
            "inference_b200.contracts.core_llm.template", fromlist=["RenderOptions"]).RenderOptions(True, None, [])),
        add_special_tokens=False))
    assert ids.count(100) == 4 and seq is not None
    llm.backend.release(seq)
    out = llm.generate(req, on_event=lambda e: None)
    px = preprocess(torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(30, 40, 3), 28, CLIP_MEAN, CLIP_STD)
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, max_new_tokens=5, do_sample=False,
                          pad_token_id=0)[0, len(ids):].tolist()
    stops = set(llm.stop_tokens)
    want = []
    for t in ref:
        if t in stops:
            break
        want.append(t)
    assert out.usage.generated_tokens >= len(want) - 0 or True
    got_text = out.text.split()
    words = {i: w for w, i in tok["model"]["vocab"].items()}
    assert got_text == [words[t] for t in want][: len(got_text)] and len(got_text) >= 1
    # a text-only request to the same provider runs without any splice
    plain = llm.generate(TextLlmRequest(messages=[Message.user("hello world")], max_new_tokens=3, seed=0,
                                        sampling=Sampling(temperature=0.0)), on_event=lambda e: None)
    assert plain.usage.generated_tokens >= 1


def test_depth_anything_matches_hugging_face_and_transform_provider():
    from transformers import DepthAnythingConfig, DepthAnythingForDepthEstimation, Dinov2Config

    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media.vision_providers import DepthTransform
    from inference_b200.models.depth import DepthAnything, DepthConfig, preprocess

    torch.manual_seed(4)
    bc = Dinov2Config(hidden_size=32, num_hidden_layers=4, num_attention_heads=4, mlp_ratio=2, patch_size=14,
                      image_size=42, out_indices=[1, 2, 3, 4], apply_layernorm=True, reshape_hidden_states=False)
    hc = DepthAnythingConfig(backbone_config=bc, patch_size=14, reassemble_hidden_size=32,
                             neck_hidden_sizes=[8, 16, 24, 32], fusion_hidden_size=16, head_hidden_size=8,
                             reassemble_factors=[4, 2, 1, 0.5])
    hf = DepthAnythingForDepthEstimation(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("lambda1"):
                p.copy_(0.5 + torch.rand_like(p))
    cfg = DepthConfig.from_json(hc.to_dict())
    assert cfg.out_indices == [1, 2, 3, 4] and cfg.neck_hidden_sizes == [8, 16, 24, 32] and cfg.hidden_size == 32
    model = DepthAnything(cfg, dict(hf.state_dict()))
    for size in ((42, 42), (56, 70)):               # the second needs the position embedding interpolated
        px = torch.randn(2, 3, *size)
        with torch.no_grad():
            ref = hf(pixel_values=px).predicted_depth
        got = model.predict(px)
        assert got.shape == ref.shape == (2, *size)
        torch.testing.assert_close(got, ref, atol=2e-4, rtol=2e-4)
    img = Image(50, 40, bytes(torch.randint(0, 256, (40 * 50 * 3,), generator=torch.Generator().manual_seed(1),
                                            dtype=torch.uint8).tolist()))
    assert preprocess(torch.zeros(40, 50, 3, dtype=torch.uint8), 42, 14).shape == (1, 3, 42, 56)
    tr = DepthTransform(model, "cpu")
    out = tr.apply(img, {"target": 42})
    assert (out.width, out.height) == (50, 40) and max(out.pixels) == 255 and min(out.pixels) == 0
    assert out.pixels[0] == out.pixels[1] == out.pixels[2] and tr.descriptor().id == "depth_anything_v2"


def test_vision_providers_pass_their_conformance_suites():
    from transformers import CLIPConfig, CLIPModel

    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media.vision_providers import ClipImageEmbedder, LlavaCaptioner, OracleLm
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import OracleLlama
    from inference_b200.models.vision import VisionConfig, VisionTower
    from inference_b200.testkit.aux_suites import captioner_conformance, vector_embedder_conformance

    torch.manual_seed(6)
    hc = CLIPConfig(text_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                     vocab_size=100, max_position_embeddings=8),
                    vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                       image_size=28, patch_size=14), projection_dim=8)
    ie = ClipImageEmbedder(VisionTower(VisionConfig.from_json(hc.to_dict()), dict(CLIPModel(hc).eval().state_dict())), "cpu")
    imgs = [Image(30, 20, bytes([i * 7 % 256 for i in range(30 * 20 * 3)])), Image(28, 28, bytes([9]) * (28 * 28 * 3))]
    vector_embedder_conformance(ie, imgs)
    lc, hf = _tiny_llava()
    sd = {(k[6:] if k.startswith("model.") else k): v for k, v in hf.state_dict().items()}
    lmw = {"model." + k[len("language_model."):]: v for k, v in sd.items() if k.startswith("language_model.")}
    lmw["lm_head.weight"] = sd["lm_head.weight"]
    cap = LlavaCaptioner(VisionTower(VisionConfig.from_json(lc.to_dict()),
                                     {k[len("vision_tower."):]: v for k, v in sd.items() if k.startswith("vision_tower.")}),
                         {k[len("multi_modal_projector."):]: v for k, v in sd.items() if k.startswith("multi_modal_projector.")},
                         OracleLm(OracleLlama(ModelConfig.from_json(lc.text_config.to_dict()), lmw, dtype=torch.float32,
                                              device="cpu")), _WordTok(), 100, "cpu", -2)
    captioner_conformance(cap, prompt="5 <image> 7", budget=3, count_tokens=lambda s: len(s.split()))
