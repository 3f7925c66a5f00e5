"""JoyCaption: the instruction builder against the reference's golden strings, trigger words, request validation, and
the captioner on a tiny LLaVA checkpoint (image features spliced into a system + user chat transcript)."""
import pytest
import torch

from inference_b200.media import joycaption as J


def test_prompt_builder_matches_reference_strings():
    o = J.CaptionOptions
    assert J.build_prompt(o()) == "Write a long detailed description for this image."
    assert J.build_prompt(o(caption_length="any")) == "Write a detailed description for this image."
    assert J.build_prompt(o(caption_length="85")) == "Write a detailed description for this image in 85 words or less."
    assert J.build_prompt(o(caption_type="MidJourney", caption_length="short")) == "Write a short MidJourney prompt for this image."
    assert J.build_prompt(o(caption_type="no such type", caption_length="any")) == "Write a detailed description for this image."
    assert J.build_prompt(o(custom_prompt="  describe the cat  ")) == "describe the cat"
    named = J.build_prompt(o(caption_length="any", extra_options=[J.JOY_NAME_OPTION], name_input="Ada"))
    assert named.endswith("you must refer to them as Ada.")
    assert "{NAME}" in J.build_prompt(o(caption_length="any", extra_options=[J.JOY_NAME_OPTION]))
    assert J.build_prompt(o(caption_type="Danbooru tag list", caption_length="40")).endswith("No extra text. 40 words or less.")
    assert len(J.CAPTION_TYPES) == 12 and J.CAPTION_LENGTHS[0] == "any"


def test_trigger_words_are_prepended_once():
    assert J.apply_trigger_words("a  red   fox", ["sks", " Fox ", ""]) == "sks, a red fox"
    assert J.apply_trigger_words("", ["sks"]) == "sks"
    assert J.apply_trigger_words("plain", []) == "plain"


def test_captioner_on_a_tiny_llava_checkpoint(tmp_path):
    from test_vision_cpu import _tiny_llava

    class _WordTok:                                   # words hash into the 99 non-image token ids
        def encode(self, text):
            return [sum(w.encode()) % 99 for w in text.split()]

        def decode(self, ids):
            return " ".join(str(i) for i in ids)
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media.vision_providers import OracleLm
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import OracleLlama
    from inference_b200.models.vision import VisionConfig, VisionTower

    hc, hf = _tiny_llava()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    strip = lambda pre: {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}      # noqa: E731
    tower = VisionTower(VisionConfig.from_json(hc.to_dict()), strip("model.vision_tower."))
    proj = strip("model.multi_modal_projector.")
    lmw = {"model." + k: v for k, v in strip("model.language_model.").items()}
    lmw["lm_head.weight"] = sd["lm_head.weight"]
    oracle = OracleLlama(ModelConfig.from_json(hc.text_config.to_dict()), lmw)
    cap = J.JoyCaptioner(tower, proj, OracleLm(oracle), _WordTok(), 100, "cpu", -2)
    g = torch.Generator().manual_seed(0)
    img = Image(32, 32, bytes(torch.randint(0, 255, (32 * 32 * 3,), generator=g).tolist()))
    a = cap.caption(img, max_new_tokens=5)
    b = cap.caption(img, max_new_tokens=5, options=J.CaptionOptions(caption_type="MidJourney", caption_length="short"))
    c = cap.caption(img, max_new_tokens=5, options=J.CaptionOptions(trigger_words=["zzq"]))
    assert isinstance(a, str) and isinstance(b, str) and c.startswith("zzq")
    # the transcript has the system prompt, the image block and the instruction in that order
    ids = cap.build_prompt("hello there", 4)
    assert ids.count(100) == 4
    d = cap.descriptor()
    assert d.id == J.JOY_CAPTION_MODEL_ID and d.family == "joycaption"
    with pytest.raises(InferenceError):
        cap.caption(img, options=J.CaptionOptions(caption_length="enormous"))
    with pytest.raises(InferenceError):
        cap.caption(img, max_new_tokens=5000)
    with pytest.raises(InferenceError):
        cap.caption(img, options=J.CaptionOptions(trigger_words=["w"] * 40))


def test_registered_in_both_bundles():
    from inference_b200.media import provider_registry

    for backend in ("cpu", "b200"):
        ids = [r.descriptor().id for r in provider_registry(backend).registrations("captioner")]
        assert J.JOY_CAPTION_MODEL_ID in ids and "llava_captioner" in ids
