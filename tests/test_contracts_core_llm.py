"""Contract-level unit tests for the text-LLM surface (validation floor, registries, stream text policies)."""
import json

import pytest

from inference_b200.contracts.core_llm import (CancelFlag, Channel, ChatMlTemplate, Constraint,
                                               ConstraintDecodeTable, ImageRef, IncrementalDetok, InferenceError,
                                               InvalidRequest, JinjaChatTemplate, JsonConstraint, Llama3Template,
                                               LoadSpec, Message, ModelFormat, ModelRequirements, PrepareReport,
                                               PrepareSpec, RenderOptions, Role, Sampling,
                                               SnapshotPreparerRegistration, SnapshotPreparerRegistryBuilder,
                                               StopMatcher, TextLlmCapabilities, TextLlmDescriptor,
                                               TextLlmRegistration, TextLlmRegistryBuilder, TextLlmRequest,
                                               ThinkingMode, ThinkingSegmenter, ToolCallSegmenter, ToolSpec,
                                               Unsupported, VideoRef, detect_format)


def test_message_and_media_validation():
    assert ImageRef(2, 2, bytes(12)).width == 2
    with pytest.raises(ValueError):
        ImageRef(2, 2, bytes(10))
    f = ImageRef(1, 1, b"\x01\x02\x03")
    with pytest.raises(ValueError):
        VideoRef((f,), (0.0, 0.5))
    with pytest.raises(ValueError):
        VideoRef((), ())
    m = Message(Role.USER, [VideoRef((f,), (0.0,)), __import__("inference_b200").contracts.core_llm.Text("describe")])
    assert m.has_video() and not m.has_image() and m.text_content() == "describe"


def test_validation_floor():
    caps = TextLlmCapabilities(max_context_tokens=128, max_new_tokens=64, supports_system_prompt=True)
    ok = TextLlmRequest([Message.user("hi")], 8)
    caps.validate_request("p", ok)
    assert ok.sampling.temperature == 0.7 and ok.sampling.top_p == 0.9 and not ok.sampling.is_greedy()
    for bad in (TextLlmRequest([], 8), TextLlmRequest([Message.user("  ")], 8), TextLlmRequest([Message.user("x")], 0),
                TextLlmRequest([Message.user("x")], 65),
                TextLlmRequest([Message.user("x")], 8, sampling=Sampling(temperature=2.5)),
                TextLlmRequest([Message.user("x")], 8, sampling=Sampling(top_p=1.5))):
        with pytest.raises(InvalidRequest):
            caps.validate_request("p", bad)
    for gap in (TextLlmRequest([Message(Role.USER, [ImageRef(1, 1, bytes(3))])], 8),
                TextLlmRequest([Message.user("x")], 8, thinking=ThinkingMode.ENABLED),
                TextLlmRequest([Message.user("x")], 8, tools=[ToolSpec("t", "d", {})]),
                TextLlmRequest([Message.user("x")], 8, constraint=Constraint.JSON)):
        with pytest.raises(Unsupported):
            caps.validate_request("p", gap)
    with pytest.raises(Unsupported):
        TextLlmCapabilities().validate_request("p", TextLlmRequest([Message.system("s"), Message.user("u")], 4))


def _reg(pid, accepts=True, vision=False, probe=None, constraints=()):
    d = TextLlmDescriptor(pid, "fam", "b200", TextLlmCapabilities(supports_vision=vision,
                                                                  supported_constraints=list(constraints)))
    return TextLlmRegistration(lambda: d, lambda spec: pid, lambda spec: accepts, probe)


def test_registry_selection():
    with pytest.raises(InferenceError):
        TextLlmRegistryBuilder().register(_reg("a")).register(_reg("a")).build()
    reg = TextLlmRegistryBuilder().extend([_reg("vlm", vision=True), _reg("text"), _reg("no", accepts=False)]).build()
    spec = LoadSpec.dense("/nonexistent")
    assert reg.load_for_model(spec) == "text"          # text preferred when vision not requested
    assert reg.load_for_model_with(spec, ModelRequirements().with_vision()) == "vlm"
    assert reg.load_textllm("vlm", spec) == "vlm"
    with pytest.raises(InferenceError):
        reg.load_textllm("missing", spec)
    with pytest.raises(Unsupported):
        reg.load_for_model_with(spec, ModelRequirements().with_constraint(Constraint.JSON))
    with pytest.raises(Unsupported):
        TextLlmRegistryBuilder().register(_reg("no", accepts=False)).build().load_for_model(spec)
    probe = TextLlmRegistryBuilder().register(_reg("generic", probe=lambda s: True)).build()
    assert probe.load_for_model_with(spec, ModelRequirements().with_vision()) == "generic"


def test_detect_format_and_preparer_registry(tmp_path):
    (tmp_path / "model.bin").write_bytes(b"GGUF\x00\x00\x00\x03rest")
    assert detect_format(tmp_path / "model.bin") is ModelFormat.GGUF
    (tmp_path / "m.gguf").write_bytes(b"xx")
    assert detect_format(tmp_path / "m.gguf") is ModelFormat.GGUF
    (tmp_path / "m.safetensors").write_bytes(b"\0\0")
    assert detect_format(tmp_path / "m.safetensors") is ModelFormat.SAFETENSORS
    hf = tmp_path / "hf"
    hf.mkdir()
    (hf / "config.json").write_text("{}")
    assert detect_format(hf) is ModelFormat.SAFETENSORS
    with pytest.raises(Unsupported):
        detect_format(tmp_path / "nope")
    rep = PrepareReport(ModelFormat.SAFETENSORS, None, tmp_path, 3, True)
    r = SnapshotPreparerRegistration(lambda: "b200", lambda s: s.source == hf, lambda s: rep)
    regs = SnapshotPreparerRegistryBuilder().register(r).build()
    assert regs.prepare_snapshot(PrepareSpec.dense(hf, tmp_path / "o")) is rep
    with pytest.raises(Unsupported):
        regs.prepare_snapshot(PrepareSpec.dense(tmp_path / "m.gguf", tmp_path / "o"))
    with pytest.raises(InferenceError):
        SnapshotPreparerRegistryBuilder().register(r).register(r).build()


def test_stop_matcher_and_detok():
    m = StopMatcher(["</s>", ""])
    out = ""
    stopped = False
    for d in ["hello <", "/s", ">tail"]:
        c = m.push(d)
        out += c.emit
        if c.stop:
            stopped = True
            break
    assert out == "hello " and stopped
    m = StopMatcher(["STOP"])
    assert m.push("abcST").emit == "abc" and m.flush() == "ST"
    assert StopMatcher([]).push("x").emit == "x"
    det = IncrementalDetok()
    s = "a🌍b".encode()
    acc, outs = b"", []
    for chunk in (s[:1], s[1:3], s[3:5], s[5:]):
        acc += chunk
        d = det.push(acc.decode("utf-8", errors="replace"))
        if d is not None:
            outs.append(d)
    assert outs == ["a", "🌍", "b"]


def test_thinking_and_tool_segmenters():
    seg = ThinkingSegmenter()
    content = thinking = ""
    for d in ["<thi", "nk>rea", "son</th", "ink>ans", "wer"]:
        for sp in seg.push(d):
            if sp.channel is Channel.CONTENT:
                content += sp.text
            else:
                thinking += sp.text
    for sp in seg.flush():
        content += sp.text
    assert (content, thinking) == ("answer", "reason")
    tool = ToolSpec("get_weather", "w", {"type": "object", "properties": {"city": {"type": "string"},
                                                                          "days": {"type": "integer"}}})
    ts = ToolCallSegmenter([tool])
    vis = "".join(sum([ts.push(d) for d in ["Sure. <tool_", "call>\n<function=get_weather>\n<parameter=city>\nParis\n"
                                             "</parameter>\n<parameter=days>3</parameter></function>\n</tool_call> done"]],
                      []))
    vis += "".join(ts.flush())
    assert vis == "Sure.  done"
    c = ts.take_calls()[0]
    assert c.name == "get_weather" and c.arguments == {"city": "Paris", "days": 3}
    ts = ToolCallSegmenter([tool])
    ts.push('<tool_call>{"name": "get_weather", "arguments": {"city": "Rome"}}</tool_call>')
    assert ts.calls()[0].arguments == {"city": "Rome"}
    ts = ToolCallSegmenter([])
    ts.push("<tool_call>garbage")
    assert "".join(ts.flush()) == "<tool_call>garbage"


def test_json_constraint_masks():
    table = ConstraintDecodeTable(['{"', 'a', '":', ' 1', '}', 'x', '', ',"'], special={6})
    jc = JsonConstraint(table)
    allowed = jc.allowed()
    assert allowed[0] and not allowed[4] and not allowed[6] and not allowed[5]
    for t in (0, 1, 2, 3):
        assert jc.accept(t)
    assert not jc.can_stop()
    assert jc.allowed()[4] and jc.allowed()[7]
    assert jc.accept(4) and jc.can_stop()
    assert not any(jc.allowed()[i] for i in (0, 1, 4))


def test_templates():
    msgs = [Message.system("S"), Message.user("U")]
    assert Llama3Template().render(msgs, True).endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert ChatMlTemplate().render(msgs, False) == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n"
    cfg = {"chat_template": [{"name": "other", "template": "X"}, {"name": "default", "template":
           "{{ bos_token }}{% for m in messages %}[{{ m.role }}:{{ m.content }}]{% endfor %}"
           "{% if enable_thinking is defined %}T={{ enable_thinking }}{% endif %}{% if tools %}{{ tools | tojson }}{% endif %}"}],
           "bos_token": {"content": "<s>"}}
    t = JinjaChatTemplate.from_tokenizer_config(cfg)
    assert t.render(msgs, False) == "<s>[system:S][user:U]"
    r = t.render_with(msgs, RenderOptions.generation().with_enable_thinking(False).with_tools([ToolSpec("f", "d", {})]))
    assert "T=False" in r and json.loads(r[r.index("[{"):])[0]["function"]["name"] == "f"
    with pytest.raises(InferenceError):
        JinjaChatTemplate("{{ raise_exception('boom') }}").render(msgs, False)
    with pytest.raises(InferenceError):
        JinjaChatTemplate("{% for %}").render(msgs, False)
    assert not CancelFlag().is_cancelled()
