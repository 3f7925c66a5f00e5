"""cpu-llama provider through its real load path on tiny synthetic snapshots: conformance, GGUF, preparer, JSON."""
import json

import pytest
import torch

from inference_b200.contracts.core_llm import (Channel, Constraint, FinishReason, LoadSpec, Message, ModelFormat,
                                               PrepareSpec, Quantize, Sampling, SnapshotPreparerRegistryBuilder,
                                               TextLlmRegistryBuilder, TextLlmRequest, ThinkingMode, TokenEvent,
                                               ToolSpec)
from inference_b200.engine.provider import CPU_LLAMA, LlamaProvider
from inference_b200.io import prepare as prep
from inference_b200.io.gguf import GgufCheckpoint, gguf_architecture
from inference_b200.io.safetensors_io import load_dir
from inference_b200.testkit import synthetic
from inference_b200.testkit.textllm import (BROKEN_FAULTS, ConformanceFailure, StubTextLlm, TextLlmProfile,
                                            check_snapshot_preparer, textllm_conformance)


def test_stub_passes_and_broken_stubs_fail():
    textllm_conformance(lambda: StubTextLlm())
    for fault in BROKEN_FAULTS:
        with pytest.raises(ConformanceFailure):
            textllm_conformance(lambda f=fault: StubTextLlm(f))


@pytest.fixture(scope="module")
def snapshot(tmp_path_factory):
    return synthetic.write_snapshot(tmp_path_factory.mktemp("snap"))


def test_cpu_provider_conformance(snapshot):
    reg = TextLlmRegistryBuilder().register(CPU_LLAMA).build()
    p = reg.load_for_model(LoadSpec.dense(str(snapshot)))
    assert p.descriptor().id == "cpu-llama" and p.descriptor().backend == "cpu"
    textllm_conformance(lambda: p, TextLlmProfile(prompt="hello world"))


def test_stop_strings_and_usage(snapshot):
    p = LlamaProvider.load(LoadSpec.dense(str(snapshot)), "cpu-llama", "cpu")
    req = TextLlmRequest([Message.system("the cat"), Message.user("hello")], 12, Sampling.greedy())
    full = p.complete(req)
    assert full.usage.generated_tokens >= 1 and full.usage.prompt_tokens > 4
    words = full.text.split()
    if len(words) >= 3:
        req2 = TextLlmRequest(req.messages, 12, Sampling.greedy(), stop=[words[2]])
        cut = p.complete(req2)
        assert words[2] not in cut.text and cut.text.strip() == " ".join(words[:2]).strip() or cut.text in full.text


def test_json_constraint_yields_valid_json_prefix(snapshot):
    p = LlamaProvider.load(LoadSpec.dense(str(snapshot)), "cpu-llama", "cpu")
    req = TextLlmRequest([Message.user("hello")], 24, Sampling.greedy(), constraint=Constraint.JSON)
    out = p.complete(req)
    from inference_b200.contracts.core_llm import JsonState

    st = JsonState.start()
    assert st.advance_str(out.text.replace(" ", "")) or st.advance_str(out.text)
    if out.finish_reason is FinishReason.STOP:
        json.loads(out.text)


def test_thinking_and_tools_template(tmp_path):
    tpl = ("{% for m in messages %}<|start_header_id|> {{ m.role }} <|end_header_id|> {{ m.content }} <|eot_id|> "
           "{% endfor %}{% if tools %}tool_call {% endif %}{% if enable_thinking is defined %}{% endif %}"
           "<|start_header_id|> assistant <|end_header_id|> ")
    snap = synthetic.write_snapshot(tmp_path / "t", chat_template=tpl)
    p = LlamaProvider.load(LoadSpec.dense(str(snap)), "cpu-llama", "cpu")
    caps = p.descriptor().capabilities
    assert caps.supports_thinking and caps.supports_tools
    textllm_conformance(lambda: p, TextLlmProfile(prompt="hello"))


def test_quantize_on_load_changes_weights_but_runs(snapshot):
    dense = LlamaProvider.load(LoadSpec.dense(str(snapshot)), "cpu-llama", "cpu")
    q8 = LlamaProvider.load(LoadSpec(str(snapshot), Quantize.Q8), "cpu-llama", "cpu")
    wd = dense.backend.model.w["model.layers.0.self_attn.q_proj.weight"]
    wq = q8.backend.model.w["model.layers.0.self_attn.q_proj.weight"]
    assert not torch.equal(wd, wq) and (wd - wq).abs().max() < 0.02
    assert q8.complete(TextLlmRequest([Message.user("hello")], 4, Sampling.greedy())).usage.generated_tokens >= 1


def test_gguf_roundtrip_and_preparer(snapshot, tmp_path):
    gg = synthetic.write_gguf_from_snapshot(snapshot, tmp_path / "m.gguf", "Q8_0")
    assert gguf_architecture(gg) == "llama"
    ck = GgufCheckpoint(gg)
    ref = load_dir(snapshot)
    got = ck.tensors()
    assert set(got) == set(ref)
    for k in ref:
        assert (got[k] - ref[k].float()).abs().max() < 0.02, k   # Q8_0 error; q/k un-permute restores HF order
    assert ck.config()["num_attention_heads"] == 4
    regs = SnapshotPreparerRegistryBuilder().register(prep.registration("cpu")).build()
    assert check_snapshot_preparer(regs, gg, tmp_path / "from_gguf", ModelFormat.GGUF) is None
    assert check_snapshot_preparer(regs, snapshot, tmp_path / "from_hf", ModelFormat.SAFETENSORS) is None
    rep = regs.prepare_snapshot(PrepareSpec.quantized(snapshot, tmp_path / "q4", Quantize.Q8))
    assert not rep.passthrough and json.loads((tmp_path / "q4" / "config.json").read_text())["quantization"] == {"bits": 8}
    reloaded = LlamaProvider.load(LoadSpec.dense(str(tmp_path / "from_hf")), "cpu-llama", "cpu")
    a = reloaded.complete(TextLlmRequest([Message.user("hello")], 6, Sampling.greedy()))
    b = LlamaProvider.load(LoadSpec.dense(str(snapshot)), "cpu-llama", "cpu").complete(
        TextLlmRequest([Message.user("hello")], 6, Sampling.greedy()))
    assert a.text == b.text
