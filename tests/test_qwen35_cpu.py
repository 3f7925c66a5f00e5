"""Qwen3.5 hybrid decoder (Gated DeltaNet + gated full attention) against Hugging Face on a tiny random config."""
import pytest
import torch


def _tiny():
    from transformers import Qwen3_5ForCausalLM, Qwen3_5TextConfig

    torch.manual_seed(0)
    hc = Qwen3_5TextConfig(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=32, linear_num_value_heads=4,
                           linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
                           linear_conv_kernel_dim=4, max_position_embeddings=256, tie_word_embeddings=False,
                           layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])
    hf = Qwen3_5ForCausalLM(hc).eval()
    with torch.no_grad():                       # zero-initialised norm weights / unit dt_bias hide mistakes: randomise
        for n, p in hf.named_parameters():
            if n.endswith(("norm.weight", "layernorm.weight", "dt_bias")):
                p.copy_(torch.randn_like(p) * 0.2)
    return hc, hf


def test_gated_delta_primitives():
    from inference_b200.models import qwen35 as q

    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 7, 6, generator=g)
    w = torch.randn(6, 4, generator=g)
    y, st = q.causal_depthwise_conv(x, w, None)
    ref = torch.nn.functional.silu(torch.nn.functional.conv1d(torch.nn.functional.pad(x.transpose(1, 2), (3, 0)),
                                                              w.unsqueeze(1), groups=6)).transpose(1, 2)
    torch.testing.assert_close(y, ref)
    assert torch.equal(st, x[:, -3:])
    # streaming the sequence in two pieces through the state equals one pass
    y1, s1 = q.causal_depthwise_conv(x[:, :3], w, None)
    y2, s2 = q.causal_depthwise_conv(x[:, 3:], w, s1)
    torch.testing.assert_close(torch.cat([y1, y2], 1), y)
    B, T, H, dk, dv = 2, 6, 3, 8, 5
    qq, kk = torch.randn(B, T, H, dk, generator=g), torch.randn(B, T, H, dk, generator=g)
    vv, gg = torch.randn(B, T, H, dv, generator=g), -torch.rand(B, T, H, generator=g)
    bb = torch.rand(B, T, H, generator=g)
    o, S = q.gated_delta_recurrence(qq, kk, vv, gg, bb, None)
    o1, S1 = q.gated_delta_recurrence(qq[:, :2], kk[:, :2], vv[:, :2], gg[:, :2], bb[:, :2], None)
    o2, S2 = q.gated_delta_recurrence(qq[:, 2:], kk[:, 2:], vv[:, 2:], gg[:, 2:], bb[:, 2:], S1)
    torch.testing.assert_close(torch.cat([o1, o2], 1), o)
    torch.testing.assert_close(S2, S)
    # with beta = 1 and no decay the state stores v exactly for an (L2-normalised) key
    o, S = q.gated_delta_recurrence(kk[:, :1], kk[:, :1], vv[:, :1], torch.zeros(B, 1, H), torch.ones(B, 1, H), None)
    torch.testing.assert_close(o[:, 0] * dk ** 0.5, vv[:, 0], atol=1e-4, rtol=1e-4)
    n = q.rms_norm_gated(torch.ones(1, 4), torch.full((4,), 2.0), torch.zeros(1, 4), 0.0)
    assert float(n.abs().max()) == 0.0                                   # SiLU(0) = 0 closes the gate
    a = q.compute_g(torch.zeros(3), torch.zeros(3), torch.zeros(3))
    torch.testing.assert_close(a, torch.full((3,), -torch.log(torch.tensor(2.0)).item()))


def test_qwen35_matches_hugging_face_prefill_and_cached_decode():
    from inference_b200.models.config import Architecture, ModelConfig
    from inference_b200.models.qwen35 import Qwen35Config, Qwen35Model

    hc, hf = _tiny()
    d = hc.to_dict()
    assert Architecture.from_config({"model_type": "qwen3_5_text", "architectures": ["Qwen3_5ForCausalLM"]}) is Architecture.QWEN35
    cfg = Qwen35Config.from_json(d)
    assert cfg.layer_types[-1] == "full_attention" and cfg.is_linear(0) and cfg.rotary_dim == 8
    model = Qwen35Model(cfg, dict(hf.state_dict()))
    ids = torch.randint(0, 160, (1, 11), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits
    torch.testing.assert_close(model.decode_logits_all(ids, None), ref, atol=3e-4, rtol=3e-4)
    # prefill 7 tokens, then decode the remaining 4 one at a time through the caches
    cache = model.make_cache()
    lg = model.decode_logits(ids[:, :7], cache, 0)
    torch.testing.assert_close(lg, ref[:, 6], atol=3e-4, rtol=3e-4)
    for t in range(7, 11):
        lg = model.decode_logits(ids[:, t:t + 1], cache, cache.offset)
        torch.testing.assert_close(lg, ref[:, t], atol=5e-4, rtol=5e-4)
    assert cache.offset == 11
    fork = cache.clone()
    fork.truncate(11)
    with pytest.raises(Exception):
        fork.truncate(5)
    fork.truncate(0)
    assert fork.offset == 0 and cache.offset == 11
    with torch.no_grad():
        want = hf.generate(input_ids=ids, max_new_tokens=5, do_sample=False)[0, 11:].tolist()
    got, _ = model.generate_greedy(ids[0].tolist(), 5)
    assert got == want
    interval = Qwen35Config.from_json({**{k: v for k, v in d.items() if k != "layer_types"}, "full_attention_interval": 2})
    assert interval.layer_types == ["linear_attention", "full_attention"] * 2


def test_qwen35_snapshot_loads_through_the_text_registry(tmp_path):
    import json

    from inference_b200.bundles import runtime_cpu
    from inference_b200.contracts.core_llm import LoadSpec, Message, TextLlmRequest
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json

    hc, hf = _tiny()
    cfg_json = {**hc.to_dict(), "architectures": ["Qwen3_5ForCausalLM"], "model_type": "qwen3_5_text"}
    (tmp_path / "config.json").write_text(json.dumps(cfg_json))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    (tmp_path / "tokenizer.json").write_text(wordlevel_tokenizer_json(160))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<|begin_of_text|>", "eos_token": "<|eot_id|>"}))
    llm = runtime_cpu.catalog().text().load_for_model(LoadSpec.dense(str(tmp_path)))
    events = []
    out = llm.generate(TextLlmRequest(messages=[Message.user("t5 t6 t7")], max_new_tokens=6, seed=0), on_event=events.append)
    assert out.usage.generated_tokens >= 1 and len(events) >= 2
    again = llm.generate(TextLlmRequest(messages=[Message.user("t5 t6 t7")], max_new_tokens=6, seed=0), on_event=lambda e: None)
    assert again.text == out.text
