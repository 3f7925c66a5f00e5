"""The fp32 oracle decoder against the Hugging Face implementations of each architecture on tiny random models: the
oracle is what every GPU test compares with, so it has to agree with an independent implementation."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from inference_b200.models import ModelConfig  # noqa: E402
from inference_b200.models.oracle import OracleLlama  # noqa: E402

BASE = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
            tie_word_embeddings=False, attention_dropout=0.0)

CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", {}),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=None)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", {}),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=32)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(pad_token_id=0)),
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM", dict(head_dim=16, query_pre_attn_scalar=16, attn_logit_softcapping=50.0,
                                                         final_logit_softcapping=30.0, sliding_window=4096,
                                                         hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)),
    "glm": ("GlmConfig", "GlmForCausalLM", dict(head_dim=16, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0)),
    "glm4": ("Glm4Config", "Glm4ForCausalLM", dict(head_dim=16, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0)),
    "qwen2_moe": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                                                shared_expert_intermediate_size=80, norm_topk_prob=False,
                                                                decoder_sparse_step=1, mlp_only_layers=[])),
    "deepseek_v2": ("DeepseekV2Config", "DeepseekV2ForCausalLM", dict(
        kv_lora_rank=16, q_lora_rank=24, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=12, n_routed_experts=4,
        n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=40, first_k_dense_replace=1,
        routed_scaling_factor=1.0, topk_method="greedy", norm_topk_prob=False, num_key_value_heads=4, head_dim=8)),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_hugging_face(name):
    cfg_cls, model_cls, extra = CASES[name]
    if not hasattr(transformers, model_cls):
        pytest.skip(f"{model_cls} not in this transformers build")
    torch.manual_seed(0)
    hf_cfg = getattr(transformers, cfg_cls)(**{**BASE, **extra})
    hf_cfg._attn_implementation = "eager"
    hf = getattr(transformers, model_cls)(hf_cfg).eval().float()
    with torch.no_grad():
        for p_ in hf.parameters():            # spread the random init so norms and biases matter
            p_.add_(torch.randn_like(p_) * 0.02)
    cfg = ModelConfig.from_json(hf_cfg.to_dict())
    oracle = OracleLlama(cfg, dict(hf.state_dict()), dtype=torch.float32)
    ids = torch.randint(0, 128, (2, 21))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits
    got = oracle.decode_logits_all(ids, None, 0)
    err = (got - ref).abs().max().item()
    assert err < 2e-4 * max(1.0, ref.abs().max().item()), (name, err)
    # incremental decoding through the KV cache gives the same last-position logits
    cache = oracle.make_cache()
    oracle.decode_logits(ids[:, :15], cache, 0)
    step = oracle.decode_logits(ids[:, 15:], cache, 15)
    assert (step - ref[:, -1]).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
