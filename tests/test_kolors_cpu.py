"""Kolors: the ChatGLM3 checkpoint renaming against Hugging Face GLM, the left-padding attention rule, the UNet's text
projection, provider conformance."""
import pytest
import torch

from inference_b200.models import chatglm3 as G

transformers = pytest.importorskip("transformers")


def test_chatglm_renaming_reproduces_hugging_face_glm():
    from transformers import GlmConfig, GlmForCausalLM

    from inference_b200.models.oracle import OracleLlama

    hc = GlmConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0,
                   rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = GlmForCausalLM(hc).eval()
    sd = {k: v for k, v in hf.state_dict().items()}
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import canonical_weights

    base_cfg = ModelConfig.from_json(hc.to_dict() | {"architectures": ["GlmForCausalLM"]})
    chat = G.chatglm_from_glm_weights(canonical_weights(sd, base_cfg), base_cfg)
    assert "transformer.encoder.layers.0.self_attention.query_key_value.weight" in chat
    cj = {"num_layers": 3, "hidden_size": 64, "ffn_hidden_size": 96, "num_attention_heads": 4, "multi_query_attention": True,
          "multi_query_group_num": 2, "kv_channels": 16, "padded_vocab_size": 128, "layernorm_epsilon": 1e-5, "seq_length": 128}
    cfg = G.glm_config_from_chatglm(cj)
    assert (cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_size, cfg.architecture.value) == (2, 16, 96, "glm")
    oracle = OracleLlama(cfg, G.glm_weights_from_chatglm(chat, cfg))
    ids = torch.tensor([[5, 9, 33, 2, 71, 8]])
    with torch.no_grad():
        ref = hf(ids, output_hidden_states=True)
    torch.testing.assert_close(oracle.decode_logits_all(ids, None, 0), ref.logits, atol=2e-5, rtol=1e-4)
    # left padding: the real tokens' states equal the un-padded run (padding is invisible to them)
    mask, pos = G.left_padded_mask(10, 6)
    assert pos.tolist() == [[0, 0, 0, 0, 0, 1, 2, 3, 4, 5]]
    assert mask[0, 0, 7].isinf().tolist() == [True] * 4 + [False] * 4 + [True] * 2 and not mask[0, 0, :4].isinf().any()
    padded = torch.cat([torch.zeros(1, 4, dtype=torch.long), ids], 1)
    h = oracle.hidden_states(padded, None, positions=pos, additive_mask=mask, num_layers=2)
    torch.testing.assert_close(h[:, 4:], ref.hidden_states[2], atol=2e-5, rtol=1e-4)


def test_kolors_provider_conforms(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.kolors import KolorsPipeline, write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    ms = KolorsPipeline.model_sampling()
    betas = torch.linspace(0.00085 ** 0.5, 0.014 ** 0.5, 1100, dtype=torch.float64) ** 2
    acp = torch.cumprod(1 - betas, 0)[-1].item()
    assert ms.num_timesteps() == 1100 and abs(ms.sigma_max() - ((1 - acp) / acp) ** 0.5) < 1e-6 * ms.sigma_max()
    d = KolorsPipeline.default_unet_config()
    assert (d.encoder_hid_dim, d.projection_class_embeddings_input_dim, d.cross_attention_dim) == (4096, 5632, 2048)
    snap = write_synthetic_snapshot(tmp_path / "kolors", text="chatglm")
    reg = provider_registry("cpu")
    assert "cpu_kolors" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_kolors", LoadSpec.from_dir(snap))
    kit.conformance(gen, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_kolors", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = gen.generate(GenerationRequest(**req, guidance=1.0)).images[0].pixels
    b = gen.generate(GenerationRequest(**req)).images[0].pixels
    c = gen.generate(GenerationRequest(**req, guidance=5.0, negative_prompt="", sampler="euler")).images[0].pixels
    assert b == c and a != b and len(a) == 256 * 256 * 3
    # the prompt encoder: 256 context rows, the prefix tokens follow the SentencePiece vocabulary
    text = gen.pipe.load_text()
    ids = text.encoder.token_ids("a red fox")
    n = text.encoder.sp.vocab_size()
    assert ids[:2] == [n + 1, n + 3] and len(ids) > 2
    cond = text.encode("a red fox")
    assert cond.context.shape == (1, 256, 64) and cond.pooled.shape == (1, 64)
