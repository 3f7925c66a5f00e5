"""T5 / CLIP text encoders against the Hugging Face implementations on tiny random configurations."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def test_t5_encoder_matches_transformers():
    from transformers import T5Config as HfCfg
    from transformers import T5EncoderModel

    from inference_b200.models.text_encoders import T5Config, T5Encoder

    torch.manual_seed(0)
    hf_cfg = HfCfg(vocab_size=100, d_model=64, d_kv=16, d_ff=128, num_layers=3, num_heads=4, feed_forward_proj="gated-gelu",
                   relative_attention_num_buckets=8, relative_attention_max_distance=20, dropout_rate=0.0)
    hf = T5EncoderModel(hf_cfg).eval()
    cfg = T5Config(vocab_size=100, d_model=64, d_kv=16, d_ff=128, num_layers=3, num_heads=4,
                   relative_attention_num_buckets=8, relative_attention_max_distance=20)
    mine = T5Encoder(cfg, dict(hf.state_dict()))
    ids = torch.randint(0, 100, (2, 37))
    with torch.no_grad():
        ref = hf(input_ids=ids).last_hidden_state
    out = mine.encode(ids)
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4), (out - ref).abs().max()
    mask = torch.ones(2, 37, dtype=torch.long)
    mask[1, 20:] = 0
    with torch.no_grad():
        ref_m = hf(input_ids=ids, attention_mask=mask).last_hidden_state
    assert torch.allclose(mine.encode(ids, mask)[1, :20], ref_m[1, :20], atol=2e-5, rtol=1e-4)


def test_clip_text_encoder_matches_transformers():
    from transformers import CLIPTextConfig, CLIPTextModel

    from inference_b200.models.text_encoders import ClipTextConfig, ClipTextEncoder

    torch.manual_seed(1)
    hf_cfg = CLIPTextConfig(vocab_size=120, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                            num_attention_heads=4, max_position_embeddings=20, eos_token_id=119, bos_token_id=118,
                            hidden_act="quick_gelu")
    hf = CLIPTextModel(hf_cfg).eval()
    cfg = ClipTextConfig(vocab_size=120, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, max_position_embeddings=20, eos_token_id=119)
    mine = ClipTextEncoder(cfg, dict(hf.state_dict()))
    ids = torch.randint(0, 118, (3, 20))
    ids[:, 0] = 118
    for b, e in enumerate((7, 19, 12)):
        ids[b, e:] = 119
    with torch.no_grad():
        ref = hf(input_ids=ids)
    hidden, pooled = mine.encode(ids)
    assert torch.allclose(hidden, ref.last_hidden_state, atol=2e-5, rtol=1e-4)
    assert torch.allclose(pooled, ref.pooler_output, atol=2e-5, rtol=1e-4)
