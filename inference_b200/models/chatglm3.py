"""ChatGLM3-6B as the Kolors prompt encoder (parity: candle-gen-kolors/src/chatglm3.rs, tokenizer.rs).

The network is the GLM decoder (RMSNorm, q/k/v bias, multi-query attention, rotary on the first half of every head in
interleaved pairs, SwiGLU) under its original tensor names: fused `query_key_value`, fused `dense_h_to_4h`. The
checkpoint is renamed and split into the standard projections and then runs on the oracle decoder.

Kolors pads prompts on the LEFT to 256 tokens. Real tokens see the real tokens before them (positions count from the
first real token); the padding rows see every position, and their states are still part of the cross-attention context.
The context is the input of the last layer (all 256 rows), the pooled vector is the last layer's output at the final
token, both without the final norm."""
from __future__ import annotations

import torch

from .config import ModelConfig

GMASK_OFFSET, SOP_OFFSET = 1, 3          # "[gMASK]" and "sop" follow the SentencePiece vocabulary ([MASK], [gMASK], [sMASK], sop)
PROMPT_TOKENS = 256


def glm_config_from_chatglm(j: dict) -> ModelConfig:
    heads = int(j["num_attention_heads"])
    hd = int(j.get("kv_channels", j["hidden_size"] // heads))
    return ModelConfig.from_json({
        "architectures": ["GlmForCausalLM"], "model_type": "glm", "hidden_size": j["hidden_size"],
        "intermediate_size": j["ffn_hidden_size"], "num_hidden_layers": j["num_layers"], "num_attention_heads": heads,
        "num_key_value_heads": j.get("multi_query_group_num", heads) if j.get("multi_query_attention", True) else heads,
        "head_dim": hd, "vocab_size": j.get("padded_vocab_size", j.get("vocab_size")),
        "rms_norm_eps": j.get("layernorm_epsilon", 1e-5), "rope_theta": 10000.0 * float(j.get("rope_ratio", 1.0)),
        "partial_rotary_factor": 0.5, "max_position_embeddings": j.get("seq_length", 8192), "tie_word_embeddings": False})


def glm_weights_from_chatglm(sd: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    out = {}
    q_rows, kv_rows = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    for k, v in sd.items():
        k = k[len("transformer."):] if k.startswith("transformer.") else k
        if k == "embedding.word_embeddings.weight":
            out["model.embed_tokens.weight"] = v
        elif k == "encoder.final_layernorm.weight":
            out["model.norm.weight"] = v
        elif k == "output_layer.weight":
            out["lm_head.weight"] = v
        elif k.startswith("encoder.layers."):
            n, rest = k[len("encoder.layers."):].split(".", 1)
            p = f"model.layers.{n}."
            if rest.startswith("self_attention.query_key_value."):
                leaf = rest.rsplit(".", 1)[1]
                for name, t in zip("qkv", (v[:q_rows], v[q_rows:q_rows + kv_rows], v[q_rows + kv_rows:])):
                    out[f"{p}self_attn.{name}_proj.{leaf}"] = t
            elif rest == "self_attention.dense.weight":
                out[p + "self_attn.o_proj.weight"] = v
            elif rest == "mlp.dense_h_to_4h.weight":
                half = v.shape[0] // 2
                out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = v[:half], v[half:]
            elif rest == "mlp.dense_4h_to_h.weight":
                out[p + "mlp.down_proj.weight"] = v
            elif rest in ("input_layernorm.weight", "post_attention_layernorm.weight"):
                out[p + rest] = v
    return out


def chatglm_from_glm_weights(sd: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    """The inverse renaming (synthetic snapshots and tests)."""
    out = {"transformer.embedding.word_embeddings.weight": sd["model.embed_tokens.weight"],
           "transformer.encoder.final_layernorm.weight": sd["model.norm.weight"],
           "transformer.output_layer.weight": sd.get("lm_head.weight", sd["model.embed_tokens.weight"])}
    for i in range(cfg.num_layers):
        p, q = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        for leaf in ("weight", "bias"):
            if f"{p}self_attn.q_proj.{leaf}" in sd:
                out[f"{q}self_attention.query_key_value.{leaf}"] = torch.cat([sd[f"{p}self_attn.{n}_proj.{leaf}"] for n in "qkv"], 0)
        out[q + "self_attention.dense.weight"] = sd[p + "self_attn.o_proj.weight"]
        out[q + "mlp.dense_h_to_4h.weight"] = torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]], 0)
        out[q + "mlp.dense_4h_to_h.weight"] = sd[p + "mlp.down_proj.weight"]
        out[q + "input_layernorm.weight"] = sd[p + "input_layernorm.weight"]
        out[q + "post_attention_layernorm.weight"] = sd[p + "post_attention_layernorm.weight"]
    return out


def left_padded_mask(total: int, real: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """(additive mask [1, 1, total, total], positions [1, total]) for `real` tokens behind total - real padding rows:
    real rows see real rows up to themselves, padding rows see everything; positions count from the first real token
    and are 0 on the padding."""
    pad = total - real
    i = torch.arange(total, device=device)
    allowed = (i[None, :] <= i[:, None]) & (i[None, :] >= pad)
    allowed[:pad] = True
    mask = torch.zeros(total, total, device=device).masked_fill(~allowed, float("-inf"))
    return mask[None, None], (i - pad).clamp(min=0)[None]


class ChatGlm3PromptEncoder:
    def __init__(self, config_json: dict, weights: dict[str, torch.Tensor], sp_model, device="cpu", dtype=torch.float32,
                 tokens: int = PROMPT_TOKENS):
        from .oracle import OracleLlama

        self.cfg = glm_config_from_chatglm(config_json)
        self.model = OracleLlama(self.cfg, glm_weights_from_chatglm(weights, self.cfg), dtype, device)
        self.sp, self.tokens = sp_model, tokens

    def token_ids(self, prompt: str) -> list[int]:
        n = self.sp.vocab_size()
        return ([n + GMASK_OFFSET, n + SOP_OFFSET] + self.sp.encode(prompt))[: self.tokens]

    @torch.no_grad()
    def encode(self, prompt: str) -> tuple[torch.Tensor, torch.Tensor]:
        """(context [1, tokens, hidden], pooled [1, hidden])."""
        ids = self.token_ids(prompt)
        real = len(ids)
        padded = torch.tensor([[0] * (self.tokens - real) + ids], dtype=torch.int64)
        mask, pos = left_padded_mask(self.tokens, real, self.model.device)
        L = self.cfg.num_layers
        penult = self.model.hidden_states(padded, None, positions=pos, additive_mask=mask, num_layers=L - 1)
        last = self.model.hidden_states(padded, None, positions=pos, additive_mask=mask)
        return penult, last[:, -1]
