"""Llama-family decoder on sm_100a kernels with a paged KV cache and tensor parallelism.

The capability target is the reference's generic `CausalLm` (candle-llm/src/models/llama.rs:31-1488):
config-dispatched Llama / Mistral / Qwen2 / Qwen3 / Phi-3 / Gemma-2 / GLM-4 decoders. The execution
design differs: weights are stored in tensor-parallel layout (column-parallel fused QKV and gate/up,
row-parallel o_proj and down_proj, vocab-parallel head) even at P = 1, every projection is a tcgen05
GEMM, norms / RoPE / KV writes / activations are fused kernels, attention reads the paged cache through
the block table, and one step consumes a flat ragged token batch so prefill, chunked prefill, decode and
speculative verify all share one forward.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .. import ops
from ..contracts.errors import LoadError, Unsupported
from ..parallel.comm import Communicator, single
from .config import Architecture, ModelConfig, build_rope
from .oracle import canonical_weights


@dataclass
class StepInputs:
    """One engine step over a flat token batch (all tensors on the model's device)."""
    input_ids: torch.Tensor            # int64 [T]
    positions: torch.Tensor            # int32 [T]
    slot_mapping: torch.Tensor         # int64 [T] flat cache slot per token (-1 = do not cache)
    block_table: torch.Tensor          # int32 [num_seqs, max_blocks]
    kv_lens: torch.Tensor              # int32 [num_seqs] context length including this step's tokens
    cu_q: torch.Tensor | None          # int32 [num_seqs + 1]; None => every sequence has max_q_len tokens
    max_q_len: int
    num_seqs: int
    decode: bool = False               # q_len * gqa_group <= 16 for every sequence
    attn_splits: int = 1
    logits_rows: torch.Tensor | None = None  # int64 rows of the hidden state to project; None => all rows
    fresh_prefill: bool = False        # every sequence starts at position 0 (context == this step's tokens)
    embed_rows: torch.Tensor | None = None    # int64 [R]: rows of the flat batch whose embedding is replaced ...
    embed_values: torch.Tensor | None = None  # ... by these [R, H] vectors (projected image features of a VLM prompt)
    rope_table: tuple[torch.Tensor, torch.Tensor] | None = None   # fp32 cos / sin [T, rot_dim / 2], one row per token of
    #                                           this step: replaces the position-indexed table (three-axis rotary phases)
    deepstack: tuple[torch.Tensor, list[torch.Tensor]] | None = None   # (int64 rows [R], taps): taps[l] [R, H] is added
    #                                           to the residual stream at those rows after decoder layer l (Qwen3-VL)


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    qkv: torch.Tensor
    qkv_bias: torch.Tensor | None
    q_norm: torch.Tensor | None
    k_norm: torch.Tensor | None
    o: torch.Tensor
    post_attn_ln: torch.Tensor | None   # sandwich: norm of the attention output
    ln2: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor
    post_mlp_ln: torch.Tensor | None    # sandwich: norm of the MLP output
    moe: "MoeWeights | None" = None     # sparse FFN (then gate_up / down are unused)


@dataclass
class MoeWeights:
    """Top-k routed experts with an optional (sigmoid-gated) shared expert (Qwen2-MoE: candle-llm models/llama.rs
    MoE FFN). Expert FFNs are sharded like the dense one: gate/up by rows, down by columns."""
    router: torch.Tensor                      # [E, H], replicated
    gate_up: torch.Tensor                     # [E, 2 * F_local, H] (stacked: the grouped GEMM indexes experts by row)
    down: torch.Tensor                        # [E, H, F_local]
    shared_gate_up: torch.Tensor | None
    shared_down: torch.Tensor | None
    shared_gate: torch.Tensor | None          # [1, H]


def _shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def _shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n]


class LlamaGpu:
    def __init__(self, cfg: ModelConfig, comm: Communicator | None = None, device: torch.device | None = None):
        if cfg.mla is not None or cfg.architecture is Architecture.QWEN35:
            raise Unsupported(f"{cfg.architecture.value}: served by the fp32 oracle path, not the sm_100a decoder")
        if cfg.head_dim != 128:
            raise Unsupported("the sm_100a attention kernels are built for head_dim 128")
        self.cfg = cfg
        self.comm = comm or single(device)
        self.device = device or self.comm.device
        P = self.comm.world
        if cfg.num_heads % P or cfg.num_kv_heads % P or cfg.intermediate_size % P or cfg.vocab_size % P:
            raise Unsupported(f"tensor parallel degree {P} does not divide heads/kv-heads/ffn/vocab")
        self.hq = cfg.num_heads // P
        self.hkv = cfg.num_kv_heads // P
        self.ffn = cfg.intermediate_size // P
        self.vocab_local = cfg.vocab_size // P
        self.layers: list[LayerWeights] = []
        self.embed: torch.Tensor | None = None      # full table on every rank (gather is local)
        self.norm: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None    # [vocab / P, hidden]
        rope = build_rope(cfg)
        self.rot_dim, self.rope_interleaved = rope.dim, rope.interleaved
        self._inv_freq = torch.tensor(rope.inv_freq, dtype=torch.float64)
        self.cos = self.sin = None
        self.max_positions = 0
        pending = getattr(self.comm, "_fused_pending", None)
        if pending and self.comm.fused is None:
            from ..parallel.symm import attach_fused

            attach_fused(self.comm, cfg.hidden_size, pending)
        self.launches = 0  # kernels launched by the last forward (for accounting)

    # ---- weights --------------------------------------------------------------------------------
    def ensure_rope(self, max_positions: int) -> None:
        if max_positions <= self.max_positions:
            return
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * self._inv_freq[None, :]
        self.cos = ang.cos().float().to(self.device).contiguous()
        self.sin = ang.sin().float().to(self.device).contiguous()
        self.max_positions = max_positions

    def load_state_dict(self, weights: dict[str, torch.Tensor], *, layers: range | None = None,
                        with_embed: bool = True, with_head: bool = True) -> "LlamaGpu":
        """Takes full (unsharded) HF-named tensors and keeps this rank's tensor-parallel slice in bf16. `layers`
        restricts the load to a contiguous block of decoder layers (one pipeline stage); a stage that is not the first
        / last skips the embedding table / the final norm and output head."""
        cfg, r, P, dev = self.cfg, self.comm.rank, self.comm.world, self.device
        w = canonical_weights(weights, cfg)
        D = cfg.head_dim

        def get(k: str) -> torch.Tensor:
            if k not in w:
                raise LoadError(f"missing tensor {k}")
            return w[k]

        def dev16(t: torch.Tensor) -> torch.Tensor:
            return t.to(device=dev, dtype=torch.bfloat16).contiguous()

        if with_embed:
            self.embed = dev16(get("model.embed_tokens.weight"))
        if with_head:
            self.norm = dev16(get("model.norm.weight"))
            head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
            self.lm_head = dev16(_shard_rows(head, r, P))
        self.layers = []
        for i in (layers if layers is not None else range(cfg.num_layers)):
            p = f"model.layers.{i}"
            q = _shard_rows(get(f"{p}.self_attn.q_proj.weight"), r, P)
            k = _shard_rows(get(f"{p}.self_attn.k_proj.weight"), r, P)
            v = _shard_rows(get(f"{p}.self_attn.v_proj.weight"), r, P)
            qkv_bias = None
            if f"{p}.self_attn.q_proj.bias" in w:
                qkv_bias = dev16(torch.cat([_shard_rows(get(f"{p}.self_attn.{n}_proj.bias"), r, P) for n in "qkv"]))
            moe = None
            if f"{p}.mlp.gate.weight" in w:
                E = cfg.moe.num_experts

                def gu(prefix):
                    return dev16(torch.cat([_shard_rows(get(f"{prefix}.gate_proj.weight"), r, P),
                                            _shard_rows(get(f"{prefix}.up_proj.weight"), r, P)]))
                has_shared = f"{p}.mlp.shared_expert.gate_proj.weight" in w
                sg = w.get(f"{p}.mlp.shared_expert_gate.weight")
                moe = MoeWeights(
                    router=dev16(get(f"{p}.mlp.gate.weight")),
                    gate_up=torch.stack([gu(f"{p}.mlp.experts.{e}") for e in range(E)]).contiguous(),
                    down=torch.stack([dev16(_shard_cols(get(f"{p}.mlp.experts.{e}.down_proj.weight"), r, P))
                                      for e in range(E)]).contiguous(),
                    shared_gate_up=gu(f"{p}.mlp.shared_expert") if has_shared else None,
                    shared_down=dev16(_shard_cols(get(f"{p}.mlp.shared_expert.down_proj.weight"), r, P))
                    if has_shared else None,
                    shared_gate=dev16(torch.cat([sg, torch.zeros(7, sg.shape[1])])) if sg is not None else None)
                gate = up = torch.zeros(8, cfg.hidden_size)
                w[f"{p}.mlp.down_proj.weight"] = torch.zeros(cfg.hidden_size, 8 * P)
            else:
                gate = _shard_rows(get(f"{p}.mlp.gate_proj.weight"), r, P)
                up = _shard_rows(get(f"{p}.mlp.up_proj.weight"), r, P)
            arch = cfg.architecture
            if arch is Architecture.GEMMA2:
                post_attn, ln2, post_mlp = (get(f"{p}.post_attention_layernorm.weight"),
                                            get(f"{p}.pre_feedforward_layernorm.weight"),
                                            get(f"{p}.post_feedforward_layernorm.weight"))
            elif arch is Architecture.GLM4:
                post_attn, ln2, post_mlp = (get(f"{p}.post_self_attn_layernorm.weight"),
                                            get(f"{p}.post_attention_layernorm.weight"),
                                            get(f"{p}.post_mlp_layernorm.weight"))
            else:
                post_attn, ln2, post_mlp = None, get(f"{p}.post_attention_layernorm.weight"), None
            qn = w.get(f"{p}.self_attn.q_norm.weight")
            kn = w.get(f"{p}.self_attn.k_norm.weight")
            self.layers.append(LayerWeights(
                ln1=dev16(get(f"{p}.input_layernorm.weight")), qkv=dev16(torch.cat([q, k, v])), qkv_bias=qkv_bias,
                q_norm=dev16(qn) if qn is not None else None, k_norm=dev16(kn) if kn is not None else None,
                o=dev16(_shard_cols(get(f"{p}.self_attn.o_proj.weight"), r, P)),
                post_attn_ln=dev16(post_attn) if post_attn is not None else None, ln2=dev16(ln2),
                gate_up=dev16(torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], -1)), down=dev16(_shard_cols(get(f"{p}.mlp.down_proj.weight"), r, P)),
                post_mlp_ln=dev16(post_mlp) if post_mlp is not None else None, moe=moe))
        assert D == 128
        self.fold_norms()
        return self

    def fold_norms(self) -> bool:
        """Multiply each layer's input / post-attention norm weight into the projection that consumes it (qkv,
        gate_up) and leave a unit norm weight behind. The model computes the same function; decode-sized steps can
        then skip the norm kernels: the o / down projections add the residual and emit per-token sums of squares in
        their epilogues and the qkv / gate_up projections scale their accumulators by 1 / rms
        (`ops.gemm_bf16_normed`). Under tensor parallelism the o / down epilogues also sum the ranks' partial products
        over peer memory (`FusedCollectives.gemm_peer_reduce`), so a sharded decode step launches the same six kernels
        per layer as an unsharded one. Only for dense layers without sandwich norms; a sharded model needs the
        peer-memory collectives (the library all-reduce path keeps its norm kernels)."""
        if self.norm_folded or os.environ.get("SWB_FOLD_NORMS", "1") == "0":
            return False
        if self.comm.is_parallel and (self.comm.fused is None or os.environ.get("SWB_TP_CHAIN", "1") == "0"):
            return False
        woff = self.cfg.norm_weight_offset
        for L in self.layers:
            if (L.moe is not None or L.post_attn_ln is not None or L.post_mlp_ln is not None or
                    not all(isinstance(t, torch.Tensor) for t in (L.qkv, L.o, L.gate_up, L.down))):
                return False
        for L in self.layers:
            for ln_name, w_name in (("ln1", "qkv"), ("ln2", "gate_up")):
                g = getattr(L, ln_name).float() + woff
                setattr(L, w_name, (getattr(L, w_name).float() * g[None, :]).to(torch.bfloat16).contiguous())
                setattr(L, ln_name, torch.full_like(getattr(L, ln_name), 1.0 - woff))
        self.norm_folded = True
        self._setup_chain()
        return True

    def _setup_chain(self) -> None:
        """Decides whether decode-sized steps can run the folded-norm GEMM chain on this rank's shard shapes."""
        H, F2 = self.cfg.hidden_size, 2 * self.ffn
        shapes = (((self.hq + 2 * self.hkv) * self.cfg.head_dim, H), (H, self.hq * self.cfg.head_dim), (F2, H),
                  (H, self.ffn))
        par = self.comm.is_parallel      # the sharded o / down projections take any K that is a multiple of 64
        self._chain_ok = (self.device.type == "cuda" and H % 128 == 0 and H // 128 * 8 <= 512 and
                          all(ops.gated_fused(64, n & ~1, k) or (par and i in (1, 3) and k % 64 == 0)
                              for i, (n, k) in enumerate(shapes)))
        if self._chain_ok:
            self._ssq = [ops.ssq_buffer(self.device) for _ in range(2)]

    def gather_unsharded(self, dst: int = 0) -> "LlamaGpu | None":
        """Collective over the model's ranks: rebuilds the complete (tensor-parallel degree 1) model on rank `dst`
        from every rank's shards and returns it there (None elsewhere). The copy shares no memory with the shards;
        it serves equivalence checks (TP = k tokens against TP = 1 tokens on the same weights) and re-sharding.
        Dense bf16 layers only."""
        import torch.distributed as dist

        if not self.comm.is_parallel:
            return self
        P, r = self.comm.world, self.comm.rank
        if self.quant_format is not None or self.has_moe:
            raise Unsupported("gather_unsharded: dense bf16 layers only")

        def gather(t: torch.Tensor) -> list[torch.Tensor] | None:
            t = t.contiguous()
            parts = [torch.empty_like(t) for _ in range(P)] if r == dst else None
            dist.gather(t, parts, dst=dst, group=self.comm.group)
            return parts

        full = LlamaGpu(self.cfg, comm=single(self.device), device=self.device) if r == dst else None
        D = self.cfg.head_dim
        nq, nkv = self.hq * D, self.hkv * D
        head = gather(self.lm_head)
        if full is not None:
            full.embed, full.norm, full.lm_head = self.embed, self.norm, torch.cat(head, 0)
            full.cos, full.sin, full.max_positions = self.cos, self.sin, self.max_positions
        for L in self.layers:
            qkv, o, gu, down = gather(L.qkv), gather(L.o), gather(L.gate_up), gather(L.down)
            bias = gather(L.qkv_bias) if L.qkv_bias is not None else None
            if full is None:
                continue

            def regroup(parts):
                return torch.cat([p[:nq] for p in parts] + [p[nq:nq + nkv] for p in parts] +
                                 [p[nq + nkv:] for p in parts], 0)
            full.layers.append(LayerWeights(
                ln1=L.ln1, qkv=regroup(qkv), qkv_bias=regroup(bias) if bias is not None else None, q_norm=L.q_norm,
                k_norm=L.k_norm, o=torch.cat(o, 1).contiguous(), post_attn_ln=L.post_attn_ln, ln2=L.ln2,
                gate_up=torch.cat(gu, 0), down=torch.cat(down, 1).contiguous(), post_mlp_ln=L.post_mlp_ln))
        if full is not None:
            full.norm_folded = self.norm_folded
            if self.norm_folded:
                full._setup_chain()
        return full

    norm_folded: bool = False
    _chain_ok: bool = False

    def init_random(self, seed: int = 0, std: float = 0.02) -> "LlamaGpu":
        """Random N(0, std) weights generated directly on the device in this rank's shard shapes."""
        cfg, dev = self.cfg, self.device
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + self.comm.rank)
        H, D = cfg.hidden_size, cfg.head_dim

        def rnd(*shape):
            t = torch.empty(*shape, dtype=torch.bfloat16, device=dev)
            t.normal_(0.0, std, generator=g)
            return t

        one = 0.0 if cfg.architecture is Architecture.GEMMA2 else 1.0

        def ones(n):
            return torch.full((n,), one, dtype=torch.bfloat16, device=dev)

        ge = torch.Generator(device=dev).manual_seed(seed * 1000 + 999)  # shared across ranks
        self.embed = torch.empty(cfg.vocab_size, H, dtype=torch.bfloat16, device=dev).normal_(0.0, std, generator=ge)
        self.norm = ones(H)
        if cfg.tie_word_embeddings:
            self.lm_head = self.embed[self.comm.rank * self.vocab_local:(self.comm.rank + 1) * self.vocab_local]
        else:
            self.lm_head = rnd(self.vocab_local, H)
        sandwich = cfg.architecture.sandwich_norms
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(LayerWeights(
                ln1=ones(H), qkv=rnd((self.hq + 2 * self.hkv) * D, H), qkv_bias=None,
                q_norm=torch.ones(D, dtype=torch.bfloat16, device=dev) if cfg.architecture.has_qk_norm else None,
                k_norm=torch.ones(D, dtype=torch.bfloat16, device=dev) if cfg.architecture.has_qk_norm else None,
                o=rnd(H, self.hq * D), post_attn_ln=ones(H) if sandwich else None, ln2=ones(H),
                gate_up=rnd(2 * self.ffn, H), down=rnd(H, self.ffn), post_mlp_ln=ones(H) if sandwich else None))
        self.fold_norms()
        return self

    def quantize_(self, fmt: str = "Q4_K") -> "LlamaGpu":
        """Replace the projection weights of every layer by packed `fmt` weights (quantise-on-load, the role of
        candle-llm's Q4_K / Q8_0 quantise-on-load: candle-llm/src/quant.rs); embeddings and the output head stay bf16.
        Decode-sized steps then run the fused dequant-GEMM; the prefill tensor-parallel scatter paths need dense
        weights and stay off."""
        from ..ops.quant import quantize_on_device

        for L in self.layers:
            for name in ("qkv", "o", "gate_up", "down"):
                w = getattr(L, name)
                if isinstance(w, torch.Tensor) and w.shape[1] % 256 == 0:
                    setattr(L, name, quantize_on_device(w, fmt))
        self.quant_format = fmt
        return self

    # bytes of the next projection's weights each decode-step norm prefetches into L2 (0 = all of them, < 0 = off).
    # Off by default: measured on B200 the prefetches lengthen the norm kernel that the GEMM's dependency waits on
    # (Llama-3-8B step 5.27 ms without, 5.50 ms with 24-48 MB, 6.06 ms with 96 MB).
    l2_prefetch_bytes: int = int(os.environ.get("SWB_L2_PREFETCH_MB", "-1")) << 20 if \
        int(os.environ.get("SWB_L2_PREFETCH_MB", "-1")) >= 0 else -1
    quant_format: str | None = None
    dense_prefill: bool = True      # False: always read K / V back from the paged cache (comparison runs)

    def weight_bytes(self) -> int:
        n, q = self.embed.numel() + self.norm.numel(), 0
        if self.lm_head.data_ptr() != self.embed.data_ptr() and not self.cfg.tie_word_embeddings:
            n += self.lm_head.numel()
        for L in self.layers:
            n += 2 * L.ln1.numel()
            for t in (L.qkv, L.o, L.gate_up, L.down):
                q += t.nbytes if not isinstance(t, torch.Tensor) else 2 * t.numel()
        return n * 2 + q

    # ---- forward --------------------------------------------------------------------------------
    def forward_hidden(self, inp: StepInputs, kv_pool: torch.Tensor, *, stage_in=None, last_stage: bool = True):
        """Runs the decoder stack; kv_pool is [layers, 2, blocks, Hkv_local, block_size, 128]. Returns the
        final (un-normed) branch output and residual folded together: rows of normed hidden states [T, H]."""
        cfg = self.cfg
        D = cfg.head_dim
        eps, woff = cfg.rms_norm_eps, cfg.norm_weight_offset
        T = inp.input_ids.numel()
        if self._use_tp_prefill(T) and inp.embed_rows is None and inp.rope_table is None and inp.deepstack is None:
            return self._forward_hidden_tp_prefill(inp, kv_pool)
        rope_pos, rope_cos, rope_sin = inp.positions, self.cos, self.sin
        if inp.rope_table is not None:
            rope_cos, rope_sin = inp.rope_table
            rope_pos = torch.arange(T, dtype=torch.int32, device=self.device)
        taps = inp.deepstack[1] if inp.deepstack is not None else []
        # decode-sized steps of a dense model: the norms are folded into a chain of GEMM epilogues
        chain = (self._chain_ok and inp.decode and T <= 64 and self.quant_format is None and
                 os.environ.get("SWB_NORM_CHAIN", "1") != "0")
        chain = chain and not taps
        fc = self.comm.fused if self.comm.is_parallel else None
        if chain and self.comm.is_parallel:
            chain = fc is not None and T <= fc.chain_tokens and stage_in is None
        if stage_in is None:
            res = ops.embedding(inp.input_ids, self.embed, scale=cfg.embed_scale)
            if inp.embed_rows is not None:
                res.index_copy_(0, inp.embed_rows, inp.embed_values.to(res.dtype))
            branch = None
        else:       # a later pipeline stage: the residual stream and the pending branch output of the previous stage
            res, branch = stage_in
        block_size = kv_pool.shape[4]
        q_cols = self.hq * D
        n = 1
        pending_h = None
        # optional: each norm asks L2 for (the first megabytes of) its consumer's weights (see l2_prefetch_bytes)
        pf_bytes = self.l2_prefetch_bytes if inp.decode else -1
        pf = (lambda t: t if (pf_bytes >= 0 and isinstance(t, torch.Tensor)) else None)
        ssq_prev = None                 # partial sums of squares of `res` (valid while branch is None)
        H = cfg.hidden_size
        for li, L in enumerate(self.layers):
            if chain and ssq_prev is not None and branch is None:
                h = None                # the qkv projection normalises the residual stream itself
            elif pending_h is not None:
                h = pending_h           # already all-reduced, added to the residual and normed with this ln1
            elif branch is None:
                h = ops.rmsnorm(res, L.ln1, eps, w_offset=woff, prefetch=pf(L.qkv), prefetch_bytes=pf_bytes)
            else:
                h = ops.rmsnorm(branch, L.ln1, eps, residual=res, w_offset=woff, prefetch=pf(L.qkv),
                                prefetch_bytes=pf_bytes)
            if h is None:
                qkv = ops.gemm_bf16_normed(res, L.qkv, bias=L.qkv_bias, ssq_in=ssq_prev, norm_dim=H, eps=eps)
            else:
                qkv = ops.linear_any(h, L.qkv, bias=L.qkv_bias)
            ops.rope_kv_write(qkv, rope_pos, inp.slot_mapping, rope_cos, rope_sin, kv_pool[li, 0], kv_pool[li, 1],
                              self.hq, self.hkv, D, rot_dim=self.rot_dim, interleaved=self.rope_interleaved,
                              q_norm=L.q_norm, k_norm=L.k_norm, norm_eps=eps, norm_w_offset=woff,
                              block_size=block_size)
            q = qkv[:, :q_cols].view(T, self.hq, D)
            if inp.fresh_prefill and inp.cu_q is not None and not cfg.attn_logit_softcap and self.dense_prefill:
                # no earlier context: causal attention straight from the projection output on the tcgen05 kernel
                kv_cols = self.hkv * D
                attn = ops.varlen_causal_attention(q, qkv[:, q_cols:q_cols + kv_cols].view(T, self.hkv, D),
                                                   qkv[:, q_cols + kv_cols:].view(T, self.hkv, D), inp.cu_q,
                                                   inp.max_q_len, scale=cfg.attn_scale)
            else:
                attn = ops.paged_attention(q, kv_pool[li, 0], kv_pool[li, 1], inp.block_table, inp.kv_lens,
                                           cu_q=inp.cu_q, max_q_len=inp.max_q_len, scale=cfg.attn_scale, causal=True,
                                           decode=inp.decode, num_splits=inp.attn_splits,
                                           softcap=cfg.attn_logit_softcap or 0.0)
            if chain:
                if branch is not None:          # first layer of the chain: fold the pending branch into the stream
                    res.add_(branch)
                    branch = None
                    n += 1
                gelu = cfg.mlp_activation in ("gelu", "gelu_tanh")
                if fc is not None:
                    fc.gemm_peer_reduce(attn.reshape(T, -1), L.o, res, 0, ssq_out=self._ssq[0], ssq_zero=self._ssq[1])
                else:
                    ops.gemm_bf16_normed(attn.reshape(T, -1), L.o, out=res, residual=res, ssq_out=self._ssq[0],
                                         ssq_zero=self._ssq[1])
                act = ops.gemm_bf16_normed(res, L.gate_up, act="geglu_pairs" if gelu else "swiglu_pairs",
                                           ssq_in=self._ssq[0], norm_dim=H, eps=eps)
                if fc is not None:
                    fc.gemm_peer_reduce(act, L.down, res, 1, ssq_out=self._ssq[1], ssq_zero=self._ssq[0])
                else:
                    ops.gemm_bf16_normed(act, L.down, out=res, residual=res, ssq_out=self._ssq[1],
                                         ssq_zero=self._ssq[0])
                ssq_prev, pending_h = self._ssq[1], None
                n += 6 + (1 if h is not None else 0)
                continue
            fused = self.comm.fused if (self.comm.fused is not None and T <= self.comm.fused.max_tokens and
                                        L.post_attn_ln is None and li >= len(taps)) else None
            if fused is not None:
                h = fused.gemm_allreduce_rmsnorm(attn, L.o, res, L.ln2, eps, woff)
            else:
                branch = ops.linear_any(attn, L.o)
                branch = self.comm.all_reduce(branch)
                if L.post_attn_ln is not None:
                    branch = ops.rmsnorm(branch, L.post_attn_ln, eps, w_offset=woff)
                    n += 1
                h = ops.rmsnorm(branch, L.ln2, eps, residual=res, w_offset=woff,
                                prefetch=pf(L.gate_up) if L.moe is None else None, prefetch_bytes=pf_bytes)
            if L.moe is not None:
                pending_h = None
                branch = self.comm.all_reduce(self._moe_ffn(h, L.moe))
                n += 9
                if li < len(taps):      # the stream after this layer is res + branch: the tap joins the pending branch
                    branch.index_add_(0, inp.deepstack[0], taps[li].to(branch.dtype))
                continue
            act = self._gated_mlp_in(h, L.gate_up)
            if fused is not None and L.post_mlp_ln is None:
                # the down-projection's all-reduce fuses with the NEXT norm (next layer's ln1 or the final norm)
                nxt = self.layers[li + 1].ln1 if li + 1 < len(self.layers) else self.norm
                pending_h = fused.gemm_allreduce_rmsnorm(act, L.down, res, nxt, eps, woff)
                branch = None
            else:
                pending_h = None
                branch = ops.linear_any(act, L.down)
                branch = self.comm.all_reduce(branch)
                if L.post_mlp_ln is not None:
                    branch = ops.rmsnorm(branch, L.post_mlp_ln, eps, w_offset=woff)
                    n += 1
            if li < len(taps):
                branch.index_add_(0, inp.deepstack[0], taps[li].to(branch.dtype))
            n += 7 + self._mlp_in_launches
        self.launches = n
        if not last_stage:
            assert pending_h is None
            return res, branch
        if pending_h is not None:
            final = pending_h
        elif branch is None:
            final = ops.rmsnorm(res, self.norm, eps, w_offset=woff)
        else:
            final = ops.rmsnorm(branch, self.norm, eps, residual=res, w_offset=woff)
        self.launches += 1
        if inp.logits_rows is not None:
            return final.index_select(0, inp.logits_rows)
        return final

    def _gated_mlp_in(self, h: torch.Tensor, gate_up) -> torch.Tensor:
        """act(h W_gate^T) * (h W_up^T). A dense layer's gate_up rows are interleaved (gate_0, up_0, gate_1, ...) so a
        decode-sized step applies the gated activation in the projection's epilogue."""
        if isinstance(gate_up, torch.Tensor) and h.device.type == "cuda":
            y = ops.linear_gated(h, gate_up, self.cfg.mlp_activation)
            self._mlp_in_launches = 1 if y.shape[0] <= 64 and ops.gated_fused(h.shape[0], *gate_up.shape) else 2
            return y
        self._mlp_in_launches = 2
        return ops.gated_act_mul(ops.linear_any(h, gate_up), self.cfg.mlp_activation, paired=True)

    def _moe_ffn(self, h: torch.Tensor, m: MoeWeights) -> torch.Tensor:
        """Sparse FFN on this rank's shard (partial sums; the caller all-reduces). Routing stays on the device:
        the (token, expert) pairs are sorted by expert into a buffer whose per-expert segments are padded to the
        128-row GEMM tile, one grouped GEMM per projection picks each tile's expert from a device table, and the
        weighted results are summed back per token. Every shape is a function of the token count only, so the step
        can be captured in a CUDA graph. (The reference visits experts serially after a host top-k:
        candle-llm/src/models/llama.rs:1415-1488.)"""
        moe = self.cfg.moe
        act = self.cfg.mlp_activation
        T, H = h.shape
        E, k = m.router.shape[0], moe.num_experts_per_tok
        logits = ops.gemm_bf16(h, m.router, out_dtype=torch.float32)
        probs = torch.softmax(logits, dim=-1)
        topv, topi = probs.topk(k, dim=-1)
        if moe.norm_topk_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        topv = topv * moe.routed_scaling_factor
        if h.device.type != "cuda" or os.environ.get("SWB_MOE") == "loop":
            out = self._moe_experts_loop(h, m, topv, topi)
        else:
            dev = h.device
            flat_e = topi.reshape(-1)
            order = torch.argsort(flat_e, stable=True)
            sorted_e = flat_e.index_select(0, order)
            counts = torch.zeros(E, dtype=torch.int64, device=dev).scatter_add_(0, flat_e, torch.ones_like(flat_e))
            padded = (counts + 127) // 128 * 128
            pad_end = torch.cumsum(padded, 0)
            seg_start = torch.cumsum(counts, 0) - counts
            dest = (pad_end - padded).index_select(0, sorted_e) + \
                (torch.arange(T * k, device=dev) - seg_start.index_select(0, sorted_e))
            R = (T * k + E * 127 + 127) // 128 * 128          # static bound on the padded row count
            tile_start = torch.arange(R // 128, device=dev) * 128
            tile_e = torch.searchsorted(pad_end, tile_start, right=True)
            tile_e = torch.where(tile_e < E, tile_e, torch.full_like(tile_e, -1)).to(torch.int32)
            src_tok = order // k
            xp = torch.zeros((R, H), dtype=torch.bfloat16, device=dev)
            xp.index_copy_(0, dest, h.index_select(0, src_tok))
            gu = ops.gemm_bf16_grouped(xp, m.gate_up, tile_e)
            y = ops.gemm_bf16_grouped(ops.gated_act_mul(gu, act), m.down, tile_e)
            wgt = topv.reshape(-1).index_select(0, order)
            out = torch.zeros((T, H), dtype=torch.float32, device=dev)
            out.index_add_(0, src_tok, y.index_select(0, dest).float() * wgt[:, None])
        if m.shared_gate_up is not None:
            y = ops.gemm_bf16(ops.gated_act_mul(ops.gemm_bf16(h, m.shared_gate_up), act), m.shared_down).float()
            if m.shared_gate is not None:
                y = y * torch.sigmoid(ops.gemm_bf16(h, m.shared_gate, out_dtype=torch.float32)[:, :1])
            out += y
        return out.to(torch.bfloat16)

    def _moe_experts_loop(self, h: torch.Tensor, m: MoeWeights, topv: torch.Tensor, topi: torch.Tensor) -> torch.Tensor:
        """Host loop over the experts that received tokens (comparison path, SWB_MOE=loop)."""
        act = self.cfg.mlp_activation
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in torch.unique(topi).tolist():
            sel = topi == e
            rows = sel.any(-1).nonzero().flatten()
            wgt = (topv * sel).sum(-1).index_select(0, rows)
            x = h.index_select(0, rows)
            y = ops.gemm_bf16(ops.gated_act_mul(ops.gemm_bf16(x, m.gate_up[e]), act), m.down[e])
            out.index_add_(0, rows, y.float() * wgt[:, None])
        return out

    @property
    def has_moe(self) -> bool:
        return any(L.moe is not None for L in self.layers)

    # ---- prefill with fused reduce-scatter / all-gather -----------------------------------------------------
    def _use_tp_prefill(self, T: int) -> bool:
        import os

        f = self.comm.fused
        if f is None or not self.comm.is_parallel or T <= f.max_tokens or os.environ.get("SWB_TP_PREFILL") == "nccl":
            return False
        if self.quant_format is not None:
            return False
        if any(L.post_attn_ln is not None or L.post_mlp_ln is not None or L.moe is not None for L in self.layers):
            return False
        return T <= self.tp_prefill_max_tokens

    tp_prefill_max_tokens = 8192

    def _tp_prefill_context(self):
        if getattr(self, "_tp_ctx", None) is None:
            from ..parallel.tp_prefill import TpPrefillContext

            self._tp_ctx = TpPrefillContext(self.comm, self.cfg.hidden_size, self.tp_prefill_max_tokens)
        return self._tp_ctx

    def _forward_hidden_tp_prefill(self, inp: StepInputs, kv_pool: torch.Tensor) -> torch.Tensor:
        """Same math as forward_hidden; the residual stream is sharded by token rows, each row-parallel GEMM scatters
        its partial sums to the row owners from its epilogue, and the owners' reduce + norm kernel gathers the normed
        rows on every rank for the next column-parallel GEMM."""
        cfg = self.cfg
        D = cfg.head_dim
        eps, woff = cfg.rms_norm_eps, cfg.norm_weight_offset
        T = inp.input_ids.numel()
        ctx = self._tp_prefill_context()
        lo, n_rows = ctx.my_rows(T)
        block_size = kv_pool.shape[4]
        q_cols = self.hq * D
        ids_l = inp.input_ids[lo:lo + n_rows]
        res = (ops.embedding(ids_l, self.embed, scale=cfg.embed_scale) if n_rows > 0 else
               torch.zeros((1, cfg.hidden_size), dtype=torch.bfloat16, device=self.device))
        h = ctx.reduce_norm_gather(T, res, self.layers[0].ln1, eps, woff, reduce=False)
        n = 3
        for li, L in enumerate(self.layers):
            qkv = ops.linear_any(h, L.qkv, bias=L.qkv_bias)
            ops.rope_kv_write(qkv, inp.positions, inp.slot_mapping, self.cos, self.sin, kv_pool[li, 0], kv_pool[li, 1],
                              self.hq, self.hkv, D, rot_dim=self.rot_dim, interleaved=self.rope_interleaved,
                              q_norm=L.q_norm, k_norm=L.k_norm, norm_eps=eps, norm_w_offset=woff,
                              block_size=block_size)
            q = qkv[:, :q_cols].view(T, self.hq, D)
            if inp.fresh_prefill and inp.cu_q is not None and not cfg.attn_logit_softcap and self.dense_prefill:
                # no earlier context: causal attention straight from the projection output on the tcgen05 kernel
                kv_cols = self.hkv * D
                attn = ops.varlen_causal_attention(q, qkv[:, q_cols:q_cols + kv_cols].view(T, self.hkv, D),
                                                   qkv[:, q_cols + kv_cols:].view(T, self.hkv, D), inp.cu_q,
                                                   inp.max_q_len, scale=cfg.attn_scale)
            else:
                attn = ops.paged_attention(q, kv_pool[li, 0], kv_pool[li, 1], inp.block_table, inp.kv_lens,
                                           cu_q=inp.cu_q, max_q_len=inp.max_q_len, scale=cfg.attn_scale, causal=True,
                                           decode=inp.decode, num_splits=inp.attn_splits,
                                           softcap=cfg.attn_logit_softcap or 0.0)
            ctx.gemm_scatter_rows(attn, L.o)
            h = ctx.reduce_norm_gather(T, res, L.ln2, eps, woff)
            act = self._gated_mlp_in(h, L.gate_up)
            ctx.gemm_scatter_rows(act, L.down)
            nxt = self.layers[li + 1].ln1 if li + 1 < len(self.layers) else self.norm
            h = ctx.reduce_norm_gather(T, res, nxt, eps, woff)
            n += 11
        self.launches = n
        if inp.logits_rows is not None:
            return h.index_select(0, inp.logits_rows)
        return h.clone()

    def logits_local(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits of this rank's vocabulary shard: [R, vocab / P]."""
        self.launches += 1
        logits = ops.gemm_bf16(hidden, self.lm_head, out_dtype=torch.float32)
        c = self.cfg.final_logit_softcap
        return torch.tanh(logits / c) * c if c else logits

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        local = self.logits_local(hidden)
        return self.comm.all_gather(local, dim=1) if self.comm.is_parallel else local

    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        """Vocab-parallel lm_head + argmax: each rank reduces its shard, then a tiny (value, index) exchange."""
        local = self.logits_local(hidden)
        self.launches += 1
        if not self.comm.is_parallel:
            return ops.argmax(local)
        f = self.comm.fused
        if f is not None and local.shape[0] <= f.max_tokens and os.environ.get("SWB_TP_ARGMAX") != "nccl":
            self.launches += 1
            return f.argmax_vocab_parallel(local, self.vocab_local)
        vals = local.max(dim=-1)
        idx = vals.indices + self.comm.rank * self.vocab_local
        packed = torch.stack((vals.values.double(), idx.double()), dim=-1)  # [R, 2]
        allp = self.comm.all_gather(packed[None], dim=0)                     # [P, R, 2]
        best = allp[..., 0].max(dim=0)
        # ties across ranks resolve to the lowest rank (= lowest global index), like a single-device argmax
        return allp[best.indices, torch.arange(allp.shape[1], device=allp.device), 1].long()
