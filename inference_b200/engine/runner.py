"""Model runner: turns host-side sequence state into device step inputs and executes the forward.

Decode steps are captured once per (batch, attention-splits) shape into a CUDA graph over static input
buffers; each step then costs one pinned host->device copy of the step metadata, one graph launch and
one device->host copy of the sampled tokens. The reference launches ~45 small kernels plus 7 library
GEMMs per layer per token with no graph capture (candle-llm/README.md:165-168 calls decode launch-bound).
"""
from __future__ import annotations

from dataclasses import dataclass

import os

import torch

from ..models.llama import LlamaGpu, StepInputs
from ..utils import tracing
from .kv_pool import PagedKvPool, PagedSequence


def _splits_for(batch: int, kv_heads: int, max_kv: int, sms: int = 148) -> int:
    """KV splits of the decode attention: enough CTAs for `SWB_ATTN_CTAS_PER_SM` (default 2) per SM, never below one
    64-key tile per split."""
    import os

    tiles = max(1, (max_kv + 63) // 64)
    per_sm = max(0.25, float(os.environ.get("SWB_ATTN_CTAS_PER_SM", "2")))
    want = max(1, int(per_sm * sms) // max(1, batch * kv_heads))
    s = 1
    while s * 2 <= min(want, tiles, 32):
        s *= 2
    return s


def _bucket(batch: int, max_batch: int) -> int:
    """Batch size a decode graph is captured for: exact up to 8 rows, then the next multiple of 8 (of 16
    above 64). A continuous-batching job whose lanes drain one by one then replays a handful of graphs
    instead of capturing one per live-lane count."""
    if batch <= 8:
        return batch
    step = 8 if batch <= 64 else 16
    return min(max_batch, (batch + step - 1) // step * step)


@dataclass
class _DecodeGraph:
    graph: torch.cuda.CUDAGraph
    tokens_out: torch.Tensor
    logits_out: torch.Tensor | None
    launches: int


class ModelRunner:
    MULTI_STEPS = 256

    def __init__(self, model: LlamaGpu, pool: PagedKvPool, max_batch: int = 64, max_seq_len: int = 8192,
                 use_graphs: bool = True):
        self.model, self.pool = model, pool
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.max_blocks = (max_seq_len + pool.block_size - 1) // pool.block_size
        self.use_graphs = use_graphs and not getattr(model, "eager_only", False)   # mixture-of-experts routing is device side, so those models capture too
        dev = model.device
        model.ensure_rope(max_seq_len + 64)
        # static decode-step buffers; one packed int64 staging area so a step is a single H2D copy
        self._n_meta = max_batch * 4 + max_batch * self.max_blocks
        self._host_meta = torch.zeros(self._n_meta, dtype=torch.int32).pin_memory() if dev.type == "cuda" else \
            torch.zeros(self._n_meta, dtype=torch.int32)
        self._host_np = self._host_meta.numpy()
        self._host_table_np = self._host_np[4 * max_batch:].reshape(max_batch, self.max_blocks)
        self._row_state: list[tuple[int, int, int]] = [(0, 0, 0)] * max_batch  # (uid, epoch, blocks written)
        self._dev_meta = torch.zeros(self._n_meta, dtype=torch.int32, device=dev)
        self._ids = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self._pos = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self._slots = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self._kvl = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self._table = torch.zeros((max_batch, self.max_blocks), dtype=torch.int32, device=dev)
        self._host_tokens = torch.zeros(max_batch, dtype=torch.int64).pin_memory() if dev.type == "cuda" else \
            torch.zeros(max_batch, dtype=torch.int64)
        # multi-step greedy runs: the metadata of up to MULTI_STEPS steps, the tokens they produce and a device-side
        # step counter; the captured graph indexes both by the counter, so a step is one graph replay and nothing else
        self._multi_meta = torch.zeros((self.MULTI_STEPS, self._n_meta), dtype=torch.int32, device=dev)
        self._multi_out = torch.zeros(self.MULTI_STEPS * max_batch, dtype=torch.int64, device=dev)
        self._step = torch.zeros(1, dtype=torch.int32, device=dev)
        self._graphs: dict[tuple[int, int, bool], _DecodeGraph] = {}
        self._meta_copy_done = None
        self.pad_batches = self.use_graphs      # decode batches are padded to a bucket so graphs are reused
        # SWB_DECODE_SPLIT=n runs a decode batch of more than n rows as consecutive sub-steps of at most n rows, so
        # that every sub-step stays inside the row limit of the chained (folded-norm, GEMM + cross-rank sum) path
        self.decode_split = int(os.environ.get("SWB_DECODE_SPLIT", "0"))
        self.captures = 0
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.launches_last = 0

    # ---- prefill (eager, ragged) ------------------------------------------------------------------
    def prefill(self, seqs: list[PagedSequence], new_tokens: list[list[int]], *, want_logits: bool = False,
                all_positions: bool = False, embed_overrides: list[tuple[list[int], torch.Tensor] | None] | None = None,
                mrope_overrides: list | None = None):
        """Appends new_tokens[i] to seqs[i] (any mix of lengths, including chunked / prefix-seeded sequences)
        and returns greedy next tokens [num_seqs] (or fp32 logits when want_logits). embed_overrides[i] =
        (positions within new_tokens[i], vectors [len(positions), hidden]) replaces those tokens' embeddings (the
        image placeholders of a vision-language prompt). mrope_overrides[i] = (positions [3, len(new_tokens[i])], next
        position, rows within new_tokens[i], taps) gives those tokens three-axis rotary positions and adds taps[l] to
        the residual stream at `rows` after decoder layer l; the sequence's later tokens continue at `next position`
        (kept on the sequence as `rope_delta`)."""
        dev = self.model.device
        ids, pos, slots, cu, kvl, rows = [], [], [], [0], [], []
        fresh = all(s.length == 0 for s in seqs)     # no earlier context: attention can read K / V from the QKV buffer
        for s, toks in zip(seqs, new_tokens):
            start = s.length
            sl = s.reserve(len(toks))
            ids += toks
            delta = getattr(s, "rope_delta", 0)
            pos += list(range(start + delta, start + delta + len(toks)))
            slots += sl
            cu.append(cu[-1] + len(toks))
            kvl.append(s.length)
            rows.append(cu[-1] - 1)
        maxb = max(len(s.blocks) for s in seqs)
        table = torch.zeros((len(seqs), maxb), dtype=torch.int32)
        for i, s in enumerate(seqs):
            table[i, : len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.int32)
        max_q = max(len(t) for t in new_tokens)
        G = self.model.cfg.groups
        decode = max_q * G <= 16 and all(len(t) == max_q for t in new_tokens)
        inp = StepInputs(
            input_ids=torch.tensor(ids, dtype=torch.int64, device=dev),
            positions=torch.tensor(pos, dtype=torch.int32, device=dev),
            slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev),
            block_table=table.to(dev), kv_lens=torch.tensor(kvl, dtype=torch.int32, device=dev),
            cu_q=None if decode else torch.tensor(cu, dtype=torch.int32, device=dev), max_q_len=max_q,
            num_seqs=len(seqs), decode=decode, fresh_prefill=fresh and not decode,
            attn_splits=_splits_for(len(seqs), self.model.hkv, max(kvl)) if decode else 1,
            logits_rows=None if all_positions else torch.tensor(rows, dtype=torch.int64, device=dev))
        if embed_overrides is not None:
            er, ev = [], []
            for i, ov in enumerate(embed_overrides):
                if ov is not None:
                    er += [cu[i] + p for p in ov[0]]
                    ev.append(ov[1].to(dev))
            if er:
                inp.embed_rows = torch.tensor(er, dtype=torch.int64, device=dev)
                inp.embed_values = torch.cat(ev, dim=0)
        if mrope_overrides is not None and any(m is not None for m in mrope_overrides):
            self._apply_mrope(inp, seqs, mrope_overrides, cu)
        with tracing.span("runner.prefill", tokens=len(ids), seqs=len(seqs)):
            hidden = self.model.forward_hidden(inp, self.pool.data)
            self.launches_last = self.model.launches
            if want_logits or all_positions:
                return self.model.logits(hidden)
            return self.model.greedy_tokens(hidden)

    def _apply_mrope(self, inp: StepInputs, seqs, overrides, cu: list[int]) -> None:
        """Per-token rotary table for a step in which some sequences carry three-axis positions (the others keep their
        scalar positions on all three axes), the flat DeepStack rows, and each such sequence's `rope_delta`."""
        from ..models.qwen3_vl import interleaved_mrope_table

        m = self.model
        pos3 = inp.positions.to(torch.int64)[None, :].repeat(3, 1)
        rows, levels = [], []
        for i, (s, ov) in enumerate(zip(seqs, overrides)):
            if ov is None:
                continue
            p3, nxt, r, taps = ov
            pos3[:, cu[i]:cu[i + 1]] = p3.to(pos3.device)
            s.rope_delta = int(nxt) - s.length
            if len(taps):
                rows.append(r.to(pos3.device, torch.int64) + cu[i])
                levels.append(taps)
        inv = torch.tensor(m._inv_freq, dtype=torch.float32, device=pos3.device) if not torch.is_tensor(m._inv_freq) \
            else m._inv_freq.to(pos3.device, torch.float32)
        cos, sin = interleaved_mrope_table(pos3, inv, m.cfg.mrope_section_resolved())
        inp.rope_table = (cos.float().contiguous(), sin.float().contiguous())
        if rows:
            depth = min(len(t) for t in levels)
            inp.deepstack = (torch.cat(rows), [torch.cat([t[l].to(pos3.device) for t in levels], dim=0) for l in range(depth)])

    # ---- decode (graph-captured, one token per sequence) ---------------------------------------------
    def _fill_decode_meta(self, seqs: list[PagedSequence], tokens: list[int], pad_to: int = 0) -> int:
        """Writes the step metadata of the live rows; rows len(seqs)..pad_to-1 become copies of row 0 (same
        token, position, slot and block table), so they recompute row 0 and store identical K / V bytes."""
        MB = self.max_batch
        h, table = self._host_np, self._host_table_np
        if self._meta_copy_done is not None:
            # a caller that kept the previous step's logits on the device never synchronised: the staging buffer is
            # rewritten only after the copy that reads it has finished
            self._meta_copy_done.synchronize()
            self._meta_copy_done = None
        max_kv = 0
        for i, s in enumerate(seqs):
            p = s.length
            slot = s.reserve(1)[0]
            h[i] = tokens[i]
            h[MB + i] = p + getattr(s, "rope_delta", 0)
            h[2 * MB + i] = slot
            h[3 * MB + i] = p + 1
            if p + 1 > max_kv:
                max_kv = p + 1
            owner, epoch, written = self._row_state[i]
            nb = len(s.blocks)
            if owner != s.uid or epoch != s.epoch or written > nb:
                table[i, :nb] = s.blocks
                self._row_state[i] = (s.uid, s.epoch, nb)
            elif written < nb:
                table[i, written:nb] = s.blocks[written:nb]
                self._row_state[i] = (s.uid, s.epoch, nb)
        if pad_to > len(seqs):
            nb0 = len(seqs[0].blocks)
            for i in range(len(seqs), pad_to):
                h[i], h[MB + i], h[2 * MB + i], h[3 * MB + i] = h[0], h[MB], h[2 * MB], h[3 * MB]
                table[i, :nb0] = table[0, :nb0]
                self._row_state[i] = (-1, -1, 0)
        return max_kv

    def _unpack_meta(self, B: int, skip_ids: bool = False, multi: bool = False) -> None:
        """One kernel: packed int32 step metadata -> the typed static input tensors. `multi` reads row
        `self._step` of the multi-step table instead of the single-step staging buffer."""
        MB, mb = self.max_batch, self.max_blocks
        if self.model.device.type != "cuda":
            m = self._dev_meta
            if not skip_ids:
                self._ids[:B].copy_(m[:B])
            self._pos[:B].copy_(m[MB:MB + B])
            self._slots[:B].copy_(m[2 * MB:2 * MB + B])
            self._kvl[:B].copy_(m[3 * MB:3 * MB + B])
            self._table[:B].copy_(m[4 * MB:4 * MB + B * mb].view(B, mb))
            return
        from .._native import kernels
        from ..ops.runtime import check, stream_ptr

        src = self._multi_meta if multi else self._dev_meta
        rc = kernels().swb_decode_meta_unpack(src.data_ptr(), self._n_meta, self._step.data_ptr() if multi else None,
                                              MB, B, mb, None if skip_ids else self._ids.data_ptr(),
                                              self._pos.data_ptr(), self._slots.data_ptr(), self._kvl.data_ptr(),
                                              self._table.data_ptr(), stream_ptr())
        check(rc, "swb_decode_meta_unpack")

    def _decode_body(self, B: int, splits: int, want_logits: bool, feedback: bool = False):
        self._unpack_meta(B, skip_ids=feedback, multi=feedback and self.model.device.type == "cuda")
        cap = self.decode_split if 0 < self.decode_split < B else B
        parts = []
        for r0 in range(0, B, cap):
            r1 = min(B, r0 + cap)
            inp = StepInputs(input_ids=self._ids[r0:r1], positions=self._pos[r0:r1], slot_mapping=self._slots[r0:r1],
                             block_table=self._table[r0:r1], kv_lens=self._kvl[r0:r1], cu_q=None, max_q_len=1,
                             num_seqs=r1 - r0, decode=True, attn_splits=splits, logits_rows=None)
            part = self.model.forward_hidden(inp, self.pool.data)
            # the model may hand back a view of a workspace that the next sub-step reuses
            parts.append(part.clone() if cap < B else part)
        hidden = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        if want_logits:
            return None, self.model.logits(hidden)
        toks = self.model.greedy_tokens(hidden)
        if feedback:
            if self.model.device.type == "cuda":
                # the next replay consumes these without a host round trip; the step counter advances
                from .._native import kernels
                from ..ops.runtime import check, stream_ptr

                rc = kernels().swb_decode_step_tail(toks.data_ptr(), self._ids.data_ptr(), self._multi_out.data_ptr(),
                                                    self._step.data_ptr(), B, stream_ptr())
                check(rc, "swb_decode_step_tail")
            else:
                self._ids[:B].copy_(toks)
        return toks, None

    def decode(self, seqs: list[PagedSequence], tokens: list[int], *, want_logits: bool = False):
        """One decode step: feeds tokens[i] at the end of seqs[i]; returns next greedy tokens as a pinned
        host tensor [B] (after a stream sync) or device fp32 logits [B, vocab]."""
        B = len(seqs)
        assert B <= self.max_batch
        with tracing.span("runner.decode", batch=B):
            return self._decode(seqs, tokens, want_logits)

    def _decode(self, seqs: list[PagedSequence], tokens: list[int], want_logits: bool):
        B = len(seqs)
        Bp = _bucket(B, self.max_batch) if self.pad_batches else B
        max_kv = self._fill_decode_meta(seqs, tokens, Bp)
        self._dev_meta.copy_(self._host_meta, non_blocking=True)
        if want_logits and self.model.device.type == "cuda":
            self._meta_copy_done = torch.cuda.Event()
            self._meta_copy_done.record()
        self.h2d_bytes_last = self._host_meta.numel() * 4
        splits = _splits_for(Bp, self.model.hkv, max_kv)
        key = (Bp, splits, want_logits)
        if not self.use_graphs or self.model.device.type != "cuda":
            toks, logits = self._decode_body(Bp, splits, want_logits)
            self.launches_last = self.model.launches
        else:
            g = self._graphs.get(key)
            if g is None:
                g = self._capture(Bp, splits, want_logits)
                self._graphs[key] = g
                self.captures += 1
            g.graph.replay()
            toks, logits = g.tokens_out, g.logits_out
            self.launches_last = g.launches
        if want_logits:
            return logits[:B]
        toks = toks[:B]
        self._host_tokens[:B].copy_(toks, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes_last = B * 8
        return self._host_tokens[:B]

    def decode_multi(self, seqs: list[PagedSequence], tokens: list[int], n_steps: int) -> torch.Tensor:
        """n_steps greedy decode steps with the sampled token fed back on the device: the host uploads the
        metadata of all steps once, then only replays one captured graph per step (the graph reads its step's
        metadata and files its tokens through a device-side step counter).
        Returns the generated tokens [n_steps, B] on the device (no synchronisation is performed)."""
        B = len(seqs)
        dev = self.model.device
        if n_steps > self.MULTI_STEPS:
            parts, toks = [], tokens
            for k0 in range(0, n_steps, self.MULTI_STEPS):
                part = self.decode_multi(seqs, toks, min(self.MULTI_STEPS, n_steps - k0))
                parts.append(part)
                toks = part[-1].tolist()
            return torch.cat(parts, dim=0)
        n_meta = self._n_meta
        host_all = torch.empty((n_steps, n_meta), dtype=torch.int32)
        if dev.type == "cuda":
            host_all = host_all.pin_memory()
        max_kv = 0
        for k in range(n_steps):
            max_kv = self._fill_decode_meta(seqs, tokens if k == 0 else [0] * B)
            host_all[k].copy_(self._host_meta)
        self.h2d_bytes_last = host_all.numel() * 4
        splits = _splits_for(B, self.model.hkv, max_kv)
        first = torch.tensor(tokens, dtype=torch.int64)
        if dev.type != "cuda" or not self.use_graphs:
            out = torch.empty((n_steps, B), dtype=torch.int64, device=dev)
            self._ids[:B].copy_(first.to(dev))
            for k in range(n_steps):
                if dev.type == "cuda":
                    self._multi_meta[0].copy_(host_all[k], non_blocking=True)
                    self._step.zero_()
                else:
                    self._dev_meta.copy_(host_all[k])
                toks, _ = self._decode_body(B, splits, False, feedback=True)
                out[k].copy_(toks)
            self.launches_last = self.model.launches * n_steps
            return out
        key = (B, splits, "feedback")
        g = self._graphs.get(key)
        if g is None:
            self._multi_meta[0].copy_(host_all[0], non_blocking=True)
            self._step.zero_()
            self._ids[:B].copy_(first.to(dev, non_blocking=True))
            g = self._capture(B, splits, False, feedback=True)
            self._graphs[key] = g
            self.captures += 1
        self._multi_meta[:n_steps].copy_(host_all, non_blocking=True)
        self._step.zero_()
        self._ids[:B].copy_(first.pin_memory().to(dev, non_blocking=True))
        for _ in range(n_steps):
            g.graph.replay()
        self.launches_last = g.launches * n_steps
        return self._multi_out[:n_steps * B].view(n_steps, B).clone()

    def _capture(self, B: int, splits: int, want_logits: bool, feedback: bool = False) -> _DecodeGraph:
        # warm-up on a side stream (sets kernel attributes, fills the tensor-map cache), then capture
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                if feedback:
                    self._step.zero_()      # every warm-up run reads the same (first) row of the step table
                self._decode_body(B, splits, want_logits, feedback)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        fused = self.model.comm.fused
        if fused is not None:
            fused.begin_capture()
        with torch.cuda.graph(graph):
            toks, logits = self._decode_body(B, splits, want_logits, feedback)
        if fused is not None:
            fused.end_capture()
        return _DecodeGraph(graph, toks, logits, self.model.launches)
