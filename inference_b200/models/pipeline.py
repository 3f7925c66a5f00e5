"""Pipeline-sharded load: a decoder too large for one GPU split into contiguous layer blocks, one per device, inside
one process (the reference's only multi-GPU strategy: candle-llm/src/models/llama.rs:321-348, 728-753).

Layer i of L goes to shard min(i * S / L, S - 1); the token embeddings live on the first device, the final norm and
output head on the last. Each stage is an ordinary `LlamaGpu` holding only its layers; the hidden state (residual
stream + pending branch output) crosses each boundary with one peer copy. This is a capacity option, not a
throughput one - tensor parallelism (`parallel/`) is the fast path - so steps run eagerly, stage after stage."""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from ..contracts.errors import LoadError
from .config import ModelConfig
from .llama import LlamaGpu, StepInputs


def shard_for_layer(layer: int, num_shards: int, num_layers: int) -> int:
    return min(layer * num_shards // max(num_layers, 1), max(num_shards - 1, 0))


def shard_plan(devices: Sequence, num_layers: int) -> Callable[[str], object]:
    """key -> device: decoder layers by contiguous block, `model.norm` / `lm_head` on the last device, the token
    embeddings and anything else on the first."""
    if not devices:
        raise LoadError("shard_plan: needs at least one device")

    def place(key: str):
        if key.startswith("model.layers."):
            idx = key[len("model.layers."):].split(".", 1)[0]
            if idx.isdigit():
                return devices[shard_for_layer(int(idx), len(devices), num_layers)]
        if key.startswith(("model.norm", "lm_head")):
            return devices[-1]
        return devices[0]
    return place


def layer_blocks(num_layers: int, num_shards: int) -> list[range]:
    """The contiguous layer range of every shard (empty ranges when there are more shards than layers)."""
    owner = [shard_for_layer(i, num_shards, num_layers) for i in range(num_layers)]
    out = []
    for s in range(num_shards):
        mine = [i for i, o in enumerate(owner) if o == s]
        out.append(range(mine[0], mine[-1] + 1) if mine else range(0, 0))
    return out


class ShardedKvPool:
    """One paged KV tensor per stage, all addressed by the same block ids (one allocator), so block tables and slot
    mappings are valid on every device."""

    def __init__(self, blocks: list[range], num_blocks: int, kv_heads: int, head_dim: int, devices, block_size: int = 16):
        from ..policy.paging import BlockAllocator

        self.num_layers = sum(len(b) for b in blocks)
        self.num_blocks, self.block_size, self.kv_heads, self.head_dim = num_blocks, block_size, kv_heads, head_dim
        self.data = [torch.zeros((max(1, len(b)), 2, num_blocks, kv_heads, block_size, head_dim), dtype=torch.bfloat16,
                                 device=d) for b, d in zip(blocks, devices)]
        self.allocator = BlockAllocator(num_blocks)

    @property
    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.data)

    def copy_block(self, src: int, dst: int) -> None:
        for t in self.data:
            t[:, :, dst].copy_(t[:, :, src])


class PipelineLlama:
    """The `LlamaGpu` surface the model runner uses (`forward_hidden`, `logits`, `greedy_tokens`, `ensure_rope`),
    over stages on several devices."""

    def __init__(self, cfg: ModelConfig, devices: Sequence[torch.device | str]):
        if not devices:
            raise LoadError("from_dir_sharded: needs at least one device")
        self.cfg = cfg
        self.devices = [torch.device(d) for d in devices]
        self.blocks = layer_blocks(cfg.num_layers, len(self.devices))
        self.stages = [LlamaGpu(cfg, device=d) for d in self.devices]
        self.device = self.devices[0]
        self.comm = self.stages[0].comm
        self.hq, self.hkv = self.stages[0].hq, self.stages[0].hkv
        self.launches = 0
        self.has_moe = False
        self.eager_only = True          # steps cross devices stage by stage; no single-device graph to capture

    def load_state_dict(self, weights: dict[str, torch.Tensor]) -> "PipelineLlama":
        last = len(self.stages) - 1
        for s, (st, blk) in enumerate(zip(self.stages, self.blocks)):
            with torch.cuda.device(st.device) if st.device.type == "cuda" else _null():
                st.load_state_dict(weights, layers=blk, with_embed=s == 0, with_head=s == last)
        self.has_moe = any(st.has_moe for st in self.stages)
        return self

    def layer_devices(self) -> list[torch.device]:
        return [self.devices[shard_for_layer(i, len(self.devices), self.cfg.num_layers)]
                for i in range(self.cfg.num_layers)]

    def make_pool(self, num_blocks: int, block_size: int = 16) -> ShardedKvPool:
        return ShardedKvPool(self.blocks, num_blocks, self.hkv, self.cfg.head_dim, self.devices, block_size)

    def ensure_rope(self, n: int) -> None:
        for st in self.stages:
            st.ensure_rope(n)

    @staticmethod
    def _inputs_on(inp: StepInputs, dev: torch.device) -> StepInputs:
        mv = lambda t: t.to(dev, non_blocking=True) if t is not None else None
        return StepInputs(input_ids=mv(inp.input_ids), positions=mv(inp.positions), slot_mapping=mv(inp.slot_mapping),
                          block_table=mv(inp.block_table), kv_lens=mv(inp.kv_lens), cu_q=mv(inp.cu_q),
                          max_q_len=inp.max_q_len, num_seqs=inp.num_seqs, decode=inp.decode,
                          attn_splits=inp.attn_splits, logits_rows=mv(inp.logits_rows),
                          fresh_prefill=inp.fresh_prefill, embed_rows=mv(inp.embed_rows),
                          embed_values=mv(inp.embed_values))

    def forward_hidden(self, inp: StepInputs, kv_pools: list[torch.Tensor]) -> torch.Tensor:
        carry = None
        n = 0
        last = len(self.stages) - 1
        out = None
        for s, st in enumerate(self.stages):
            local = inp if st.device == inp.input_ids.device else self._inputs_on(inp, st.device)
            with torch.cuda.device(st.device) if st.device.type == "cuda" else _null():
                if carry is not None:
                    carry = tuple(t.to(st.device, non_blocking=True) if t is not None else None for t in carry)
                if len(self.blocks[s]) == 0 and s != last:
                    if carry is None:                  # an empty first stage still owns the embedding
                        carry = st.forward_hidden(local, kv_pools[s], last_stage=False)
                    continue
                r = st.forward_hidden(local, kv_pools[s], stage_in=carry, last_stage=s == last)
                n += st.launches
            if s == last:
                out = r
            else:
                carry = r
        self.launches = n
        return out.to(self.device)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        st = self.stages[-1]
        with torch.cuda.device(st.device) if st.device.type == "cuda" else _null():
            return st.logits(hidden.to(st.device)).to(self.device)

    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        st = self.stages[-1]
        with torch.cuda.device(st.device) if st.device.type == "cuda" else _null():
            return st.greedy_tokens(hidden.to(st.device)).to(self.device)

    def weight_bytes(self) -> list[int]:
        """Resident weight bytes per device."""
        out = []
        for s, st in enumerate(self.stages):
            n = sum(2 * t.numel() for L in st.layers for t in (L.qkv, L.o, L.gate_up, L.down, L.ln1, L.ln2)
                    if isinstance(t, torch.Tensor))
            n += 2 * st.embed.numel() if st.embed is not None else 0
            n += 2 * st.lm_head.numel() if st.lm_head is not None else 0
            out.append(n)
        return out


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def from_dir_sharded(path, devices: Sequence[torch.device | str]) -> PipelineLlama:
    """Loads a Hugging Face snapshot directory pipeline-sharded over `devices` (dense bf16; not combined with
    quantise-on-load - use one or the other to fit)."""
    from ..io.safetensors_io import load_dir

    cfg = ModelConfig.from_dir(path)
    return PipelineLlama(cfg, devices).load_state_dict(load_dir(path))
