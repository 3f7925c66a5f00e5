"""Host policy unit tests, re-deriving the reference's unit cases (scheduler, paging, prefix, speculative, sampler)."""
import math

import pytest

from inference_b200.contracts.core_llm import FinishReason
from inference_b200.policy.paging import BlockAllocator, OutOfBlocks
from inference_b200.policy.prefix import PrefixIndex
from inference_b200.policy.sampler import SamplingParams, SplitMix64, sample, shaped_candidates
from inference_b200.policy.schedule import Scheduler, SeqSpec
from inference_b200.policy.speculative import accept_greedy_run, accept_token, ngram_propose, sample_weighted


def test_scheduler_laws():
    s = Scheduler()
    a = s.admit(SeqSpec([1, 2, 3], 3, [99]))
    b = s.admit(SeqSpec([3], 8, [99]))
    z = s.admit(SeqSpec([1, 2], 0, []))
    assert (a, b, z) == (0, 1, 2) and s.active() == [0, 1] and s.finish_reason(z) is FinishReason.LENGTH
    assert s.offset(a) == 3
    assert s.record(a, 10) is None and s.offset(a) == 4
    assert s.record(b, 5) is None and s.record(b, 99) is FinishReason.STOP
    assert s.generated(b) == [5]
    assert s.record(a, 11) is None and s.record(a, 12) is FinishReason.LENGTH
    assert s.generated(a) == [10, 11, 12]
    assert s.record(a, 13) is None and s.generated(a) == [10, 11, 12]
    assert s.all_finished() and s.finished() == [0, 1, 2]


def test_block_allocator_lifo_and_cow():
    al = BlockAllocator(3)
    a, b = al.alloc(), al.alloc()
    assert (a, b) == (0, 1)
    al.retain(a)
    assert al.refcount(a) == 2 and al.shared_blocks() == 1
    al.release(a)
    al.release(a)
    assert al.refcount(a) == 0 and al.live_blocks() == 1
    assert al.alloc() == a  # LIFO recycle
    c = al.alloc()
    assert c == 2 and al.peak_live_blocks() == 3
    with pytest.raises(OutOfBlocks):
        al.alloc()
    with pytest.raises(ValueError):
        al.release(7)


def test_prefix_index():
    idx = PrefixIndex(2)
    assert idx.longest_match([1, 2, 3]) is None and idx.longest_match([]) is None
    a = idx.insert([1, 2, 3, 4, 5]).id
    m = idx.longest_match([1, 2, 3, 9])
    assert m.id == a and m.matched_len == 3
    assert idx.longest_match([7, 2, 3]) is None
    again = idx.insert([1, 2, 3, 4, 5])
    assert again.id == a and not again.evicted and len(idx) == 1
    b = idx.insert([1, 2]).id
    idx.longest_match([1, 2, 3, 4, 5, 6])  # touches a -> b becomes LRU
    out = idx.insert([8, 8])
    assert out.evicted == [b] and not idx.contains(b) and idx.contains(a)
    assert out.id not in (a, b)


def test_ngram_and_greedy_accept():
    assert ngram_propose([1, 2, 3, 1, 2], 3, 1) == [3]
    assert ngram_propose([1, 2, 3, 1, 2], 3, 3) == [3, 1, 2]
    assert ngram_propose([9, 1, 2, 4, 7, 9, 1, 2], 3, 1) == [4]
    assert ngram_propose([1, 2, 3, 4], 3, 4) == [] and ngram_propose([1], 3, 4) == []
    assert accept_greedy_run([1, 2, 9], [1, 2]) == 2
    assert accept_greedy_run([1, 5, 9], [1, 2]) == 1
    assert accept_greedy_run([9], []) == 0


def test_stochastic_acceptance_preserves_target_distribution():
    p = [(0, 0.5), (1, 0.3), (2, 0.2)]
    q = [(0, 0.2), (1, 0.7), (2, 0.1)]
    assert accept_token([(0, 0.9), (1, 0.1)], [(0, 1.0)], 0, 0.5, 0.0) == (True, 0)
    rng = SplitMix64(7)
    counts = {0: 0, 1: 0, 2: 0}
    n = 30000
    for _ in range(n):
        proposed = sample_weighted(q, rng.next_f32(), 0)
        _, tok = accept_token(p, q, proposed, rng.next_f32(), rng.next_f32())
        counts[tok] += 1
    for t, pt in p:
        assert abs(counts[t] / n - pt) < 0.015, counts


def test_splitmix_and_sampler():
    r = SplitMix64(0)
    assert r.next_u64() == 0xE220A8397B1DCDAF and r.next_u64() == 0x6E789E6AA1B965F4
    r = SplitMix64(42)
    assert all(0.0 <= r.next_f32() < 1.0 for _ in range(1000))
    logits = [0.1, 5.0, 0.2, -1.0]
    assert sample(logits, [], SamplingParams(), SplitMix64(0)) == 1
    # mask forces the best allowed token
    assert sample(logits, [], SamplingParams(), SplitMix64(0), allowed=[1, 0, 1, 1]) == 2
    # repetition penalty demotes a positive logit
    assert sample([2.0, 1.9], [0], SamplingParams(repetition_penalty=2.0, repetition_context=8), SplitMix64(0)) == 1
    # top-k = 1 is greedy regardless of temperature
    assert sample(logits, [], SamplingParams(temperature=1.5, top_k=1), SplitMix64(3)) == 1
    # seeded determinism and rough frequency
    pa = SamplingParams(temperature=1.0)
    seq1 = [sample([0.0, math.log(3.0)], [], pa, SplitMix64(s)) for s in range(2000)]
    seq2 = [sample([0.0, math.log(3.0)], [], pa, SplitMix64(s)) for s in range(2000)]
    assert seq1 == seq2 and abs(sum(seq1) / 2000 - 0.75) < 0.04
    cands = shaped_candidates([0.0, 1.0, 2.0, 3.0], [], SamplingParams(temperature=1.0, top_p=0.6))
    assert [c[0] for c in cands] == [3]  # e^0 / sum = 0.64 >= 0.6
    cands = shaped_candidates([0.0, 1.0, 2.0, 3.0], [], SamplingParams(temperature=1.0, top_k=2))
    assert sorted(c[0] for c in cands) == [2, 3]


def test_pipeline_shard_plan_splits_layers_contiguously():
    from inference_b200.models.pipeline import layer_blocks, shard_for_layer, shard_plan

    assert [shard_for_layer(i, 2, 4) for i in range(4)] == [0, 0, 1, 1]
    assert [shard_for_layer(i, 3, 8) for i in range(8)] == [0, 0, 0, 1, 1, 1, 2, 2]
    assert [shard_for_layer(i, 4, 2) for i in range(2)] == [0, 2]          # more shards than layers
    assert shard_for_layer(0, 1, 0) == 0
    assert layer_blocks(8, 3) == [range(0, 3), range(3, 6), range(6, 8)]
    assert layer_blocks(2, 4) == [range(0, 1), range(0, 0), range(1, 2), range(0, 0)]
    place = shard_plan(["d0", "d1"], 4)
    assert place("model.embed_tokens.weight") == "d0" and place("model.layers.1.mlp.up_proj.weight") == "d0"
    assert place("model.layers.2.self_attn.q_proj.weight") == "d1" and place("model.norm.weight") == "d1"
    assert place("lm_head.weight") == "d1" and place("something.else") == "d0"
