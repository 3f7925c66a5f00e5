"""Exactness laws of the generation loops on the CPU oracle backend with a tiny random-weight model."""
import pytest
import torch

from inference_b200.contracts.core_llm import CancelFlag, FinishReason
from inference_b200.engine.backend import OracleBackend
from inference_b200.engine.decode import (BatchExactness, ContinuousConfig, ContinuousRequest, GenerationConfig,
                                          PrefixCache, SpeculativeConfig, generate, generate_batch, generate_cached,
                                          generate_continuous, generate_draft_speculative, generate_prompt_lookup)
from inference_b200.models import ModelConfig
from inference_b200.models.oracle import OracleLlama, random_llama_weights
from inference_b200.policy.sampler import SamplingParams


def _model(seed=0, layers=2, hidden=32):
    cfg = ModelConfig(hidden_size=hidden, intermediate_size=64, num_layers=layers, num_heads=4, num_kv_heads=2,
                      head_dim=8, vocab_size=96, rope_theta=10000.0, tie_word_embeddings=True)
    return OracleBackend(OracleLlama(cfg, random_llama_weights(cfg, seed=seed, std=0.3)))


PROMPTS = [[1, 5, 9, 2, 7, 7, 3], [4, 4, 8], [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21], [2]]


def test_solo_matches_oracle_greedy():
    be = _model()
    ref, _ = be.model.generate_greedy(PROMPTS[0], 12)
    got = generate(be, PROMPTS[0], GenerationConfig(max_new_tokens=12))
    assert got.tokens == ref and got.finish_reason is FinishReason.LENGTH and got.prompt_tokens == 7


def test_stop_token_cancel_and_sink():
    be = _model()
    ref, _ = be.model.generate_greedy(PROMPTS[0], 12)
    r = generate(be, PROMPTS[0], GenerationConfig(max_new_tokens=12, stop_tokens=(ref[4],)))
    first = ref.index(ref[4])
    assert r.tokens == ref[:first] and r.finish_reason is FinishReason.STOP
    c = CancelFlag()
    seen = []

    def sink(t):
        seen.append(t)
        if len(seen) == 3:
            c.cancel()
        return True

    r = generate(be, PROMPTS[0], GenerationConfig(max_new_tokens=12, cancel=c), sink)
    assert r.tokens == ref[:3] and r.finish_reason is FinishReason.CANCELLED
    pre = CancelFlag()
    pre.cancel()
    assert generate(be, PROMPTS[0], GenerationConfig(max_new_tokens=4, cancel=pre)).finish_reason is FinishReason.CANCELLED


def test_seeded_sampling_is_deterministic():
    be = _model()
    cfg = GenerationConfig(max_new_tokens=10, sampling=SamplingParams(temperature=0.9, top_p=0.95), seed=7)
    a, b = generate(be, PROMPTS[1], cfg), generate(be, PROMPTS[1], cfg)
    assert a.tokens == b.tokens
    c = generate(be, PROMPTS[1], GenerationConfig(max_new_tokens=10, sampling=cfg.sampling, seed=8))
    assert len(c.tokens) == 10


def test_batched_equals_solo():
    be = _model()
    cfg = GenerationConfig(max_new_tokens=9)
    solo = [generate(be, p, cfg).tokens for p in PROMPTS]
    assert [r.tokens for r in generate_batch(be, PROMPTS, cfg)] == solo


@pytest.mark.parametrize("exact", [BatchExactness.EXACT, BatchExactness.THROUGHPUT])
def test_continuous_equals_solo(exact):
    be = _model()
    budgets = [5, 9, 3, 7]
    solo = [generate(be, p, GenerationConfig(max_new_tokens=b)).tokens for p, b in zip(PROMPTS, budgets)]
    reqs = [ContinuousRequest(p, b) for p, b in zip(PROMPTS, budgets)]
    streamed = {i: [] for i in range(4)}
    res = generate_continuous(be, reqs, ContinuousConfig(max_batch=2, exactness=exact),
                              sink=lambda i, t: streamed[i].append(t))
    assert [r.tokens for r in res] == solo
    assert [streamed[i] for i in range(4)] == solo
    assert all(r.finish_reason is FinishReason.LENGTH for r in res)


@pytest.mark.parametrize("chunk", [1, 3, 64])
def test_chunked_prefill_mixed_with_decode_equals_solo(chunk):
    """Prompt tokens enter in slices of `chunk` alongside the decode rows of running sequences: same tokens as solo
    runs, and no forward ever carries more than `chunk` prompt tokens once decode rows exist."""
    be = _model()
    budgets = [5, 9, 3, 7]
    solo = [generate(be, p, GenerationConfig(max_new_tokens=b)).tokens for p, b in zip(PROMPTS, budgets)]
    reqs = [ContinuousRequest(p, b) for p, b in zip(PROMPTS, budgets)]
    seen = []
    real = be.forward_greedy

    def spy(seqs, new):
        seen.append([len(n) for n in new])
        return real(seqs, new)
    be.forward_greedy = spy
    try:
        res = generate_continuous(be, reqs, ContinuousConfig(max_batch=3, prefill_chunk=chunk))
    finally:
        be.forward_greedy = real
    assert [r.tokens for r in res] == solo
    assert all(sum(n for n in step if n > 1) <= max(chunk, 1) or chunk >= 64 for step in seen)
    if chunk == 3:
        assert any(1 in step and any(n > 1 for n in step) for step in seen)       # decode rows rode with prompt slices
    if chunk == 1:
        assert all(all(n == 1 for n in step) for step in seen)


def test_prefix_cached_equals_cold():
    be = _model()
    cache = PrefixCache(be, capacity=2)
    cfg = GenerationConfig(max_new_tokens=6)
    sys_prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    p1, p2 = sys_prompt + [10, 11], sys_prompt + [20, 21, 22]
    cold1, cold2 = generate(be, p1, cfg).tokens, generate(be, p2, cfg).tokens
    assert generate_cached(be, cache, p1, cfg).tokens == cold1
    assert cache.stats.hits == 0
    assert generate_cached(be, cache, p2, cfg).tokens == cold2
    assert cache.stats.hits == 1 and cache.stats.reused_tokens == len(sys_prompt)
    assert generate_cached(be, cache, p1, cfg).tokens == cold1   # exact repeat: reuse all but the last token
    assert cache.stats.hits == 2 and cache.stats.reused_tokens == len(sys_prompt) + len(p1) - 1


def test_speculative_greedy_equals_plain_greedy():
    target, draft = _model(seed=0), _model(seed=0, layers=1)
    prompt = [1, 2, 3, 1, 2, 3, 1, 2]
    cfg = GenerationConfig(max_new_tokens=14)
    plain = generate(target, prompt, cfg).tokens
    r, st = generate_prompt_lookup(target, prompt, cfg, SpeculativeConfig(3, 4))
    assert r.tokens == plain and st.forwards >= 2 and st.accepted <= st.proposed
    r2, st2 = generate_draft_speculative(target, draft, prompt, cfg, SpeculativeConfig(3, 3))
    assert r2.tokens == plain and st2.proposed > 0
    same, st3 = generate_draft_speculative(target, _model(seed=0), prompt, cfg, SpeculativeConfig(3, 4))
    assert same.tokens == plain and st3.accepted == st3.proposed   # identical draft: everything accepted
    stop = plain[5]
    rs, _ = generate_prompt_lookup(target, prompt, GenerationConfig(max_new_tokens=14, stop_tokens=(stop,)))
    assert rs.tokens == plain[:plain.index(stop)] and rs.finish_reason is FinishReason.STOP


def test_speculative_stochastic_runs_and_is_seeded():
    target, draft = _model(seed=0), _model(seed=1, layers=1)
    cfg = GenerationConfig(max_new_tokens=12, sampling=SamplingParams(temperature=0.8, top_k=20), seed=3)
    a, sa = generate_draft_speculative(target, draft, [5, 6, 7], cfg)
    b, sb = generate_draft_speculative(target, draft, [5, 6, 7], cfg)
    assert a.tokens == b.tokens and len(a.tokens) == 12 and sa.proposed == sb.proposed


def test_repetition_penalty_window_includes_the_prompt():
    """The penalty window is prompt + generated tokens (candle-llm decode/stream.rs:210-285): build a prompt that
    contains the token plain greedy would pick first, so a strong penalty must change that pick, and check the
    solo, batched and speculative loops against a direct restatement."""
    import numpy as np

    from inference_b200.policy import sampler as hs

    be = _model(seed=3)
    base = [1, 5, 9, 2]
    first_plain = generate(be, base, GenerationConfig(max_new_tokens=1)).tokens[0]
    prompt = base[:-1] + [first_plain] + base[-1:]           # the would-be winner now sits in the prompt
    params = SamplingParams(temperature=0.0, repetition_penalty=50.0)
    cfg = GenerationConfig(max_new_tokens=6, sampling=params)

    # restatement: greedy over penalised logits, window = prompt + generated
    seq = be.new_sequence()
    logits = be.forward([seq], [prompt])[0]
    hist, want = list(prompt), []
    rng = hs.SplitMix64(0)
    for _ in range(6):
        t = hs.sample(logits.float().numpy(), hist, params, rng, None)
        want.append(t)
        hist.append(t)
        logits = be.forward([seq], [[t]])[0]
    be.release(seq)
    plain_first = int(np.argmax(be.forward([be.new_sequence()], [prompt])[0].float().numpy()))

    got = generate(be, prompt, cfg)
    assert got.tokens == want
    if plain_first in prompt:
        assert got.tokens[0] != plain_first                   # a prompt token lost its lead to the penalty
    assert generate_batch(be, [prompt, PROMPTS[1]], cfg)[0].tokens == want
    spec, _ = generate_prompt_lookup(be, prompt, cfg, SpeculativeConfig(max_ngram=2, num_draft=3))
    assert spec.tokens == want
    draft = _model(seed=3)
    dspec, _ = generate_draft_speculative(be, draft, prompt, cfg, SpeculativeConfig(num_draft=3))
    assert dspec.tokens == want
