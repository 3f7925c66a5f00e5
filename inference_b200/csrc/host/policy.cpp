// Tensor-free host policy of the LLM engine, C ABI (loaded by ctypes, linkable from C / Rust):
// refcounted KV block allocator, continuous-batching scheduler, LRU prefix index, speculative-decoding
// acceptance math and the host token sampler. Behavioural parity targets: core-llm/src/paging.rs:42-127,
// schedule.rs:49-223, prefix.rs:43-176, speculative.rs:32-156, candle-llm/src/primitives/sampler.rs:19-256.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <limits>
#include <queue>
#include <vector>

#define SWB_API extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------------
// Block allocator: dense ids, LIFO recycle, reference counts for copy-on-write sharing.
// ------------------------------------------------------------------------------------------------
struct BlockAllocator {
  long capacity;  // < 0: unbounded
  std::vector<int> refs;
  std::vector<int> free_list;
  long live = 0, peak = 0;
};

SWB_API void* swb_alloc_new(long capacity) {
  auto* a = new BlockAllocator();
  a->capacity = capacity;
  return a;
}
SWB_API void swb_alloc_free(void* h) { delete static_cast<BlockAllocator*>(h); }
SWB_API long swb_alloc_alloc(void* h) {
  auto* a = static_cast<BlockAllocator*>(h);
  long b;
  if (!a->free_list.empty()) {
    b = a->free_list.back();
    a->free_list.pop_back();
  } else {
    if (a->capacity >= 0 && (long)a->refs.size() >= a->capacity) return -1;
    b = (long)a->refs.size();
    a->refs.push_back(0);
  }
  a->refs[b] = 1;
  a->live += 1;
  a->peak = std::max(a->peak, a->live);
  return b;
}
SWB_API int swb_alloc_retain(void* h, long b) {
  auto* a = static_cast<BlockAllocator*>(h);
  if (b < 0 || b >= (long)a->refs.size() || a->refs[b] <= 0) return -1;
  a->refs[b] += 1;
  return 0;
}
SWB_API int swb_alloc_release(void* h, long b) {
  auto* a = static_cast<BlockAllocator*>(h);
  if (b < 0 || b >= (long)a->refs.size() || a->refs[b] <= 0) return -1;
  if (--a->refs[b] == 0) {
    a->free_list.push_back((int)b);
    a->live -= 1;
  }
  return 0;
}
SWB_API int swb_alloc_refcount(void* h, long b) {
  auto* a = static_cast<BlockAllocator*>(h);
  return (b >= 0 && b < (long)a->refs.size()) ? a->refs[b] : 0;
}
SWB_API long swb_alloc_live(void* h) { return static_cast<BlockAllocator*>(h)->live; }
SWB_API long swb_alloc_peak(void* h) { return static_cast<BlockAllocator*>(h)->peak; }
SWB_API long swb_alloc_shared(void* h) {
  auto* a = static_cast<BlockAllocator*>(h);
  long n = 0;
  for (int r : a->refs) n += r > 1;
  return n;
}
SWB_API long swb_alloc_capacity(void* h) { return static_cast<BlockAllocator*>(h)->capacity; }

// ------------------------------------------------------------------------------------------------
// Scheduler: per-sequence budget / stop-token bookkeeping for iteration-level batching.
// finish reasons: 0 none, 1 stop, 2 length
// ------------------------------------------------------------------------------------------------
struct SeqState {
  size_t prompt_len;
  std::vector<int32_t> generated;
  size_t max_new;
  std::vector<int32_t> stops;
  int finish;
};
struct Scheduler {
  std::vector<SeqState> seqs;
};

SWB_API void* swb_sched_new() { return new Scheduler(); }
SWB_API void swb_sched_free(void* h) { delete static_cast<Scheduler*>(h); }
SWB_API long swb_sched_admit(void* h, long prompt_len, long max_new, const int32_t* stops, long n_stops) {
  auto* s = static_cast<Scheduler*>(h);
  SeqState st;
  st.prompt_len = (size_t)prompt_len;
  st.max_new = (size_t)max_new;
  st.stops.assign(stops, stops + n_stops);
  st.finish = max_new == 0 ? 2 : 0;  // a zero budget is admitted already finished
  s->seqs.push_back(std::move(st));
  return (long)s->seqs.size() - 1;
}
SWB_API long swb_sched_len(void* h) { return (long)static_cast<Scheduler*>(h)->seqs.size(); }
// Records a sampled token: returns 1 (stop: token excluded), 2 (length: token included), 0 (continue),
// -1 (unknown or already finished sequence: no-op).
SWB_API int swb_sched_record(void* h, long id, int32_t token) {
  auto* s = static_cast<Scheduler*>(h);
  if (id < 0 || id >= (long)s->seqs.size()) return -1;
  SeqState& st = s->seqs[id];
  if (st.finish) return -1;
  if (std::find(st.stops.begin(), st.stops.end(), token) != st.stops.end()) {
    st.finish = 1;
    return 1;
  }
  st.generated.push_back(token);
  if (st.generated.size() >= st.max_new) {
    st.finish = 2;
    return 2;
  }
  return 0;
}
SWB_API int swb_sched_finish_reason(void* h, long id) {
  auto* s = static_cast<Scheduler*>(h);
  return (id >= 0 && id < (long)s->seqs.size()) ? s->seqs[id].finish : 0;
}
SWB_API long swb_sched_generated(void* h, long id, int32_t* out, long cap) {
  auto* s = static_cast<Scheduler*>(h);
  if (id < 0 || id >= (long)s->seqs.size()) return 0;
  const auto& g = s->seqs[id].generated;
  const long n = std::min<long>(cap, (long)g.size());
  if (out && n > 0) std::memcpy(out, g.data(), n * sizeof(int32_t));
  return (long)g.size();
}
SWB_API long swb_sched_prompt_len(void* h, long id) {
  auto* s = static_cast<Scheduler*>(h);
  return (id >= 0 && id < (long)s->seqs.size()) ? (long)s->seqs[id].prompt_len : 0;
}
SWB_API long swb_sched_offset(void* h, long id) {
  auto* s = static_cast<Scheduler*>(h);
  return (id >= 0 && id < (long)s->seqs.size()) ? (long)(s->seqs[id].prompt_len + s->seqs[id].generated.size()) : 0;
}
// Writes the ids of active (finished == 0) or finished (finished == 1) sequences; returns their count.
SWB_API long swb_sched_list(void* h, int finished, long* out, long cap) {
  auto* s = static_cast<Scheduler*>(h);
  long n = 0;
  for (size_t i = 0; i < s->seqs.size(); ++i) {
    if ((s->seqs[i].finish != 0) == (finished != 0)) {
      if (out && n < cap) out[n] = (long)i;
      ++n;
    }
  }
  return n;
}

// ------------------------------------------------------------------------------------------------
// Prefix index: token-granular longest-common-prefix lookup with LRU eviction; ids are never reused.
// ------------------------------------------------------------------------------------------------
struct PrefixEntry {
  uint64_t id;
  std::vector<int32_t> tokens;
};
struct PrefixIndex {
  size_t capacity;
  uint64_t next_id = 0;
  std::deque<PrefixEntry> entries;  // front = least recently used
};

SWB_API void* swb_prefix_new(long capacity) {
  auto* p = new PrefixIndex();
  p->capacity = (size_t)std::max<long>(0, capacity);
  return p;
}
SWB_API void swb_prefix_free(void* h) { delete static_cast<PrefixIndex*>(h); }
SWB_API long swb_prefix_len(void* h) { return (long)static_cast<PrefixIndex*>(h)->entries.size(); }
SWB_API int swb_prefix_contains(void* h, uint64_t id) {
  for (auto& e : static_cast<PrefixIndex*>(h)->entries)
    if (e.id == id) return 1;
  return 0;
}
static uint64_t prefix_touch(PrefixIndex* p, size_t idx) {
  PrefixEntry e = std::move(p->entries[idx]);
  p->entries.erase(p->entries.begin() + (long)idx);
  uint64_t id = e.id;
  p->entries.push_back(std::move(e));
  return id;
}
// Longest stored entry sharing a non-empty prefix with tokens (most recently used wins ties); marks it used.
// Returns 1 and fills id / matched_len, or 0 on a miss.
SWB_API int swb_prefix_longest_match(void* h, const int32_t* tokens, long n, uint64_t* id, long* matched_len) {
  auto* p = static_cast<PrefixIndex*>(h);
  if (n <= 0) return 0;
  long best_idx = -1;
  size_t best_len = 0;
  for (long i = (long)p->entries.size() - 1; i >= 0; --i) {
    const auto& t = p->entries[i].tokens;
    size_t m = 0, lim = std::min<size_t>(t.size(), (size_t)n);
    while (m < lim && t[m] == tokens[m]) ++m;
    if (m > 0 && m > best_len) {
      best_len = m;
      best_idx = i;
    }
  }
  if (best_idx < 0) return 0;
  *id = prefix_touch(p, (size_t)best_idx);
  *matched_len = (long)best_len;
  return 1;
}
// Inserts (or refreshes an identical entry); evicted ids are written to `evicted` (cap entries). Returns the
// number evicted; *id receives the entry id.
SWB_API long swb_prefix_insert(void* h, const int32_t* tokens, long n, uint64_t* id, uint64_t* evicted, long cap) {
  auto* p = static_cast<PrefixIndex*>(h);
  for (size_t i = 0; i < p->entries.size(); ++i) {
    const auto& t = p->entries[i].tokens;
    if ((long)t.size() == n && std::equal(t.begin(), t.end(), tokens)) {
      *id = prefix_touch(p, i);
      return 0;
    }
  }
  PrefixEntry e;
  e.id = p->next_id++;
  e.tokens.assign(tokens, tokens + n);
  *id = e.id;
  p->entries.push_back(std::move(e));
  long n_ev = 0;
  while (p->entries.size() > p->capacity) {
    if (evicted && n_ev < cap) evicted[n_ev] = p->entries.front().id;
    ++n_ev;
    p->entries.pop_front();
  }
  return n_ev;
}

// ------------------------------------------------------------------------------------------------
// Speculative decoding policy (RNG-free: uniform draws are passed in).
// ------------------------------------------------------------------------------------------------
// Prompt-lookup proposer: longest n-gram suffix (n <= max_ngram) that re-occurs earlier, most recent match first;
// proposes up to max_proposal tokens that followed it. Returns the number written to out.
SWB_API long swb_ngram_propose(const int32_t* tokens, long len, long max_ngram, long max_proposal, int32_t* out) {
  if (len < 2 || max_ngram <= 0 || max_proposal <= 0) return 0;
  const long max_n = std::min(max_ngram, len - 1);
  for (long n = max_n; n >= 1; --n) {
    const int32_t* suffix = tokens + (len - n);
    for (long start = len - n - 1; start >= 0; --start) {
      if (std::equal(suffix, suffix + n, tokens + start)) {
        const long from = start + n;
        const long to = std::min(from + max_proposal, len);
        if (from < to) {
          std::copy(tokens + from, tokens + to, out);
          return to - from;
        }
      }
    }
  }
  return 0;
}
// Length of the longest prefix of drafts equal to the target argmaxes (target has one extra bonus slot).
SWB_API long swb_accept_greedy_run(const int32_t* target_argmax, const int32_t* drafts, long n_drafts) {
  long a = 0;
  while (a < n_drafts && target_argmax[a] == drafts[a]) ++a;
  return a;
}
static float weight_of(const int32_t* ids, const float* w, long n, int32_t t) {
  for (long i = 0; i < n; ++i)
    if (ids[i] == t) return w[i];
  return 0.f;
}
SWB_API int32_t swb_sample_weighted(const int32_t* ids, const float* w, long n, float u, int32_t fallback) {
  float total = 0.f;
  for (long i = 0; i < n; ++i) total += std::max(w[i], 0.f);
  if (!(total > 0.f)) return fallback;
  float target = std::min(std::max(u, 0.f), 1.f) * total;
  for (long i = 0; i < n; ++i) {
    target -= std::max(w[i], 0.f);
    if (target <= 0.f) return ids[i];
  }
  return n > 0 ? ids[n - 1] : fallback;
}
// Distribution-preserving acceptance of one proposed token: accept with probability min(1, p/q), otherwise
// resample from the normalised residual max(0, p - q). Returns 1 accepted / 0 rejected; *token is the result.
SWB_API int swb_accept_token(const int32_t* t_ids, const float* t_w, long nt, const int32_t* d_ids, const float* d_w,
                             long nd, int32_t proposed, float u_accept, float u_resample, int32_t* token) {
  float p_total = 0.f, q_total = 0.f;
  for (long i = 0; i < nt; ++i) p_total += std::max(t_w[i], 0.f);
  for (long i = 0; i < nd; ++i) q_total += std::max(d_w[i], 0.f);
  const float pmin = std::numeric_limits<float>::min();
  auto p_of = [&](int32_t t) { return std::max(weight_of(t_ids, t_w, nt, t), 0.f) / std::max(p_total, pmin); };
  auto q_of = [&](int32_t t) { return std::max(weight_of(d_ids, d_w, nd, t), 0.f) / std::max(q_total, pmin); };
  const float p_t = p_of(proposed), q_t = q_of(proposed);
  const float accept_prob = q_t > 0.f ? std::min(p_t / q_t, 1.f) : 1.f;
  if (u_accept < accept_prob) {
    *token = proposed;
    return 1;
  }
  std::vector<int32_t> r_ids;
  std::vector<float> r_w;
  auto consider = [&](int32_t t) {
    if (std::find(r_ids.begin(), r_ids.end(), t) != r_ids.end()) return;
    const float r = p_of(t) - q_of(t);
    if (r > 0.f) {
      r_ids.push_back(t);
      r_w.push_back(r);
    }
  };
  // the residual keeps first-seen order over target then draft supports (tokens with r <= 0 may be revisited,
  // which is harmless: they are never added)
  for (long i = 0; i < nt; ++i) consider(t_ids[i]);
  for (long i = 0; i < nd; ++i) consider(d_ids[i]);
  *token = swb_sample_weighted(r_ids.data(), r_w.data(), (long)r_ids.size(), u_resample, proposed);
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Host sampler: SplitMix64, repetition penalty, temperature, top-k, top-p nucleus, inverse-CDF draw.
// ------------------------------------------------------------------------------------------------
SWB_API uint64_t swb_splitmix64_next(uint64_t* state) {
  *state += 0x9E3779B97F4A7C15ULL;
  uint64_t z = *state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
SWB_API float swb_splitmix64_next_f32(uint64_t* state) {
  return (float)(swb_splitmix64_next(state) >> 40) / (float)(1ULL << 24);
}

namespace {
struct Cand {
  int32_t id;
  float w;
};
// descending weight, ties to the lower index
inline bool cand_before(const Cand& a, const Cand& b) { return a.w > b.w || (a.w == b.w && a.id < b.id); }

void apply_mask_and_penalty(std::vector<float>& v, const uint8_t* allowed, long n_allowed, const int32_t* history,
                            long n_hist, float rep_penalty, long rep_context) {
  const long V = (long)v.size();
  if (allowed)
    for (long i = 0; i < V; ++i)
      if (i >= n_allowed || !allowed[i]) v[i] = -INFINITY;
  if (rep_penalty != 1.f && rep_context > 0) {
    const long start = std::max<long>(0, n_hist - rep_context);
    for (long k = start; k < n_hist; ++k) {
      const int32_t t = history[k];
      if (t >= 0 && t < V) v[t] = v[t] < 0.f ? v[t] * rep_penalty : v[t] / rep_penalty;
    }
  }
}

int32_t argmax_host(const std::vector<float>& v) {
  long best = 0;
  float bv = -INFINITY;
  for (long i = 0; i < (long)v.size(); ++i)
    if (v[i] > bv) {
      bv = v[i];
      best = i;
    }
  return (int32_t)best;
}

std::vector<Cand> nucleus_weights(const std::vector<float>& v, float temperature, long top_k, float top_p) {
  float mx = -INFINITY;
  for (float x : v) mx = std::max(mx, x);
  std::vector<Cand> w;
  if (!std::isfinite(mx)) return w;
  const float inv_t = 1.f / temperature;
  w.resize(v.size());
  for (size_t i = 0; i < v.size(); ++i) w[i] = Cand{(int32_t)i, std::exp((v[i] - mx) * inv_t)};
  if (top_k > 0 && top_k < (long)w.size()) {
    std::nth_element(w.begin(), w.begin() + (top_k - 1), w.end(), cand_before);
    w.resize((size_t)top_k);
  }
  if (top_p < 1.f) {
    float total = 0.f;
    for (auto& c : w) total += c.w;
    const float threshold = std::max(top_p, 0.f) * total;
    auto heap_less = [](const Cand& a, const Cand& b) { return cand_before(b, a); };
    std::priority_queue<Cand, std::vector<Cand>, decltype(heap_less)> heap(heap_less, w);
    std::vector<Cand> kept;
    float cum = 0.f;
    while (!heap.empty()) {
      Cand c = heap.top();
      heap.pop();
      kept.push_back(c);
      cum += c.w;
      if (cum >= threshold) break;
    }
    w.swap(kept);
  }
  return w;
}
}  // namespace

// Samples one token from fp32 logits[V]. allowed (optional, uint8[n_allowed]) masks the vocabulary, history is
// the generated-token window for the repetition penalty; *rng_state is a SplitMix64 state advanced only when a
// stochastic draw happens.
SWB_API int32_t swb_sample(const float* logits, long V, const int32_t* history, long n_hist, float temperature,
                           float top_p, long top_k, float rep_penalty, long rep_context, const uint8_t* allowed,
                           long n_allowed, uint64_t* rng_state) {
  std::vector<float> v(logits, logits + V);
  apply_mask_and_penalty(v, allowed, n_allowed, history, n_hist, rep_penalty, rep_context);
  if (temperature <= 0.f) return argmax_host(v);
  std::vector<Cand> w = nucleus_weights(v, temperature, top_k, top_p);
  float total = 0.f;
  for (auto& c : w) total += c.w;
  if (!(total > 0.f) || !std::isfinite(total)) return argmax_host(v);
  float target = swb_splitmix64_next_f32(rng_state) * total;
  for (auto& c : w) {
    target -= c.w;
    if (target <= 0.f) return c.id;
  }
  return w.empty() ? 0 : w.back().id;
}

// The shaped candidate distribution (ids + unnormalised weights) the stochastic sampler draws from; used by
// speculative decoding to record q_i / p_i. Returns the candidate count (writes up to cap).
SWB_API long swb_shaped_candidates(const float* logits, long V, const int32_t* history, long n_hist, float temperature,
                                   float top_p, long top_k, float rep_penalty, long rep_context,
                                   const uint8_t* allowed, long n_allowed, int32_t* out_ids, float* out_w, long cap) {
  std::vector<float> v(logits, logits + V);
  apply_mask_and_penalty(v, allowed, n_allowed, history, n_hist, rep_penalty, rep_context);
  std::vector<Cand> w = nucleus_weights(v, temperature > 0.f ? temperature : 1.f, top_k, top_p);
  const long n = std::min<long>(cap, (long)w.size());
  for (long i = 0; i < n; ++i) {
    out_ids[i] = w[i].id;
    out_w[i] = w[i].w;
  }
  return (long)w.size();
}
