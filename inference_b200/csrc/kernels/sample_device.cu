// Temperature / top-k / top-p sampling on the device: one 1024-thread block per row, the row never leaves the GPU.
//
// The host sampler (policy/sampler.py, the reference's candle-llm/src/primitives/sampler.rs) needs the whole logits
// row on the host: 513 KB per sequence and step at a 128 K vocabulary. This kernel draws from the same distribution
// - softmax of logits / temperature, restricted to the k largest weights and to the smallest set of largest weights
// whose mass reaches top_p, renormalised - with the row read a few times from L2 and 8 bytes written back.
// The caller supplies one uniform number per row (from its own generator), so runs are reproducible; the mapping
// from that number to a token is by token index over the kept set, not by the host sampler's weight order, so the
// two samplers agree in distribution, not token by token.
//
// Passes over the row (each thread owns one contiguous chunk, weights are recomputed as exp((l - max) / T) by the
// same expression every time, so every pass sees identical values):
//   1. maximum of the allowed logits            2. Z = sum of weights
//   3-5. radix select (11 + 11 + 10 bits of the weight's bit pattern, largest first) of the threshold weight at which
//        the kept count reaches top_k or the kept mass reaches top_p * Z, whichever comes first; ties at the threshold
//        are admitted in index order
//   6. inverse CDF over the kept set in index order at u * (kept mass)
// top_k <= 0 and top_p >= 1 skip passes 3-5. A row without any allowed finite logit yields token 0.
#include "common.cuh"

namespace swb {

SWB_REGISTER_STATUS_UNIT(sample_device);

namespace {

constexpr int SD_THREADS = 1024;
constexpr int SD_BINS = 2048;

template <typename T>
__device__ __forceinline__ float sd_load(const T* x, long long i);
template <>
__device__ __forceinline__ float sd_load<float>(const float* x, long long i) { return x[i]; }
template <>
__device__ __forceinline__ float sd_load<bf16>(const bf16* x, long long i) { return __bfloat162float(x[i]); }

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[threadIdx.x & 31];
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  return v;
}

// exclusive scan of one value per thread across the block (index order); returns the exclusive prefix, *total = sum
template <typename V>
__device__ __forceinline__ V block_excl_scan(V v, V* warp_tot, V* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  V inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    const V n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  V wv = warp_tot[lane], winc = wv;
  for (int o = 1; o < 32; o <<= 1) {
    const V n = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += n;
  }
  const V warp_off = __shfl_sync(0xffffffffu, winc - wv, warp);
  *total = __shfl_sync(0xffffffffu, winc, 31);
  return warp_off + inc - v;
}

template <typename T>
__global__ void __launch_bounds__(SD_THREADS) sample_device_kernel(const T* __restrict__ logits, long long ld, int V,
                                                                   float inv_temp, int top_k, float top_p,
                                                                   const float* __restrict__ uniforms,
                                                                   const uint8_t* __restrict__ allow, long long* out_ids,
                                                                   float* out_prob) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  __shared__ unsigned int h_cnt[SD_BINS];
  __shared__ float h_sum[SD_BINS];
  __shared__ float scan_f[32];
  __shared__ unsigned int scan_u[32];
  __shared__ unsigned int s_prefix, s_take_ties;
  __shared__ float s_mass_above;
  __shared__ unsigned int s_cnt_above;

  const int row = blockIdx.x;
  const T* x = logits + (size_t)row * ld;
  const long long per = ((long long)V + SD_THREADS - 1) / SD_THREADS;
  const long long i0 = min((long long)V, (long long)threadIdx.x * per), i1 = min((long long)V, i0 + per);
  auto allowed = [&](long long i, float l) { return (!allow || allow[i]) && l == l && l > -INFINITY; };

  float m = -INFINITY;
  for (long long i = i0; i < i1; ++i) {
    const float l = sd_load<T>(x, i);
    if (allowed(i, l)) m = fmaxf(m, l);
  }
  m = block_reduce(m, red, true);
  if (!(m > -INFINITY)) {
    if (threadIdx.x == 0) {
      out_ids[row] = 0;
      if (out_prob) out_prob[row] = 0.f;
    }
    return;
  }
  auto weight = [&](long long i) -> float {
    const float l = sd_load<T>(x, i);
    return allowed(i, l) ? __expf((l - m) * inv_temp) : 0.f;
  };
  float z = 0.f;
  for (long long i = i0; i < i1; ++i) z += weight(i);
  z = block_reduce(z, red, false);

  // ---- threshold: bit pattern `thr` such that weights with pattern > thr are kept, == thr kept for the first
  //      s_take_ties of them in index order ----
  const bool filter = (top_k > 0 && top_k < V) || top_p < 1.f;
  unsigned int thr = 0u;          // keep everything with a positive weight by default
  if (filter) {
    const unsigned int want_k = top_k > 0 ? (unsigned int)top_k : 0xFFFFFFFFu;
    const float want_mass = top_p < 1.f ? top_p * z : INFINITY;
    if (threadIdx.x == 0) {
      s_prefix = 0u;
      s_cnt_above = 0u;
      s_mass_above = 0.f;
    }
    const int shifts[3] = {21, 10, 0}, widths[3] = {11, 11, 10};
    for (int r = 0; r < 3; ++r) {
      for (int b = threadIdx.x; b < SD_BINS; b += SD_THREADS) {
        h_cnt[b] = 0u;
        h_sum[b] = 0.f;
      }
      __syncthreads();
      const unsigned int prefix = s_prefix;
      const int sh = shifts[r], wd = widths[r];
      const unsigned int hi_mask = r == 0 ? 0u : (0xFFFFFFFFu << (sh + wd));
      for (long long i = i0; i < i1; ++i) {
        const float w = weight(i);
        if (w <= 0.f) continue;
        const unsigned int bits = __float_as_uint(w);
        if ((bits & hi_mask) != prefix) continue;
        const unsigned int bin = (bits >> sh) & ((1u << wd) - 1u);
        atomicAdd(&h_cnt[bin], 1u);
        atomicAdd(&h_sum[bin], w);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned int cnt = s_cnt_above;
        float mass = s_mass_above;
        int b = (1 << wd) - 1;
        for (; b > 0; --b) {
          if (h_cnt[b] == 0u) continue;
          if (cnt + h_cnt[b] >= want_k || mass + h_sum[b] >= want_mass) break;
          cnt += h_cnt[b];
          mass += h_sum[b];
        }
        // bin b holds the threshold (or b == 0: the last bin, taken whole below if still short)
        s_cnt_above = cnt;
        s_mass_above = mass;
        s_prefix = prefix | ((unsigned int)b << sh);
      }
      __syncthreads();
    }
    thr = s_prefix;
    if (threadIdx.x == 0) {
      // all weights with pattern == thr are equal: admit as many as the count / mass budget still needs (at least one)
      const float wt = __uint_as_float(thr);
      unsigned int need_k = want_k > s_cnt_above ? want_k - s_cnt_above : 0u;
      unsigned int need_p = 0xFFFFFFFFu;
      if (want_mass < INFINITY && wt > 0.f) {
        const float short_mass = want_mass - s_mass_above;
        need_p = short_mass > 0.f ? (unsigned int)ceilf(short_mass / wt) : 0u;
      }
      unsigned int take = min(need_k, need_p);
      s_take_ties = max(take, (s_cnt_above == 0u) ? 1u : 0u);
    }
    __syncthreads();
  }
  const unsigned int take_ties = filter ? s_take_ties : 0xFFFFFFFFu;

  // ---- draw: kept mass, then inverse CDF in index order ----
  unsigned int my_ties = 0u;
  if (filter)
    for (long long i = i0; i < i1; ++i) my_ties += (__float_as_uint(weight(i)) == thr && thr != 0u) ? 1u : 0u;
  unsigned int tie_total = 0u;
  unsigned int tie_rank = filter ? block_excl_scan<unsigned int>(my_ties, scan_u, &tie_total) : 0u;
  float mine = 0.f;
  {
    unsigned int rank = tie_rank;
    for (long long i = i0; i < i1; ++i) {
      const float w = weight(i);
      if (w <= 0.f) continue;
      const unsigned int bits = __float_as_uint(w);
      if (!filter || bits > thr) mine += w;
      else if (bits == thr && rank++ < take_ties) mine += w;
    }
  }
  float kept = 0.f;
  const float before = block_excl_scan<float>(mine, scan_f, &kept);
  const float target = fminf(fmaxf(uniforms[row], 0.f), 0.99999994f) * kept;
  // the owner of the target walks its chunk; the last thread with kept weight catches rounding at the upper end
  __shared__ long long s_pick;
  __shared__ float s_pick_w;
  if (threadIdx.x == 0) s_pick = -1;
  __syncthreads();
  if (mine > 0.f && target >= before && target < before + mine) {
    float acc = before;
    unsigned int rank = tie_rank;
    long long pick = -1;
    float pw = 0.f;
    for (long long i = i0; i < i1; ++i) {
      const float w = weight(i);
      if (w <= 0.f) continue;
      const unsigned int bits = __float_as_uint(w);
      const bool keep = !filter || bits > thr || (bits == thr && rank++ < take_ties);
      if (!keep) continue;
      pick = i;
      pw = w;
      acc += w;
      if (target < acc) break;
    }
    s_pick = pick;
    s_pick_w = pw;
  }
  __syncthreads();
  if (s_pick < 0) {
    // rounding left the target past every owner's range: take the last kept token
    __shared__ long long s_last[32];
    long long last = -1;
    unsigned int rank = tie_rank;
    for (long long i = i0; i < i1; ++i) {
      const float w = weight(i);
      if (w <= 0.f) continue;
      const unsigned int bits = __float_as_uint(w);
      if (!filter || bits > thr || (bits == thr && rank++ < take_ties)) last = i;
    }
    for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    if ((threadIdx.x & 31) == 0) s_last[threadIdx.x >> 5] = last;
    __syncthreads();
    if (threadIdx.x < 32) {
      last = s_last[threadIdx.x];
      for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
      if (threadIdx.x == 0) {
        s_pick = last < 0 ? 0 : last;
        s_pick_w = last < 0 ? 0.f : weight(last);
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    out_ids[row] = s_pick;
    if (out_prob) out_prob[row] = kept > 0.f ? s_pick_w / kept : 0.f;
  }
}

}  // namespace
}  // namespace swb

extern "C" {

// logits: [rows, V] fp32 (is_fp32) or bf16, row stride ld elements (read only: apply penalties before). temperature > 0.
// top_k <= 0: no count limit; top_p >= 1: no mass limit. uniforms: fp32 [rows] in [0, 1). allow_mask: uint8 [V] or null.
// out_ids: int64 [rows]; out_prob (optional): fp32 [rows], the drawn token's probability within the kept set.
int swb_sample_device(const void* logits, int is_fp32, long long ld, int rows, int V, float temperature, int top_k, float top_p,
                      const void* uniforms, const void* allow_mask, long long* out_ids, float* out_prob, void* stream) {
  using namespace swb;
  if (rows <= 0) return 0;
  if (!logits || !uniforms || !out_ids || V < 1 || ld < V || !(temperature > 0.f)) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float inv_t = 1.f / temperature;
  const uint8_t* allow = reinterpret_cast<const uint8_t*>(allow_mask);
  const float* u = reinterpret_cast<const float*>(uniforms);
  if (is_fp32)
    return launch_kernel(sample_device_kernel<float>, dim3(rows), dim3(SD_THREADS), 0, s, reinterpret_cast<const float*>(logits),
                         ld, V, inv_t, top_k, top_p, u, allow, out_ids, out_prob);
  return launch_kernel(sample_device_kernel<bf16>, dim3(rows), dim3(SD_THREADS), 0, s, reinterpret_cast<const bf16*>(logits), ld,
                       V, inv_t, top_k, top_p, u, allow, out_ids, out_prob);
}

}  // extern "C"
