// Device-side token selection: greedy argmax over the vocabulary (ties resolve to the lowest index,
// like the reference's host argmax in candle-llm/src/primitives/sampler.rs:213-235), optional
// allow-mask for constrained decoding, repetition penalty, and the speculative-decoding greedy verify
// (longest matching prefix of draft tokens against target argmaxes, candle-llm/src/decode/speculative.rs:399-421).
#include "common.cuh"

#include <algorithm>

namespace swb {

SWB_REGISTER_STATUS_UNIT(sampling);
namespace {

struct ArgMax {
  float v;
  long long i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

template <typename T>
__device__ __forceinline__ float to_f(T x);
template <>
__device__ __forceinline__ float to_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f<bf16>(bf16 x) { return __bfloat162float(x); }

// allow: optional uint8 [V] (1 = allowed). penalty_ids: optional [n_pen] token ids whose logit is divided
// (positive) or multiplied (negative) by `penalty` before the comparison.
// grid (rows, chunks): each CTA reduces one contiguous vocabulary chunk of one row. With chunks == 1 the
// result goes straight to out_ids; otherwise (value, index) partials go to `part` and argmax_merge_kernel
// finishes the row, so a 128k vocabulary at batch 1..64 still fills the GPU.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, long long ld, int V,
                                                      const uint8_t* __restrict__ allow, long long* out_ids,
                                                      float* out_vals, float* part_val, long long* part_idx) {
  pdl_launch_dependents();
  pdl_wait(TL_ARGMAX);
  __shared__ ArgMax red[32];
  const int row = blockIdx.x;
  const int chunks = gridDim.y;
  const int per = (V + chunks - 1) / chunks;
  const int v0 = blockIdx.y * per;
  const int v1 = min(V, v0 + per);
  const T* x = logits + (size_t)row * ld;
  ArgMax best{-INFINITY, (long long)V};
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    if (allow && !allow[i]) continue;
    float v = to_f<T>(x[i]);
    if (v != v) continue;  // NaN never wins
    best = better(best, ArgMax{v, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? red[lane] : ArgMax{-INFINITY, (long long)V};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (lane == 0) {
      if (chunks == 1) {
        out_ids[row] = best.i < V ? best.i : 0;
        if (out_vals) out_vals[row] = best.v;
      } else {
        part_val[row * chunks + blockIdx.y] = best.v;
        part_idx[row * chunks + blockIdx.y] = best.i;
      }
    }
  }
}

__global__ void __launch_bounds__(32) argmax_merge_kernel(const float* __restrict__ part_val,
                                                         const long long* __restrict__ part_idx, int chunks, int V,
                                                         long long* out_ids, float* out_vals) {
  pdl_launch_dependents();
  pdl_wait(TL_ARGMAX_MERGE);
  const int row = blockIdx.x;
  ArgMax best{-INFINITY, (long long)V};
  for (int c = threadIdx.x; c < chunks; c += 32)
    best = better(best, ArgMax{part_val[row * chunks + c], part_idx[row * chunks + c]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) {
    out_ids[row] = best.i < V ? best.i : 0;
    if (out_vals) out_vals[row] = best.v;
  }
}

// Greedy speculative verify for one sequence: target_ids[0..k] are the target argmaxes at the k+1
// verified positions, draft[0..k-1] the proposed tokens. Writes n_accepted (longest prefix with
// target_ids[i] == draft[i]) and the bonus/correction token target_ids[n_accepted].
__global__ void spec_verify_greedy_kernel(const long long* __restrict__ target_ids, const long long* __restrict__ draft,
                                          int k, int num_seqs, int* n_accepted, long long* next_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= num_seqs) return;
  const long long* t = target_ids + (size_t)s * (k + 1);
  const long long* d = draft + (size_t)s * k;
  int n = 0;
  while (n < k && t[n] == d[n]) ++n;
  n_accepted[s] = n;
  next_token[s] = t[n];
}

// In-place repetition penalty on fp32 logits: for each id in history[row, :len[row]] once.
__global__ void rep_penalty_kernel(float* logits, long long ld, int V, const long long* __restrict__ history,
                                   int hist_ld, const int* __restrict__ hist_len, float penalty) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int n = hist_len[row];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long long id = history[(size_t)row * hist_ld + i];
    if (id < 0 || id >= V) continue;
    bool first = true;  // apply once per distinct id: only the first occurrence applies it
    for (int j = 0; j < i; ++j)
      if (history[(size_t)row * hist_ld + j] == id) {
        first = false;
        break;
      }
    if (!first) continue;
    float& x = logits[(size_t)row * ld + id];
    x = x > 0.f ? x / penalty : x * penalty;
  }
}

static thread_local int launch_rc = 0;
inline int last_err() { return launch_rc; }

}  // namespace
}  // namespace swb

extern "C" {

// scratch: >= rows * 32 * 12 bytes when rows * V is large enough to be chunked (may be null: single pass).
int swb_argmax(const void* logits, int is_fp32, long long ld, int rows, int V, const void* allow_mask,
               long long* out_ids, float* out_vals, void* scratch, size_t scratch_bytes, void* stream) {
  using namespace swb;
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int chunks = 1;
  if (scratch && V >= 16384) {
    chunks = std::min(32, std::max(1, 296 / rows));
    while (chunks > 1 && (size_t)rows * chunks * 12 > scratch_bytes) chunks /= 2;
  }
  float* pv = reinterpret_cast<float*>(scratch);
  long long* pi = reinterpret_cast<long long*>(reinterpret_cast<uint8_t*>(scratch) + (size_t)rows * chunks * 4 +
                                               ((8 - ((size_t)rows * chunks * 4) % 8) % 8));
  const uint8_t* allow = reinterpret_cast<const uint8_t*>(allow_mask);
  if (is_fp32)
    launch_rc = launch_kernel(argmax_kernel<float>, dim3(rows, chunks), dim3(1024), 0, s,
                              reinterpret_cast<const float*>(logits), ld, V, allow, out_ids, out_vals, pv, pi);
  else
    launch_rc = launch_kernel(argmax_kernel<bf16>, dim3(rows, chunks), dim3(1024), 0, s,
                              reinterpret_cast<const bf16*>(logits), ld, V, allow, out_ids, out_vals, pv, pi);
  if (launch_rc || chunks == 1) return launch_rc;
  launch_rc = launch_kernel(argmax_merge_kernel, dim3(rows), dim3(32), 0, s, pv, pi, chunks, V, out_ids, out_vals);
  return launch_rc;
}

int swb_spec_verify_greedy(const long long* target_ids, const long long* draft, int k, int num_seqs, int* n_accepted,
                           long long* next_token, void* stream) {
  using namespace swb;
  if (num_seqs <= 0) return 0;
  launch_rc = launch_kernel(spec_verify_greedy_kernel, dim3((num_seqs + 127) / 128), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), target_ids, draft, k, num_seqs, n_accepted, next_token);
  return last_err();
}

int swb_rep_penalty(float* logits, long long ld, int rows, int V, const long long* history, int hist_ld,
                    const int* hist_len, float penalty, void* stream) {
  using namespace swb;
  if (rows <= 0) return 0;
  launch_rc = launch_kernel(rep_penalty_kernel, dim3(rows), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), logits, ld, V, history, hist_ld,
                                                                               hist_len, penalty);
  return last_err();
}

}  // extern "C"
