// swb_argmax_static: single-launch chunked argmax whose scratch is a file-scope device array (see argmax_static.h
// for the contract). Chunk results go to the array; the last block to arrive for a row (per-row counter) merges
// them and puts the counter back to zero.
#include "argmax_static.h"

#include "common.cuh"

#include <cstdio>
#include <mutex>

namespace swb {
namespace {

constexpr int MAX_ROWS = SWB_ARGMAX_STATIC_MAX_ROWS;
constexpr int MAX_CHUNKS = SWB_ARGMAX_STATIC_MAX_CHUNKS;
constexpr size_t OFF_VALS = (size_t)MAX_ROWS * 4;
constexpr size_t OFF_IDX = OFF_VALS + (size_t)MAX_ROWS * MAX_CHUNKS * 4;
static_assert(OFF_IDX % 8 == 0, "int64 slots must be 8-byte aligned");
static_assert(OFF_IDX + (size_t)MAX_ROWS * MAX_CHUNKS * 8 == SWB_ARGMAX_STATIC_SCRATCH_BYTES, "layout / header mismatch");

// Zero when the module is loaded; only the kernel below touches it.
static __device__ __align__(256) unsigned char g_argmax_scratch[SWB_ARGMAX_STATIC_SCRATCH_BYTES];

struct Best {
  float v;
  long long i;
};
__device__ __forceinline__ Best pick(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ Best warp_pick(Best b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    b = pick(b, Best{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)});
  return b;
}
template <typename T>
__device__ __forceinline__ float as_float(T x);
template <>
__device__ __forceinline__ float as_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ float as_float<bf16>(bf16 x) { return __bfloat162float(x); }

// grid (rows, chunks), 1024 threads. scratch: the array above, passed as a pointer.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_static_kernel(const T* __restrict__ logits, long long ld, int V,
                                                             const uint8_t* __restrict__ allow, long long* out_ids,
                                                             float* out_vals, unsigned char* scratch) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ Best red[32];
  __shared__ int s_last;
  int* counters = reinterpret_cast<int*>(scratch);
  float* part_val = reinterpret_cast<float*>(scratch + OFF_VALS);
  long long* part_idx = reinterpret_cast<long long*>(scratch + OFF_IDX);
  const int row = blockIdx.x, chunks = gridDim.y;
  // 64-bit index arithmetic: V may be anywhere up to INT_MAX
  const long long per = ((long long)V + chunks - 1) / chunks;
  const long long v0 = min((long long)V, (long long)blockIdx.y * per), v1 = min((long long)V, v0 + per);
  const T* x = logits + (size_t)row * ld;
  Best best{-INFINITY, (long long)V};
  for (long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    if (allow && !allow[i]) continue;
    const float v = as_float<T>(x[i]);
    if (v != v) continue;
    best = pick(best, Best{v, i});
  }
  best = warp_pick(best);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (warp != 0) return;
  best = warp_pick(red[lane]);
  if (chunks == 1) {
    if (lane == 0) {
      out_ids[row] = best.i < V ? best.i : 0;
      if (out_vals) out_vals[row] = best.v;
    }
    return;
  }
  if (lane == 0) {
    const int slot = row * MAX_CHUNKS + blockIdx.y;
    __stcg(&part_val[slot], best.v);
    __stcg(&part_idx[slot], best.i);
    __threadfence();
    s_last = (atomicAdd(&counters[row], 1) == chunks - 1);
  }
  __syncwarp();
  if (!s_last) return;
  __threadfence();
  Best m{-INFINITY, (long long)V};
  if (lane < chunks) m = Best{__ldcg(&part_val[row * MAX_CHUNKS + lane]), __ldcg(&part_idx[row * MAX_CHUNKS + lane])};
  m = warp_pick(m);
  if (lane == 0) {
    out_ids[row] = m.i < V ? m.i : 0;
    if (out_vals) out_vals[row] = m.v;
    counters[row] = 0;  // ready for the next call
  }
}

// One address per device, looked up on the first call made with that device current.
unsigned char* scratch_for_current_device(int* rc) {
  static std::mutex mu;
  static unsigned char* addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = SWB_ARGMAX_STATIC_E_SETUP;
    return nullptr;
  }
  std::lock_guard<std::mutex> g(mu);
  if (!addr[dev]) {
    unsigned char* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_argmax_scratch);
    if (e != cudaSuccess || !p) {
      std::fprintf(stderr, "swb_argmax_static: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                   cudaGetErrorString(e));
      *rc = SWB_ARGMAX_STATIC_E_SETUP;
      return nullptr;
    }
    addr[dev] = p;
  }
  return addr[dev];
}

}  // namespace
}  // namespace swb

extern "C" int swb_argmax_static(const void* logits, int is_fp32, long long ld, int rows, int V,
                                 const void* allow_mask, long long* out_ids, float* out_vals, void* stream) {
  using namespace swb;
  if (rows == 0) return 0;
  if (rows < 0 || rows > MAX_ROWS || V < 1) {
    std::fprintf(stderr, "swb_argmax_static: rows=%d V=%d outside the supported range (1..%d rows, V >= 1)\n", rows, V,
                 MAX_ROWS);
    return SWB_ARGMAX_STATIC_E_SIZE;
  }
  if (!logits || !out_ids || ld < V) return SWB_ARGMAX_STATIC_E_ARG;
  int rc = 0;
  unsigned char* scratch = scratch_for_current_device(&rc);
  if (!scratch) return rc;
  // enough blocks to cover the GPU about twice at small batch; one block per row once rows alone do that
  int chunks = 1;
  if (V >= 16384) {
    chunks = 296 / rows;
    if (chunks > MAX_CHUNKS) chunks = MAX_CHUNKS;
    if (chunks < 1) chunks = 1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* allow = reinterpret_cast<const uint8_t*>(allow_mask);
  if (is_fp32)
    return launch_kernel(argmax_static_kernel<float>, dim3(rows, chunks), dim3(1024), 0, s,
                         reinterpret_cast<const float*>(logits), ld, V, allow, out_ids, out_vals, scratch);
  return launch_kernel(argmax_static_kernel<bf16>, dim3(rows, chunks), dim3(1024), 0, s,
                       reinterpret_cast<const bf16*>(logits), ld, V, allow, out_ids, out_vals, scratch);
}
