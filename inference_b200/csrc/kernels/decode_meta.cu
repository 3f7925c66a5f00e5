// Decode-step bookkeeping on the device: one kernel unpacks a step's packed int32 metadata into the typed input
// tensors of the forward, one kernel files the sampled tokens. Both index a device-side step counter, so a
// multi-step greedy run is nothing but replays of one captured graph: no host copy between steps.
// (The reference rebuilds its step tensors on the host every token: candle-llm/src/decode/batch.rs:133-214.)
#include "common.cuh"

namespace swb {

SWB_REGISTER_STATUS_UNIT(decode_meta);
namespace {

// meta rows: [ids MB][positions MB][slots MB][kv lens MB][block table MB * mb], int32.
__global__ void __launch_bounds__(256) decode_meta_unpack_kernel(const int* __restrict__ meta_all, long long n_meta,
                                                                 const int* __restrict__ step_ptr, int MB, int B,
                                                                 int mb, long long* ids, int* pos, long long* slots,
                                                                 int* kvl, int* table) {
  pdl_launch_dependents();
  pdl_wait(TL_META);
  const int step = step_ptr ? *step_ptr : 0;
  const int* m = meta_all + (size_t)step * n_meta;
  const int n_table = B * mb;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_table + B; i += gridDim.x * blockDim.x) {
    if (i < n_table) {
      table[i] = m[4 * MB + i];
    } else {
      const int r = i - n_table;
      if (ids) ids[r] = m[r];
      pos[r] = m[MB + r];
      slots[r] = m[2 * MB + r];
      kvl[r] = m[3 * MB + r];
    }
  }
}

// ids[r] = tokens[r] (feedback for the next replay), out_all[step, r] = tokens[r], then the step counter advances.
__global__ void __launch_bounds__(128) decode_step_tail_kernel(const long long* __restrict__ tokens, long long* ids,
                                                               long long* out_all, int* step_ptr, int B) {
  pdl_launch_dependents();
  pdl_wait(TL_TAIL);
  const int step = *step_ptr;
  for (int r = threadIdx.x; r < B; r += blockDim.x) {
    const long long t = tokens[r];
    if (ids) ids[r] = t;
    if (out_all) out_all[(size_t)step * B + r] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) *step_ptr = step + 1;
}

}  // namespace
}  // namespace swb

extern "C" {

int swb_decode_meta_unpack(const void* meta_all, long long n_meta, const void* step_ptr, int MB, int B, int mb,
                           void* ids, void* pos, void* slots, void* kvl, void* table, void* stream) {
  using namespace swb;
  if (B <= 0 || B > MB || mb <= 0) return -3;
  const int n = B * mb + B;
  const int grid = (n + 255) / 256 < 32 ? (n + 255) / 256 : 32;
  return launch_kernel(decode_meta_unpack_kernel, dim3(grid), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const int*>(meta_all), n_meta, reinterpret_cast<const int*>(step_ptr), MB, B,
                       mb, reinterpret_cast<long long*>(ids), reinterpret_cast<int*>(pos),
                       reinterpret_cast<long long*>(slots), reinterpret_cast<int*>(kvl), reinterpret_cast<int*>(table));
}

int swb_decode_step_tail(const void* tokens, void* ids, void* out_all, void* step_ptr, int B, void* stream) {
  using namespace swb;
  if (B <= 0 || !step_ptr) return -3;
  return launch_kernel(decode_step_tail_kernel, dim3(1), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const long long*>(tokens), reinterpret_cast<long long*>(ids),
                       reinterpret_cast<long long*>(out_all), reinterpret_cast<int*>(step_ptr), B);
}

}  // extern "C"
