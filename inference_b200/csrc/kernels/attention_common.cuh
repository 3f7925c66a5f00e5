// Shared definitions of the attention kernels (parameter block, mma.sync / ldmatrix / cp.async wrappers).
#pragma once
#include "common.cuh"

namespace swb {
namespace attn {

constexpr int HD = 128;
constexpr int KV_TILE = 64;
constexpr int TILE_BYTES = KV_TILE * HD * 2;  // 16 KB

struct AttnParams {
  const bf16* q;
  long long q_stride_tok;
  int q_stride_head;
  bf16* out;
  long long out_stride_tok;
  const bf16* k;
  const bf16* v;
  const int* block_table;  // non-null => paged
  int max_blocks;
  int block_size;
  long long kv_stride_tok;  // dense layout strides (elements)
  int kv_stride_head;
  const int* cu_q;     // [num_seqs + 1] or null (uniform_q_len)
  const int* cu_k;     // dense only: [num_seqs + 1] or null (uniform_kv_len)
  const int* kv_lens;  // [num_seqs] or null (uniform_kv_len)
  int uniform_q_len, uniform_kv_len;
  int num_seqs, Hq, Hkv, G;
  float scale;
  float softcap;
  int causal;
  int num_splits;
  float* part_o;
  float* part_ml;
  int cluster_merge;     // the splits of a (sequence, kv head) are one thread-block cluster (num_splits <= 8)
  int* split_counters;   // [num_seqs * Hkv] zero between launches: in-kernel merge by the last split to arrive (TMA kernel)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float score_transform(float s, float scale, float softcap) {
  // returns the score in log2 units
  if (softcap > 0.f) return softcap * tanhf(s * scale / softcap) * 1.4426950408889634f;
  return s * (scale * 1.4426950408889634f);
}

}  // namespace attn

// attention_tcgen05.cu
void attn_dense_tcgen05_set_tiles(int tiles);
int attn_dense_tcgen05_supported(const void* q, const void* k, const void* v, long long q_stride_tok, int q_stride_head,
                                 long long kv_stride_tok, int kv_stride_head, long long out_stride_tok, int D,
                                 int causal);
int attn_dense_tcgen05_launch(const void* q, long long q_stride_tok, int q_stride_head, const void* k, const void* v,
                              long long kv_stride_tok, int kv_stride_head, void* out, long long out_stride_tok,
                              int batch, int q_len, int kv_len, int Hq, int Hkv, float scale, cudaStream_t stream,
                              void* const* peers = nullptr, int world = 0, int split = 0, int n0 = 0, int n1 = 0,
                              int col_offset = 0, int causal = 0, const int* cu_q = nullptr, int total_tokens = 0,
                              int head_dim = 128, const int* kv_lens = nullptr, const int* block_table = nullptr,
                              int max_blocks = 0, int block_size = 0, int num_blocks = 0);
}  // namespace swb
