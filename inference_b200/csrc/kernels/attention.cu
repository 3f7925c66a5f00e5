// Attention for sm_100a over a paged or dense KV layout, head_dim 128.
//
//   attn_prefill_kernel : 64 query rows per CTA (4 warps x 16 rows), streaming 64-token KV tiles through
//                         a cp.async double buffer, online softmax, causal (bottom-right aligned) or full.
//                         Serves LLM prefill / chunked prefill over the block table and the DiT joint
//                         attention over dense [token, head, dim] tensors.
//   attn_decode_kernel  : one CTA per (sequence, kv head, KV split); the <=16 rows are the GQA group's
//                         query heads (times up to a few query tokens for speculative verify); the four
//                         warps take different 16-token slices of every KV tile and merge in shared
//                         memory; optional split-KV partials are merged by attn_merge_kernel.
// The KV cache layout is [block, kv_head, block_size, head_dim] so one head's tokens of a block are
// contiguous. Replaces the reference's gather(index_select) + repeat_kv + FlashAttention-2 varlen /
// eager SDPA path (candle-llm/src/primitives/attention.rs:59-68,136-302; paged_kv_cache.rs:248-283).
#include "attention_common.cuh"
#include "gemm_tcgen05.cuh"

namespace swb {

SWB_REGISTER_STATUS_UNIT(attention);
int g_dense_impl = 0;
using namespace attn;
namespace {

// byte offset of 16-byte chunk `c` of row `r` in a [rows][128 bf16] tile with an XOR swizzle
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ const bf16* kv_row_ptr(const AttnParams& p, const bf16* base, int seq, int kv_start,
                                                  int kvh, int tok) {
  if (p.block_table) {
    const int blk = __ldg(&p.block_table[(size_t)seq * p.max_blocks + tok / p.block_size]);
    return base + (((size_t)blk * p.Hkv + kvh) * p.block_size + (tok % p.block_size)) * (size_t)HD;
  }
  return base + (size_t)(kv_start + tok) * p.kv_stride_tok + (size_t)kvh * p.kv_stride_head;
}

// All 128 threads copy one 64-token tile of K and of V into shared memory (zero-filling past kv_len).
__device__ __forceinline__ void load_kv_tile(const AttnParams& p, int seq, int kv_start, int kvh, int tile,
                                             int kv_len, uint32_t sK, uint32_t sV) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 128;
    const int row = idx >> 4, c = idx & 15;
    const int tok = tile * KV_TILE + row;
    const bool valid = tok < kv_len;
    const bf16* kr = valid ? kv_row_ptr(p, p.k, seq, kv_start, kvh, tok) + c * 8 : p.k;
    const bf16* vr = valid ? kv_row_ptr(p, p.v, seq, kv_start, kvh, tok) + c * 8 : p.v;
    const uint32_t off = tile_off(row, c);
    cp_async16(sK + off, kr, valid ? 16u : 0u);
    cp_async16(sV + off, vr, valid ? 16u : 0u);
  }
}

// ------------------------------------------------------------------------------------------------
// prefill / dense attention
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait(TL_ATTN_PREFILL);
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sKV = sQ + TILE_BYTES;  // stage s: K at sKV + s*2*TILE, V at + TILE

  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int kvh = head / p.G;
  const int q_start = p.cu_q ? p.cu_q[seq] : seq * p.uniform_q_len;
  const int q_len = p.cu_q ? p.cu_q[seq + 1] - q_start : p.uniform_q_len;
  const int kv_len = p.kv_lens ? p.kv_lens[seq] : p.uniform_kv_len;
  const int kv_start = p.block_table ? 0 : (p.cu_k ? p.cu_k[seq] : seq * p.uniform_kv_len);
  const int n_qt = (q_len + 63) / 64;
  // heavy (late) causal tiles first
  const int qt = p.causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
  if (qt >= n_qt) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int q0 = qt * 64;
  const int causal_shift = kv_len - q_len;  // query i sees keys <= i + shift

  int kv_end = kv_len;
  if (p.causal) kv_end = min(kv_len, q0 + 64 + causal_shift);
  const int n_tiles = kv_end > 0 ? (kv_end + KV_TILE - 1) / KV_TILE : 0;

  // Q tile -> shared
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 128;
    const int row = idx >> 4, c = idx & 15;
    const bool valid = (q0 + row) < q_len;
    const bf16* src =
        valid ? p.q + (size_t)(q_start + q0 + row) * p.q_stride_tok + (size_t)head * p.q_stride_head + c * 8 : p.q;
    cp_async16(sQ + tile_off(row, c), src, valid ? 16u : 0u);
  }
  if (n_tiles > 0) load_kv_tile(p, seq, kv_start, kvh, 0, kv_len, sKV, sKV + TILE_BYTES);
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  uint32_t qf[8][4];

  for (int j = 0; j < n_tiles; ++j) {
    const uint32_t sK = sKV + (uint32_t)((j & 1) * 2 * TILE_BYTES);
    const uint32_t sV = sK + TILE_BYTES;
    if (j + 1 < n_tiles) {
      const uint32_t nK = sKV + (uint32_t)(((j + 1) & 1) * 2 * TILE_BYTES);
      load_kv_tile(p, seq, kv_start, kvh, j + 1, kv_len, nK, nK + TILE_BYTES);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (j == 0) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int mi = lane >> 3;
        const int row = warp * 16 + (mi & 1) * 8 + (lane & 7);
        ldsm_x4(sQ + tile_off(row, kk * 2 + (mi >> 1)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    // S = Q K^T
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        const int mi = lane >> 3;
        const int tok = np * 16 + (mi >> 1) * 8 + (lane & 7);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + tile_off(tok, kk * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_16816(s[2 * np], qf[kk], b0, b1);
        mma_16816(s[2 * np + 1], qf[kk], b2, b3);
      }
    }
    // scale + mask
    const int tile_base = j * KV_TILE;
    const bool need_mask = (tile_base + KV_TILE > kv_len) || (p.causal && (tile_base + KV_TILE - 1 > q0 + warp * 16 + causal_shift));
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float val = score_transform(s[nt][e], p.scale, p.softcap);
        if (need_mask) {
          const int col = tile_base + nt * 8 + t4 * 2 + (e & 1);
          const int qi = q0 + warp * 16 + g + ((e >> 1) ? 8 : 0);
          const bool ok = (col < kv_len) && (!p.causal || col <= qi + causal_shift);
          if (!ok) val = -INFINITY;
        }
        s[nt][e] = val;
      }
    }
    // online softmax
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * hr], s[nt][2 * hr + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hr], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run[hr] - m_safe);
      float rs = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float p0 = exp2f(s[nt][2 * hr] - m_safe);
        const float p1 = exp2f(s[nt][2 * hr + 1] - m_safe);
        s[nt][2 * hr] = p0;
        s[nt][2 * hr + 1] = p1;
        rs += p0 + p1;
      }
      l_run[hr] = l_run[hr] * alpha + rs;
      m_run[hr] = m_new;
#pragma unroll
      for (int dn = 0; dn < 16; ++dn) {
        o[dn][2 * hr] *= alpha;
        o[dn][2 * hr + 1] *= alpha;
      }
    }
    // O += P V
#pragma unroll
    for (int kk2 = 0; kk2 < 4; ++kk2) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk2][0], s[2 * kk2][1]);
      a[1] = pack_bf16(s[2 * kk2][2], s[2 * kk2][3]);
      a[2] = pack_bf16(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]);
      a[3] = pack_bf16(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int mi = lane >> 3;
        const int tok = kk2 * 16 + (mi & 1) * 8 + (lane & 7);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(sV + tile_off(tok, dp * 2 + (mi >> 1)), b0, b1, b2, b3);
        mma_16816(o[2 * dp], a, b0, b1);
        mma_16816(o[2 * dp + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  if (n_tiles == 0) cp_async_wait<0>();

  // finalize
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int qi = q0 + warp * 16 + g + hr * 8;
    if (qi < q_len) {
      bf16* dst = p.out + (size_t)(q_start + qi) * p.out_stride_tok + (size_t)head * HD;
#pragma unroll
      for (int dn = 0; dn < 16; ++dn) {
        const uint32_t pk = pack_bf16(o[dn][2 * hr] * inv, o[dn][2 * hr + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + dn * 8 + t4 * 2) = pk;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode attention (<= 16 packed rows = query tokens x GQA group heads)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait(TL_ATTN_DECODE);
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);           // 16 rows x 256 B = 4 KB
  const uint32_t sKV = sQ + 16 * 256;            // 2 stages x (K, V)
  float* sMerge = reinterpret_cast<float*>(smem + 16 * 256);  // reused after the loop

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int seq = blockIdx.z;
  const int q_start = p.cu_q ? p.cu_q[seq] : seq * p.uniform_q_len;
  const int q_len = p.cu_q ? p.cu_q[seq + 1] - q_start : p.uniform_q_len;
  const int kv_len = p.kv_lens ? p.kv_lens[seq] : p.uniform_kv_len;
  const int kv_start = p.block_table ? 0 : (p.cu_k ? p.cu_k[seq] : seq * p.uniform_kv_len);
  const int nrows = min(16, q_len * p.G);
  const int causal_shift = kv_len - q_len;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int total_tiles = (kv_len + KV_TILE - 1) / KV_TILE;
  const int per = (total_tiles + p.num_splits - 1) / p.num_splits;
  const int t0 = split * per;
  const int t1 = min(total_tiles, t0 + per);
  const int n_tiles = max(0, t1 - t0);

  // Q rows -> shared (row r = query token r / G, head kvh * G + r % G)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + i * 128;
    const int row = idx >> 4, c = idx & 15;
    const bool valid = row < nrows;
    const int qtok = row / p.G, hg = row % p.G;
    const bf16* src = valid ? p.q + (size_t)(q_start + qtok) * p.q_stride_tok +
                                  (size_t)(kvh * p.G + hg) * p.q_stride_head + c * 8
                            : p.q;
    cp_async16(sQ + tile_off(row, c), src, valid ? 16u : 0u);
  }
  if (n_tiles > 0) load_kv_tile(p, seq, kv_start, kvh, t0, kv_len, sKV, sKV + TILE_BYTES);
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  uint32_t qf[8][4];

  for (int j = 0; j < n_tiles; ++j) {
    const uint32_t sK = sKV + (uint32_t)((j & 1) * 2 * TILE_BYTES);
    const uint32_t sV = sK + TILE_BYTES;
    if (j + 1 < n_tiles) {
      const uint32_t nK = sKV + (uint32_t)(((j + 1) & 1) * 2 * TILE_BYTES);
      load_kv_tile(p, seq, kv_start, kvh, t0 + j + 1, kv_len, nK, nK + TILE_BYTES);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (j == 0) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int mi = lane >> 3;
        const int row = (mi & 1) * 8 + (lane & 7);
        ldsm_x4(sQ + tile_off(row, kk * 2 + (mi >> 1)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    // this warp's 16 tokens of the tile
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int mi = lane >> 3;
      const int tok = warp * 16 + (mi >> 1) * 8 + (lane & 7);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(sK + tile_off(tok, kk * 2 + (mi & 1)), b0, b1, b2, b3);
      mma_16816(s[0], qf[kk], b0, b1);
      mma_16816(s[1], qf[kk], b2, b3);
    }
    const int tok_base = (t0 + j) * KV_TILE + warp * 16;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float val = score_transform(s[nt][e], p.scale, p.softcap);
        const int col = tok_base + nt * 8 + t4 * 2 + (e & 1);
        const int row = g + ((e >> 1) ? 8 : 0);
        const int qtok = row / p.G;
        const bool ok = (col < kv_len) && (!p.causal || col <= qtok + causal_shift);
        s[nt][e] = ok ? val : -INFINITY;
      }
    }
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float mx = fmaxf(fmaxf(s[0][2 * hr], s[0][2 * hr + 1]), fmaxf(s[1][2 * hr], s[1][2 * hr + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hr], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run[hr] - m_safe);
      float rs = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = exp2f(s[nt][2 * hr] - m_safe);
        const float p1 = exp2f(s[nt][2 * hr + 1] - m_safe);
        s[nt][2 * hr] = p0;
        s[nt][2 * hr + 1] = p1;
        rs += p0 + p1;
      }
      l_run[hr] = l_run[hr] * alpha + rs;
      m_run[hr] = m_new;
#pragma unroll
      for (int dn = 0; dn < 16; ++dn) {
        o[dn][2 * hr] *= alpha;
        o[dn][2 * hr + 1] *= alpha;
      }
    }
    {
      uint32_t a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int mi = lane >> 3;
        const int tok = warp * 16 + (mi & 1) * 8 + (lane & 7);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(sV + tile_off(tok, dp * 2 + (mi >> 1)), b0, b1, b2, b3);
        mma_16816(o[2 * dp], a, b0, b1);
        mma_16816(o[2 * dp + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  if (n_tiles == 0) {
    cp_async_wait<0>();
    __syncthreads();
  }

  // cross-warp merge through shared memory: per warp [16][128] fp32 O, then [16] m and [16] l
  float* wO = sMerge + warp * (16 * HD);
  float* wM = sMerge + 4 * 16 * HD + warp * 16;
  float* wL = wM + 4 * 16;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = g + hr * 8;
    if (t4 == 0) {
      wM[row] = m_run[hr];
      wL[row] = l;
    }
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) {
      wO[row * HD + dn * 8 + t4 * 2] = o[dn][2 * hr];
      wO[row * HD + dn * 8 + t4 * 2 + 1] = o[dn][2 * hr + 1];
    }
  }
  __syncthreads();
  const int d = threadIdx.x;  // one output column per thread
  for (int row = 0; row < nrows; ++row) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sMerge[4 * 16 * HD + w * 16 + row]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = exp2f(sMerge[4 * 16 * HD + w * 16 + row] - Ms);
      L += sc * sMerge[4 * 16 * HD + 4 * 16 + w * 16 + row];
      acc += sc * sMerge[w * 16 * HD + row * HD + d];
    }
    const int qtok = row / p.G, hg = row % p.G;
    if (p.num_splits == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      p.out[(size_t)(q_start + qtok) * p.out_stride_tok + (size_t)(kvh * p.G + hg) * HD + d] =
          __float2bfloat16(acc * inv);
    } else {
      const size_t base = (((size_t)seq * p.Hkv + kvh) * p.num_splits + split) * 16 + row;
      p.part_o[base * HD + d] = acc;
      if (d == 0) {
        p.part_ml[base * 2] = M;
        p.part_ml[base * 2 + 1] = L;
      }
    }
  }
}

__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait(TL_ATTN_MERGE);
  const int kvh = blockIdx.x;
  const int seq = blockIdx.y;
  const int q_start = p.cu_q ? p.cu_q[seq] : seq * p.uniform_q_len;
  const int q_len = p.cu_q ? p.cu_q[seq + 1] - q_start : p.uniform_q_len;
  const int nrows = min(16, q_len * p.G);
  const int d = threadIdx.x;
  for (int row = 0; row < nrows; ++row) {
    const size_t base0 = (((size_t)seq * p.Hkv + kvh) * p.num_splits) * 16 + row;
    float M = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) M = fmaxf(M, p.part_ml[(base0 + (size_t)s * 16) * 2]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
      const size_t b = base0 + (size_t)s * 16;
      const float sc = exp2f(p.part_ml[b * 2] - Ms);
      L += sc * p.part_ml[b * 2 + 1];
      acc += sc * p.part_o[b * HD + d];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int qtok = row / p.G, hg = row % p.G;
    p.out[(size_t)(q_start + qtok) * p.out_stride_tok + (size_t)(kvh * p.G + hg) * HD + d] =
        __float2bfloat16(acc * inv);
  }
}

constexpr int PREFILL_SMEM = TILE_BYTES + 4 * TILE_BYTES;  // Q + 2 x (K, V) = 80 KB
constexpr int DECODE_SMEM = 16 * 256 + 4 * TILE_BYTES;     // 68 KB (merge area 4*16*128*4 + 512 B fits)

int configure_once() {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || done[dev]) return 0;
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM);
  if (e != cudaSuccess) return -(int)e;
  e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DECODE_SMEM);
  if (e != cudaSuccess) return -(int)e;
  done[dev] = true;
  return 0;
}

static thread_local int launch_rc = 0;
inline int last_err() { return launch_rc; }

}  // namespace

int attn_decode_tma_launch(const AttnParams& p, int num_blocks, cudaStream_t stream);

}  // namespace swb

extern "C" {

// Bytes of fp32 scratch the decode path needs for `num_splits` KV splits.
// Split-KV scratch: [ticket counters: num_seqs * Hkv ints, rounded up to 256 bytes][partial O][partial max / sum].
// The counters must be zero before the first launch (the kernel leaves them zero).
static size_t attn_counter_bytes(int num_seqs, int Hkv) { return (((size_t)num_seqs * Hkv * sizeof(int)) + 255) / 256 * 256; }
size_t swb_attn_decode_workspace_bytes(int num_seqs, int Hkv, int num_splits) {
  return attn_counter_bytes(num_seqs, Hkv) + (size_t)num_seqs * Hkv * num_splits * 16 * (swb::HD + 2) * sizeof(float);
}

// Paged-KV attention. q: [T, Hq, 128] with element strides; out: [T, Hq*128] rows of stride out_stride_tok.
// mode 0 = prefill (any q_len per sequence, max_q_len bounds the grid); mode 1 = decode (q_len * G <= 16).
int swb_attn_paged(const void* q, long long q_stride_tok, int q_stride_head, void* out, long long out_stride_tok,
                   const void* kcache, const void* vcache, const int* block_table, int max_blocks, int block_size,
                   int num_blocks, const int* cu_q, const int* kv_lens, int num_seqs, int max_q_len, int Hq, int Hkv, int D,
                   float scale, float softcap, int causal, int mode, int num_splits, void* workspace,
                   size_t workspace_bytes, void* stream) {
  using namespace swb;
  if (num_seqs <= 0) return 0;
  if (D != HD || Hq % Hkv != 0 || block_size <= 0) return -3;
  int rc = configure_once();
  if (rc) return rc;
  AttnParams p{};
  p.q = reinterpret_cast<const bf16*>(q);
  p.q_stride_tok = q_stride_tok;
  p.q_stride_head = q_stride_head;
  p.out = reinterpret_cast<bf16*>(out);
  p.out_stride_tok = out_stride_tok;
  p.k = reinterpret_cast<const bf16*>(kcache);
  p.v = reinterpret_cast<const bf16*>(vcache);
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.cu_q = cu_q;
  p.kv_lens = kv_lens;
  p.uniform_q_len = max_q_len;
  p.num_seqs = num_seqs;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.G = Hq / Hkv;
  p.scale = scale;
  p.softcap = softcap;
  p.causal = causal;
  p.num_splits = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (mode == 0) {
    dim3 grid((max_q_len + 63) / 64, Hq, num_seqs);
    launch_rc = launch_kernel(attn_prefill_kernel, dim3(grid), dim3(128), PREFILL_SMEM, s, p);
    return last_err();
  }
  if (max_q_len * p.G > 16) return -4;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1) {
    if (!workspace || workspace_bytes < swb_attn_decode_workspace_bytes(num_seqs, Hkv, num_splits)) return -5;
    if (num_splits > 32) num_splits = 32;
    p.part_o = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + attn_counter_bytes(num_seqs, Hkv));
    p.part_ml = p.part_o + (size_t)num_seqs * Hkv * num_splits * 16 * HD;
  }
  p.num_splits = num_splits;
  if (block_size == 16 && num_blocks > 0 && kv_lens != nullptr) {
    // TMA-fed warp-specialised kernel (the cp.async kernel below serves other block sizes); it merges its own splits
    if (num_splits > 1) p.split_counters = reinterpret_cast<int*>(workspace);
    return attn_decode_tma_launch(p, num_blocks, s);
  } else {
    dim3 grid(num_splits, Hkv, num_seqs);
    launch_rc = launch_kernel(attn_decode_kernel, dim3(grid), dim3(128), DECODE_SMEM, s, p);
    rc = last_err();
  }
  if (rc || num_splits == 1) return rc;
  launch_rc = launch_kernel(attn_merge_kernel, dim3(dim3(Hkv, num_seqs)), dim3(128), 0, s, p);
  return last_err();
}

// Dense non-causal attention (tcgen05 kernel only, batch 1) whose epilogue returns every output row to the rank
// that owns the token: see OutScatter in attention_tcgen05.cu. peers: `world` pointers to [local rows, out_stride_tok].
int swb_attn_dense_scatter(const void* q, long long q_stride_tok, int q_stride_head, const void* k, const void* v,
                           long long kv_stride_tok, int kv_stride_head, void* const* peers, int world,
                           long long out_stride_tok, int col_offset, int row_split, int n0, int n1, int q_len,
                           int kv_len, int Hq, int Hkv, float scale, void* stream) {
  using namespace swb;
  if (q_len <= 0 || kv_len <= 0 || Hq % Hkv != 0) return -3;
  if (!attn_dense_tcgen05_supported(q, k, v, q_stride_tok, q_stride_head, kv_stride_tok, kv_stride_head, out_stride_tok,
                                    128, 0))
    return -3;
  return attn_dense_tcgen05_launch(q, q_stride_tok, q_stride_head, k, v, kv_stride_tok, kv_stride_head, nullptr,
                                   out_stride_tok, 1, q_len, kv_len, Hq, Hkv, scale,
                                   reinterpret_cast<cudaStream_t>(stream), peers, world, row_split, n0, n1, col_offset);
}

// Causal self-attention over a packed batch of fresh sequences (no earlier context): sequence s covers tokens
// [cu_q[s], cu_q[s + 1]) of q / k / v / out, which share one flat token axis (prefill straight from the QKV
// projection output). cu_q: device int32 [num_seqs + 1]. tcgen05 kernel only (head dim 128).
int swb_attn_varlen_causal(const void* q, long long q_stride_tok, int q_stride_head, const void* k, const void* v,
                           long long kv_stride_tok, int kv_stride_head, void* out, long long out_stride_tok,
                           const int* cu_q, int num_seqs, int max_q_len, int total_tokens, int Hq, int Hkv, float scale,
                           void* stream) {
  using namespace swb;
  if (num_seqs <= 0 || total_tokens <= 0) return 0;
  if (!cu_q || max_q_len <= 0 || Hq % Hkv != 0) return -3;
  if (!attn_dense_tcgen05_supported(q, k, v, q_stride_tok, q_stride_head, kv_stride_tok, kv_stride_head, out_stride_tok,
                                    128, 1))
    return -3;
  return attn_dense_tcgen05_launch(q, q_stride_tok, q_stride_head, k, v, kv_stride_tok, kv_stride_head, out,
                                   out_stride_tok, num_seqs, max_q_len, max_q_len, Hq, Hkv, scale,
                                   reinterpret_cast<cudaStream_t>(stream), nullptr, 0, 0, 0, 0, 0, 1, cu_q, total_tokens);
}

// Prefill over paged keys / values on the tcgen05 kernel: sequence s has query tokens [cu_q[s], cu_q[s + 1]) of the flat
// q / out token axis (total_tokens rows) and kv_lens[s] keys (earlier context + these tokens, already in the cache) in
// pages block_table[s, :]; its queries sit at the last positions (bottom-right aligned causal mask). Caches:
// [num_blocks, Hkv, block_size, 128] contiguous, block_size a multiple of 8 dividing 128. Returns -3 when the problem
// is outside the kernel's reach (the caller then takes swb_attn_paged).
int swb_attn_paged_prefill_tc(const void* q, long long q_stride_tok, int q_stride_head, void* out, long long out_stride_tok,
                              const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                              int block_size, int num_blocks, const int* cu_q, const int* kv_lens, int num_seqs,
                              int max_q_len, int total_tokens, int Hq, int Hkv, float scale, int causal, void* stream) {
  using namespace swb;
  if (num_seqs <= 0 || total_tokens <= 0) return 0;
  if (g_dense_impl != 0 || !cu_q || !kv_lens || !block_table || max_q_len <= 0 || Hq % Hkv != 0) return -3;
  if (!attn_dense_tcgen05_supported(q, kcache, vcache, q_stride_tok, q_stride_head, 128, 128, out_stride_tok, 128, causal))
    return -3;
  return attn_dense_tcgen05_launch(q, q_stride_tok, q_stride_head, kcache, vcache, 128, 128, out, out_stride_tok,
                                   num_seqs, max_q_len, max_q_len, Hq, Hkv, scale, reinterpret_cast<cudaStream_t>(stream),
                                   nullptr, 0, 0, 0, 0, 0, causal, cu_q, total_tokens, 128, kv_lens, block_table,
                                   max_blocks, block_size, num_blocks);
}

// 0: pick the tcgen05 kernel whenever it supports the problem; 1: always the mma.sync kernel (comparison runs).
void swb_attn_dense_set_impl(int impl) { swb::g_dense_impl = impl; }
// 0: pick the number of query tiles per CTA per problem; 1 / 2: fixed (comparison runs).
void swb_attn_dense_set_tiles(int tiles) { swb::attn_dense_tcgen05_set_tiles(tiles); }

// Dense attention over q/k/v laid out [batch * seq, heads, 128] (arbitrary element strides), uniform lengths.
int swb_attn_dense(const void* q, long long q_stride_tok, int q_stride_head, const void* k, const void* v,
                   long long kv_stride_tok, int kv_stride_head, void* out, long long out_stride_tok, int batch,
                   int q_len, int kv_len, int Hq, int Hkv, int D, float scale, int causal, void* stream) {
  using namespace swb;
  if (batch <= 0 || q_len <= 0) return 0;
  if ((D != HD && D != 64) || Hq % Hkv != 0) return -3;
  if (kv_len <= 0) return -3;
  if ((g_dense_impl == 0 || D == 64) && (!causal || q_len == kv_len) &&
      attn_dense_tcgen05_supported(q, k, v, q_stride_tok, q_stride_head, kv_stride_tok, kv_stride_head, out_stride_tok, D,
                                   causal))
    return attn_dense_tcgen05_launch(q, q_stride_tok, q_stride_head, k, v, kv_stride_tok, kv_stride_head, out,
                                     out_stride_tok, batch, q_len, kv_len, Hq, Hkv, scale,
                                     reinterpret_cast<cudaStream_t>(stream), nullptr, 0, 0, 0, 0, 0, causal, nullptr, 0, D);
  if (D != HD) return -3;            // 64-wide heads exist on the tcgen05 kernel only
  int rc = configure_once();
  if (rc) return rc;
  AttnParams p{};
  p.q = reinterpret_cast<const bf16*>(q);
  p.q_stride_tok = q_stride_tok;
  p.q_stride_head = q_stride_head;
  p.out = reinterpret_cast<bf16*>(out);
  p.out_stride_tok = out_stride_tok;
  p.k = reinterpret_cast<const bf16*>(k);
  p.v = reinterpret_cast<const bf16*>(v);
  p.block_table = nullptr;
  p.block_size = 1;
  p.kv_stride_tok = kv_stride_tok;
  p.kv_stride_head = kv_stride_head;
  p.uniform_q_len = q_len;
  p.uniform_kv_len = kv_len;
  p.num_seqs = batch;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.G = Hq / Hkv;
  p.scale = scale;
  p.softcap = 0.f;
  p.causal = causal;
  p.num_splits = 1;
  dim3 grid((q_len + 63) / 64, Hq, batch);
  launch_rc = launch_kernel(attn_prefill_kernel, dim3(grid), dim3(128), PREFILL_SMEM, reinterpret_cast<cudaStream_t>(stream), p);
  return last_err();
}

}  // extern "C"
