// Decode attention over the paged KV cache with TMA-fed, warp-specialised CTAs (block_size 16, head_dim 128).
//
// One CTA per (KV split, kv head, sequence). Warp 4 is the producer: for every 64-token tile it looks up
// the four 16-token blocks in the block table and issues one tiled TMA copy per (block, K|V, 64-column
// half) with the 128-byte swizzle into a 3-stage ring, completing on an mbarrier. Warps 0..3 each take a
// 16-token slice of every tile: S = Q K^T and O += P V on mma.sync with ldmatrix from the swizzled ring,
// online softmax in registers, then a cross-warp merge in shared memory. The <=16 MMA rows are the GQA
// group's query heads times the (1..4) query tokens of the step. With num_splits > 1 the CTA writes an
// un-normalised partial (O, max, sum); the last split CTA of a (sequence, kv head) to finish merges them (ticket
// counter in the workspace, reset by the merger), so split-KV decode is still one launch.
// The decode step is bandwidth bound (KV bytes >> FLOPs), so the design goal is bytes in flight:
// 2 CTAs/SM x 3 stages x 32 KB with no per-thread address arithmetic on the load path.
#include "attention_common.cuh"
#include "gemm_tcgen05.cuh"

namespace swb {
using namespace attn;

SWB_REGISTER_STATUS_UNIT(attn_decode_tma);

namespace {

#ifndef SWB_DEC_STAGES
#define SWB_DEC_STAGES 3
#endif
#ifndef SWB_DEC_MIN_CTAS
#define SWB_DEC_MIN_CTAS 1
#endif
constexpr int STAGES = SWB_DEC_STAGES;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;  // K tile + V tile = 32 KB
constexpr int Q_BYTES = 16 * 256;            // 4 KB
constexpr int SMEM_BYTES = 1024 + Q_BYTES + STAGES * STAGE_BYTES + 256;

// Offset of 16-byte chunk c (0..15) of token row `tok` (0..63) inside a tile written by TMA as
// 8 boxes of [16 rows][64 bf16] with SWIZZLE_128B: box = (tok / 16) * 2 + (c / 8), 2 KB each.
__device__ __forceinline__ uint32_t tma_tile_off(int tok, int c) {
  const int r = tok & 15;
  return (uint32_t)((((tok >> 4) * 2 + (c >> 3)) << 11) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}
// Q rows are written by ordinary stores with the simple XOR swizzle of the other kernels.
__device__ __forceinline__ uint32_t q_off(int r, int c) { return (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4)); }

__global__ void __launch_bounds__(160, SWB_DEC_MIN_CTAS) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                              const __grid_constant__ CUtensorMap tmap_v,
                                                              const AttnParams p) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  uint8_t* ring = smem;                                  // STAGES x 32 KB, 1024-aligned
  uint8_t* sQp = smem + STAGES * STAGE_BYTES;            // 4 KB
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(sQp + Q_BYTES);
  uint64_t* bar_empty = bar_full + STAGES;
  volatile int* s_abort = reinterpret_cast<volatile int*>(bar_empty + STAGES);
  float* sMerge = reinterpret_cast<float*>(ring);        // reused after the loop (33 KB)

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  pdl_wait(TL_ATTN_DECODE);  // everything below reads what the preceding kernels wrote (q, the newest K/V, kv_lens)

  const int q_start = p.cu_q ? p.cu_q[seq] : seq * p.uniform_q_len;
  const int q_len = p.cu_q ? p.cu_q[seq + 1] - q_start : p.uniform_q_len;
  const int kv_len = p.kv_lens[seq];
  const int nrows = min(16, q_len * p.G);
  const int causal_shift = kv_len - q_len;
  const int total_tiles = (kv_len + KV_TILE - 1) / KV_TILE;
  const int per = (total_tiles + p.num_splits - 1) / p.num_splits;
  const int t0 = split * per;
  const int n_tiles = max(0, min(total_tiles, t0 + per) - t0);

  // Q rows -> shared (row r = query token r / G, head kvh * G + r % G), zero rows past nrows
  for (int idx = threadIdx.x; idx < 256; idx += blockDim.x) {
    const int row = idx >> 4, c = idx & 15;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row < nrows) {
      const int qtok = row / p.G, hg = row % p.G;
      val = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_start + qtok) * p.q_stride_tok +
                                            (size_t)(kvh * p.G + hg) * p.q_stride_head + c * 8);
    }
    *reinterpret_cast<uint4*>(sQp + q_off(row, c)) = val;
  }
  __syncthreads();

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const int* table = p.block_table + (size_t)seq * p.max_blocks;
      const int first_block = __ldg(&table[0]);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t outstanding = 0, issue_phase = 0;
      for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait(&bar_empty[stage], phase ^ 1, s_abort, 500 + stage)) break;
        outstanding &= ~(1u << stage);
        uint8_t* sK = ring + stage * STAGE_BYTES;
        uint8_t* sV = sK + TILE_BYTES;
        mbar_arrive_expect_tx(&bar_full[stage], STAGE_BYTES);
        const int tok0 = (t0 + j) * KV_TILE;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int tstart = tok0 + b * 16;
          // blocks wholly past the context reuse the first block: finite data, masked in the softmax
          const int blk = tstart < kv_len ? __ldg(&table[tstart >> 4]) : first_block;
          const int row0 = (blk * p.Hkv + kvh) * 16;
          tma_load_2d(sK + (b * 2 + 0) * 2048, &tmap_k, &bar_full[stage], 0, row0);
          tma_load_2d(sK + (b * 2 + 1) * 2048, &tmap_k, &bar_full[stage], 64, row0);
          tma_load_2d(sV + (b * 2 + 0) * 2048, &tmap_v, &bar_full[stage], 0, row0);
          tma_load_2d(sV + (b * 2 + 1) * 2048, &tmap_v, &bar_full[stage], 64, row0);
        }
        outstanding |= 1u << stage;
        issue_phase = (issue_phase & ~(1u << stage)) | (phase << stage);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (*s_abort) {
        for (int s = 0; s < STAGES; ++s)
          if (outstanding & (1u << s))
            for (int it = 0; it < (1 << 20); ++it)
              if (mbar_try_wait(&bar_full[s], (issue_phase >> s) & 1u)) break;
      }
    }
  } else {
    // ------------------------------ consumers (4 warps, 16 tokens of each tile per warp) --------------
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t sQ = smem_u32(sQp);
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int mi = lane >> 3;
      const int row = (mi & 1) * 8 + (lane & 7);
      ldsm_x4(sQ + q_off(row, kk * 2 + (mi >> 1)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    int stage = 0;
    uint32_t phase = 0;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(&bar_full[stage], phase, s_abort, 600 + stage)) break;
      const uint32_t sK = smem_u32(ring + stage * STAGE_BYTES);
      const uint32_t sV = sK + TILE_BYTES;
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int mi = lane >> 3;
        const int tok = warp * 16 + (mi >> 1) * 8 + (lane & 7);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + tma_tile_off(tok, kk * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_16816(s[0], qf[kk], b0, b1);
        mma_16816(s[1], qf[kk], b2, b3);
      }
      const int tok_base = (t0 + j) * KV_TILE + warp * 16;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float val = score_transform(s[nt][e], p.scale, p.softcap);
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
          ldsm_x4_trans(sV + tma_tile_off(tok, dp * 2 + (mi >> 1)), b0, b1, b2, b3);
          mma_16816(o[2 * dp], a, b0, b1);
          mma_16816(o[2 * dp + 1], a, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_empty[stage]);
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
  }
  __syncthreads();  // every issued tile has been consumed (or the CTA aborted and drained): the ring is free

  if (warp < 4) {
    const int g = lane >> 2, t4 = lane & 3;
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
        *reinterpret_cast<float2*>(&wO[row * HD + dn * 8 + t4 * 2]) = make_float2(o[dn][2 * hr], o[dn][2 * hr + 1]);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int d = threadIdx.x;
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
  if (p.num_splits > 1 && p.split_counters) {
    // Merge of the splits inside this launch. Cluster launch (the splits of a (sequence, kv head) form one
    // thread-block cluster): a cluster barrier orders the partials, the first CTA merges. Otherwise the last split
    // to arrive (ticket counter in the workspace, reset by the merger) merges.
    int* ctr = p.split_counters + (size_t)seq * p.Hkv + kvh;
    if (p.cluster_merge) {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (split != 0) return;
    } else {
      __shared__ int s_last;
      __threadfence();                       // this CTA's partials are visible device-wide before its ticket
      __syncthreads();
      if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == p.num_splits - 1) ? 1 : 0;
      __syncthreads();
      if (!s_last) return;
      __threadfence();
    }
    const int S = p.num_splits;            // <= 32
    float* sSc = sMerge;                   // [16][32] weights of the splits, then normalised
    float* sL = sMerge + 16 * 32;          // [16][32]
    const size_t base0 = ((size_t)seq * p.Hkv + kvh) * S * 16;
    __syncthreads();                       // (cluster path: the cross-warp merge area is free)
    for (int i = threadIdx.x; i < nrows * S; i += blockDim.x) {
      const int row = i / S, sp = i % S;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (base0 + (size_t)sp * 16 + row) * 2));
      sSc[row * 32 + sp] = ml.x;
      sL[row * 32 + sp] = ml.y;
    }
    // the partial outputs do not depend on the weights: request them now (up to 4 rows x 8 splits stay in registers)
    float po[4][8];
    const bool small = nrows <= 4 && S <= 8 && threadIdx.x < 128;
    if (small) {
#pragma unroll
      for (int row = 0; row < 4; ++row)
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          po[row][sp] = (row < nrows && sp < S)
                            ? __ldcg(p.part_o + (base0 + (size_t)sp * 16 + row) * HD + threadIdx.x) : 0.f;
    }
    __syncthreads();
    if ((int)threadIdx.x < nrows) {
      const int row = threadIdx.x;
      float M = -INFINITY;
      for (int sp = 0; sp < S; ++sp) M = fmaxf(M, sSc[row * 32 + sp]);
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f;
      for (int sp = 0; sp < S; ++sp) {
        const float sc = exp2f(sSc[row * 32 + sp] - Ms);
        sSc[row * 32 + sp] = sc;
        L += sc * sL[row * 32 + sp];
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      for (int sp = 0; sp < S; ++sp) sSc[row * 32 + sp] *= inv;
    }
    __syncthreads();
    if (threadIdx.x < 128) {
      const int d = threadIdx.x;
      if (small) {
#pragma unroll
        for (int row = 0; row < 4; ++row) {
          if (row < nrows) {
            float acc = 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
              if (sp < S) acc += sSc[row * 32 + sp] * po[row][sp];
            const int qtok = row / p.G, hg = row % p.G;
            p.out[(size_t)(q_start + qtok) * p.out_stride_tok + (size_t)(kvh * p.G + hg) * HD + d] = __float2bfloat16(acc);
          }
        }
      } else {
        for (int row = 0; row < nrows; ++row) {
          float acc = 0.f;
#pragma unroll 8
          for (int sp = 0; sp < S; ++sp)
            acc += sSc[row * 32 + sp] * __ldcg(p.part_o + (base0 + (size_t)sp * 16 + row) * HD + d);
          const int qtok = row / p.G, hg = row % p.G;
          p.out[(size_t)(q_start + qtok) * p.out_stride_tok + (size_t)(kvh * p.G + hg) * HD + d] = __float2bfloat16(acc);
        }
      }
    }
    if (!p.cluster_merge && threadIdx.x == 0) *ctr = 0;        // ready for the next launch
  }
}

}  // namespace

// Launches the TMA decode kernel; kcache / vcache are one layer's [blocks, Hkv, 16, 128] tensors.
int attn_decode_tma_launch(const AttnParams& p, int num_blocks, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(attn_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  CUtensorMap tk, tv;
  const int rows = num_blocks * p.Hkv * 16;
  int rc = make_tmap_bf16_2d(&tk, p.k, rows, HD, HD, 16);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tv, p.v, rows, HD, HD, 16);
  if (rc) return rc;
  dim3 grid(p.num_splits, p.Hkv, p.num_seqs);
  if (p.num_splits > 1 && p.num_splits <= 8 && p.split_counters) {
    // the splits of one (sequence, kv head) as a thread-block cluster: merged after a cluster barrier
    AttnParams pc = p;
    pc.cluster_merge = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(160);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.num_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    int na = 1;
    if (pdl_enabled()) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_tma_kernel, tk, tv, pc);
    return e == cudaSuccess ? 0 : -(int)e;
  }
  return launch_kernel(attn_decode_tma_kernel, grid, dim3(160), SMEM_BYTES, stream, tk, tv, p);
}

}  // namespace swb
