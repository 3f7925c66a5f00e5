// bf16 GEMM for sm_100a: D[T, N] = act(A[T, K] * W[N, K]^T + bias) + residual.
//
// Replaces the reference's cuBLAS-backed `linear` (candle-llm/src/primitives/nn.rs:14-19 and every
// dense projection in models/llama.rs) with a hand-written Blackwell kernel:
//   * operands staged global -> shared by TMA (128-byte swizzle, one 64-wide K slab per stage),
//   * tcgen05.mma (kind::f16, M=128, N=16..256) issued by one thread, accumulating fp32 in TMEM,
//   * a 4..8 stage mbarrier pipeline, two TMEM accumulator stages so the epilogue of tile i overlaps
//     the mainloop of tile i+1, persistent CTAs (one per SM),
//   * fused epilogue (bias, SiLU / tanh-GELU, residual add, bf16 or fp32 output),
//   * token counts <= 256 run "swapped": the weight is the M=128 operand and tokens the N operand, so
//     decode-sized batches waste no tensor-core rows; small problems are split along K across CTAs and
//     the last-arriving CTA of a tile reduces the fp32 partials in a fixed order (deterministic).
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue.
#include "common.cuh"
#include "gemm_tcgen05.cuh"

#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

namespace swb {

SWB_REGISTER_STATUS_UNIT(gemm);

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;

// Decode-sized (swapped) problems are bandwidth bound: their pipelines are sized so two CTAs share an
// SM, which lets a dependent kernel's CTAs (programmatic dependent launch) become resident and prefetch
// weights while the predecessor drains. Large problems take the whole SM for one deep pipeline.
template <int BLOCK_N, bool SWAPPED>
struct GemmCfg {
  static constexpr bool TWO_PER_SM = false;  // (decode-sized problems that want two CTAs per SM use the cluster kernel)
  static constexpr int STAGES = TWO_PER_SM ? (BLOCK_N >= 128 ? 3 : (BLOCK_N >= 64 ? 4 : 5))
                                           : (BLOCK_N >= 256 ? 4 : (BLOCK_N >= 128 ? 6 : 8));
  static constexpr int MIN_CTAS = TWO_PER_SM ? 2 : 1;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BLOCK_N * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t TMEM_COLS = (2 * BLOCK_N < 32) ? 32 : 2 * BLOCK_N;
  // staging slabs of the coalescing epilogue: 4 warps x 32 rows x 128 bf16 columns (tokens-as-M, wide tiles only)
  static constexpr uint32_t EPI_BYTES = (!SWAPPED && BLOCK_N >= 128) ? 4 * 32 * 256 : 0;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + EPI_BYTES;
};

// One contiguous run of k-blocks of one output tile, as processed by one CTA.
struct Seg {
  int tile, tm, tn, kb0, kb1;
  bool first;  // first segment of this CTA (selects the partial-sum slot)
};

// Work decomposition shared by the three warp roles so they walk identical segment sequences.
//  * data parallel: CTA c owns whole tiles c, c + grid, ...
//  * stream-K: the tiles x k-blocks iteration space is cut into equal contiguous ranges, one per CTA; a
//    CTA's range may start and end inside a tile, those partial tiles are reduced through the workspace.
struct SegIter {
  const GemmParams& p;
  int it, it_end, next_tile, nseg;
  __device__ explicit SegIter(const GemmParams& pp) : p(pp), nseg(0) {
    it = (int)blockIdx.x * p.iters_per_cta;
    it_end = min(it + p.iters_per_cta, p.tiles_m * p.tiles_n * p.kblocks_total);
    next_tile = (int)blockIdx.x;
  }
  __device__ __forceinline__ void coords(Seg& s) const {
    const int per_group = GROUP_M * p.tiles_n;
    const int g = s.tile / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(GROUP_M, p.tiles_m - first_m);
    const int r = s.tile - g * per_group;
    s.tm = first_m + r % gsize;
    s.tn = r / gsize;
  }
  __device__ __forceinline__ bool next(Seg& s) {
    if (p.stream_k) {
      if (it >= it_end) return false;
      s.tile = it / p.kblocks_total;
      s.kb0 = it - s.tile * p.kblocks_total;
      s.kb1 = min(p.kblocks_total, s.kb0 + (it_end - it));
      it += s.kb1 - s.kb0;
    } else {
      // grouped mode: tiles of row blocks without a weight group are passed over; every role walks the
      // same table, so the sequences stay identical
      for (;;) {
        if (next_tile >= p.tiles_m * p.tiles_n) return false;
        s.tile = next_tile;
        next_tile += (int)gridDim.x;
        if (!p.group_of_mtile) break;
        coords(s);
        if (__ldg(p.group_of_mtile + s.tm) >= 0) break;
      }
      s.kb0 = 0;
      s.kb1 = p.kblocks_total;
    }
    s.first = (nseg++ == 0);
    coords(s);
    return true;
  }
};

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == SWB_ACT_SILU) return silu_f(x);
  if (act == SWB_ACT_GELU_TANH) return gelu_tanh_f(x);
  return x;
}

// One thread's 16 consecutive accumulator columns -> global memory.
// Normal layout: row = token, columns = features. Transposed (swapped operands): row = feature, columns = tokens.
template <bool TRANSPOSED>
__device__ __forceinline__ void epilogue_store16(const GemmParams& p, float* v, int row, int col0) {
  if (row >= p.M) return;
  const int nvalid = min(16, p.N - col0);
  if (nvalid <= 0) return;
  if constexpr (!TRANSPOSED) {
    const size_t off = (size_t)row * p.ldd + col0;
    if (p.vec_ok && nvalid == 16) {
      if (p.bias) {
        const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
        uint4 b0 = __ldg(bp), b1 = __ldg(bp + 1);
        const bf16* bb0 = reinterpret_cast<const bf16*>(&b0);
        const bf16* bb1 = reinterpret_cast<const bf16*>(&b1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] += __bfloat162float(bb0[j]);
          v[8 + j] += __bfloat162float(bb1[j]);
        }
      }
      if (p.act != SWB_ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = apply_act(v[j], p.act);
      }
      if (p.residual) {
        const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ld_res + col0);
        uint4 r0 = rp[0], r1 = rp[1];
        const bf16* rr0 = reinterpret_cast<const bf16*>(&r0);
        const bf16* rr1 = reinterpret_cast<const bf16*>(&r1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] += __bfloat162float(rr0[j]);
          v[8 + j] += __bfloat162float(rr1[j]);
        }
      }
      if (p.out_fp32) {
        float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off);
#pragma unroll
        for (int j = 0; j < 4; ++j) op[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      } else {
        uint4 o[2];
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + off);
        if (p.scatter.enabled == 1) {   // a 16-column chunk never straddles a head (128 columns)
          const GemmScatter& sc = p.scatter;
          const int which = col0 / sc.hd_total;
          const int rem = col0 - which * sc.hd_total;
          const int h = rem >> 7;
          const int r = h / sc.heads_per_rank;
          const int grow = row + (row < sc.row_split ? sc.row_off0 : sc.row_off1);
          op = reinterpret_cast<uint4*>(sc.peer[r] + (size_t)grow * sc.ld +
                                        (which * sc.heads_per_rank + (h - r * sc.heads_per_rank)) * 128 + (rem & 127));
        } else if (p.scatter.enabled == 2) {
          const GemmScatter& sc = p.scatter;
          const int r = row / sc.rows_per_rank;
          op = reinterpret_cast<uint4*>(sc.peer[r] +
                                        ((size_t)sc.src_rank * sc.rows_per_rank + (row - r * sc.rows_per_rank)) * sc.ld +
                                        col0);
        }
        op[0] = o[0];
        op[1] = o[1];
      }
    } else {
      for (int j = 0; j < nvalid; ++j) {
        float x = v[j];
        if (p.bias) x += __bfloat162float(p.bias[col0 + j]);
        x = apply_act(x, p.act);
        if (p.residual) x += __bfloat162float(p.residual[(size_t)row * p.ld_res + col0 + j]);
        if (p.out_fp32)
          reinterpret_cast<float*>(p.out)[off + j] = x;
        else
          reinterpret_cast<bf16*>(p.out)[off + j] = __float2bfloat16(x);
      }
    }
  } else {
    const float b = p.bias ? __bfloat162float(p.bias[row]) : 0.f;
#pragma unroll 4
    for (int j = 0; j < nvalid; ++j) {
      const int tok = col0 + j;
      float x = apply_act(v[j] + b, p.act);
      if (p.residual) x += __bfloat162float(p.residual[(size_t)tok * p.ld_res + row]);
      const size_t off = (size_t)tok * p.ldd + row;
      if (p.out_fp32)
        reinterpret_cast<float*>(p.out)[off] = x;
      else
        reinterpret_cast<bf16*>(p.out)[off] = __float2bfloat16(x);
    }
  }
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Destination of the 8 bf16 at (row, col0 .. col0 + 7) under the peer dispatch modes of GemmScatter.
__device__ __forceinline__ bf16* scatter_dst(const GemmScatter& sc, int row, int col0) {
  if (sc.enabled == 1) {
    const int which = col0 / sc.hd_total;
    const int rem = col0 - which * sc.hd_total;
    const int h = rem >> 7;
    const int r = h / sc.heads_per_rank;
    const int grow = row + (row < sc.row_split ? sc.row_off0 : sc.row_off1);
    return sc.peer[r] + (size_t)grow * sc.ld + (which * sc.heads_per_rank + (h - r * sc.heads_per_rank)) * 128 +
           (rem & 127);
  }
  const int r = row / sc.rows_per_rank;
  return sc.peer[r] + ((size_t)sc.src_rank * sc.rows_per_rank + (row - r * sc.rows_per_rank)) * sc.ld + col0;
}

// Coalescing epilogue for peer dispatch: every epilogue warp stages its 32 rows x 128 columns (bf16, bias and
// activation applied) in shared memory, then writes each row's 256 bytes with 16 lanes x 16 bytes, so what crosses
// NVLink are 256-byte contiguous runs instead of 32-byte fragments. 16-byte chunk c of row r is stored at c ^ (r & 7).
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_scatter_staged(const GemmParams& p, uint32_t taddr, uint8_t* slab, int lane,
                                                        int row0, int col_base) {
#pragma unroll 1
  for (int sl = 0; sl < BLOCK_N / 128; ++sl) {
#pragma unroll 1
    for (int ch = 0; ch < 8; ++ch) {
      float v[16];
      tmem_ld_32x32b_x16(taddr + sl * 128 + ch * 16, v);
      const int col0 = col_base + sl * 128 + ch * 16;
      if (p.bias && col0 < p.N) {
        const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
        const uint4 b0 = __ldg(bp), b1 = __ldg(bp + 1);
        const bf16* bb0 = reinterpret_cast<const bf16*>(&b0);
        const bf16* bb1 = reinterpret_cast<const bf16*>(&b1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] += __bfloat162float(bb0[j]);
          v[8 + j] += __bfloat162float(bb1[j]);
        }
      }
      if (p.act != SWB_ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = apply_act(v[j], p.act);
      }
      if (p.residual && row0 + lane < p.M && col0 < p.N) {
        const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (size_t)(row0 + lane) * p.ld_res + col0);
        const uint4 r0 = rp[0], r1 = rp[1];
        const bf16* rr0 = reinterpret_cast<const bf16*>(&r0);
        const bf16* rr1 = reinterpret_cast<const bf16*>(&r1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] += __bfloat162float(rr0[j]);
          v[8 + j] += __bfloat162float(rr1[j]);
        }
      }
      uint4 o[2];
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      uint8_t* rowp = slab + lane * 256;
      *reinterpret_cast<uint4*>(rowp + (((2 * ch) ^ (lane & 7)) << 4)) = o[0];
      *reinterpret_cast<uint4*>(rowp + (((2 * ch + 1) ^ (lane & 7)) << 4)) = o[1];
    }
    __syncwarp();
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int r = 2 * it + (lane >> 4), c = lane & 15;
      const uint4 val = *reinterpret_cast<const uint4*>(slab + r * 256 + ((c ^ (r & 7)) << 4));
      const int row = row0 + r, col0 = col_base + sl * 128 + c * 8;
      if (row < p.M && col0 < p.N) {
        bf16* dst = p.scatter.enabled ? scatter_dst(p.scatter, row, col0)
                                      : reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldd + col0;
        *reinterpret_cast<uint4*>(dst) = val;
      }
    }
    __syncwarp();
  }
}

template <int BLOCK_N, bool TRANSPOSED>
__global__ void __launch_bounds__(GEMM_THREADS, (GemmCfg<BLOCK_N, TRANSPOSED>::MIN_CTAS))
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  using Cfg = GemmCfg<BLOCK_N, TRANSPOSED>;
  constexpr int STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_tfull = bar_empty + STAGES;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_last = s_abort + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar_tfull[a], 1);
      mbar_init(&bar_tempty[a], 4);
    }
    *s_abort = 0;
    *s_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const uint64_t pol_a = p.stream_a ? l2_policy_evict_first() : l2_policy_evict_last();
      const uint64_t pol_b = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t outstanding = 0;       // stages whose TMA was issued and not yet known consumed
      uint32_t issue_phase_bits = 0;  // parity each outstanding stage's full barrier will complete
      bool ok = true;
      Seg c;
      // A static weight operand does not depend on the predecessor kernel: start streaming it into the
      // (still empty) ring before waiting on the programmatic dependency.
      int prefetched = 0;
      if (p.stream_a) {
        SegIter pre(p);
        while (prefetched < STAGES && pre.next(c)) {
          for (int kb = c.kb0; kb < c.kb1 && prefetched < STAGES; ++kb) {
            uint8_t* sa = smem + prefetched * Cfg::STAGE_BYTES;
            mbar_arrive_expect_tx(&bar_full[prefetched], Cfg::STAGE_BYTES);
            tma_load_2d_hint(sa, &tmap_a, &bar_full[prefetched], kb * BK, c.tm * BM, pol_a);
            outstanding |= 1u << prefetched;
            ++prefetched;
          }
        }
      }
      pdl_wait(TL_GEMM);
      int issued = 0;
      SegIter iter(p);
      while (ok && iter.next(c)) {
        const int b_row = c.tn * BLOCK_N + (p.group_of_mtile ? __ldg(p.group_of_mtile + c.tm) * p.group_rows : 0);
        for (int kb = c.kb0; kb < c.kb1; ++kb, ++issued) {
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (issued < prefetched) {
            // the A half of this stage is already in flight (first pass over the ring: stage == issued)
            tma_load_2d_hint(sb, &tmap_b, &bar_full[stage], kb * BK, b_row, pol_b);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          ok = mbar_wait(&bar_empty[stage], phase ^ 1, s_abort, 100 + stage);
          if (!ok) break;
          outstanding &= ~(1u << stage);
          mbar_arrive_expect_tx(&bar_full[stage], Cfg::STAGE_BYTES);
          if (p.conv_c) {
            // implicit 3x3 convolution: this k-block is one tap of the window over one 64-channel slab
            const int slabs = p.conv_c / BK, tap = kb / slabs, c0 = (kb - tap * slabs) * BK;
            const int hw = p.conv_h * p.conv_w, m0 = c.tm * BM, img = m0 / hw, rem = m0 - img * hw;
            const int y0 = rem / p.conv_w, x0 = rem - y0 * p.conv_w;
            tma_load_4d_hint(sa, &tmap_a, &bar_full[stage], c0, x0 + tap % 3 - 1, y0 + tap / 3 - 1, img, pol_a);
          } else {
            tma_load_2d_hint(sa, &tmap_a, &bar_full[stage], kb * BK, c.tm * BM, pol_a);
          }
          tma_load_2d_hint(sb, &tmap_b, &bar_full[stage], kb * BK, b_row, pol_b);
          outstanding |= 1u << stage;
          issue_phase_bits = (issue_phase_bits & ~(1u << stage)) | (phase << stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (*s_abort) {
        // Drain: let every copy this thread issued land before the CTA's shared memory is released.
        for (int s = 0; s < STAGES; ++s) {
          if (outstanding & (1u << s)) {
            const uint32_t par = (issue_phase_bits >> s) & 1u;
            for (int it = 0; it < (1 << 20); ++it)
              if (mbar_try_wait(&bar_full[s], par)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      SegIter iter(p);
      Seg c;
      pdl_wait(TL_GEMM);
      while (ok && iter.next(c)) {
        const int kb0 = c.kb0, kb1 = c.kb1;
        ok = mbar_wait(&bar_tempty[acc], acc_phase ^ 1, s_abort, 200 + acc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BLOCK_N);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&bar_full[stage], phase, s_abort, 300 + stage);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint64_t adesc = umma_desc_kmajor_sw128(sa);
          const uint64_t bdesc = umma_desc_kmajor_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advance 16 bf16 = 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
            umma_f16_ss(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                        (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bar_empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&bar_tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    SegIter iter(p);
    Seg c;
    pdl_wait();
    while (ok && iter.next(c)) {
      ok = mbar_wait(&bar_tfull[acc], acc_phase, s_abort, 400 + acc);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N);
      const int row = c.tm * BM + row_in_tile;
      const int col_base = c.tn * BLOCK_N;
      const bool whole = (c.kb0 == 0 && c.kb1 == p.kblocks_total);
      if (whole) {
        if constexpr (Cfg::EPI_BYTES > 0) {
          if (p.scatter.enabled || p.staged_epilogue) {
            uint8_t* slab = smem + STAGES * Cfg::STAGE_BYTES + 256 + (warp - 2) * (32 * 256);
            epilogue_scatter_staged<BLOCK_N>(p, taddr, slab, lane, c.tm * BM + quarter * 32, col_base);
          } else {
#pragma unroll 1
            for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
              float v[16];
              tmem_ld_32x32b_x16(taddr + ch * 16, v);
              epilogue_store16<TRANSPOSED>(p, v, row, col_base + ch * 16);
            }
          }
        } else {
#pragma unroll 1
          for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
            float v[16];
            tmem_ld_32x32b_x16(taddr + ch * 16, v);
            epilogue_store16<TRANSPOSED>(p, v, row, col_base + ch * 16);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_tempty[acc]);
      } else {
        // partial tile: park fp32 partial sums in this CTA's slot, the last contributor reduces them
        constexpr size_t SLOT = (size_t)BLOCK_N * BM;
        float* ws_mine = p.workspace + ((size_t)blockIdx.x * 2 + (c.first ? 0 : 1)) * SLOT;
#pragma unroll 1
        for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
          float v[16];
          tmem_ld_32x32b_x16(taddr + ch * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(&ws_mine[(ch * 16 + j) * BM + row_in_tile], v[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_tempty[acc]);
        const int tile_it0 = c.tile * p.kblocks_total;
        const int first_cta = tile_it0 / p.iters_per_cta;
        const int last_cta = (tile_it0 + p.kblocks_total - 1) / p.iters_per_cta;
        const int contributors = last_cta - first_cta + 1;
        __threadfence();
        epi_bar_sync();
        if (epi_tid == 0) {
          const int old = atomicAdd(&p.counters[c.tile], 1);
          const int last = (old == contributors - 1) ? 1 : 0;
          if (last) p.counters[c.tile] = 0;  // ready for the next launch
          *s_last = last;
        }
        epi_bar_sync();
        if (*s_last) {
          __threadfence();
#pragma unroll 1
          for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
            for (int cta = first_cta; cta <= last_cta; ++cta) {
              // a contributor whose range starts inside this tile used slot 0, otherwise slot 1
              const int slot = (cta * p.iters_per_cta >= tile_it0) ? 0 : 1;
              const float* wsp = p.workspace + ((size_t)cta * 2 + slot) * SLOT + (ch * 16) * BM + row_in_tile;
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += __ldcg(&wsp[j * BM]);
            }
            epilogue_store16<TRANSPOSED>(p, v, row, col_base + ch * 16);
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

}  // namespace

// 2-D bf16 row-major [rows, cols] (row stride ld elements), box = 64 columns x box_rows rows, 128B swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  auto encode = get_encode_fn();
  if (!encode) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 1000;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// Cached 2-D map over 16-bit elements (packed quantised weights are moved as opaque 16-bit words):
// [rows, cols] with a row pitch in bytes, box = box_cols x box_rows, optional 128-byte swizzle.
int make_tmap_u16_2d(CUtensorMap* out, const void* ptr, long long cols, long long rows, long long row_pitch_bytes,
                     int box_cols, int box_rows, int swizzle128) {
  struct Key {
    const void* ptr;
    long long cols, rows, pitch;
    int bc, br, sw;
    bool operator==(const Key& o) const {
      return ptr == o.ptr && cols == o.cols && rows == o.rows && pitch == o.pitch && bc == o.bc && br == o.br && sw == o.sw;
    }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      size_t h = reinterpret_cast<size_t>(k.ptr);
      for (long long v : {k.cols, k.rows, k.pitch, (long long)k.bc, (long long)k.br, (long long)k.sw})
        h = h * 1000003u ^ (size_t)v;
      return h;
    }
  };
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  const Key key{ptr, cols, rows, row_pitch_bytes, box_cols, box_rows, swizzle128};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  auto encode = get_encode_fn();
  if (!encode) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 1000;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// Uncached 3-D map over 32-bit words, no swizzle: dims / box innermost first, strides in bytes for dims 1 and 2.
int make_tmap_u32_3d(CUtensorMap* out, const void* ptr, const unsigned long long dims[3], const unsigned long long strides[2],
                     const unsigned box[3]) {
  auto encode = get_encode_fn();
  if (!encode) return -1;
  cuuint64_t d[3] = {dims[0], dims[1], dims[2]};
  cuuint64_t st[2] = {strides[0], strides[1]};
  cuuint32_t b[3] = {box[0], box[1], box[2]};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(ptr), d, st, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// NHWC bf16 activation [n, h, w, c] (contiguous): dims (c, w, h, n), box (64, box_w, box_h, 1), 128-byte swizzle, zero
// fill outside (rows of the box land in (y, x) order, 128 bytes each: the K-major A tile the MMA descriptor expects).
int make_tmap_bf16_nhwc(CUtensorMap* out, const void* ptr, int n, int h, int w, int c, int box_w, int box_h) {
  auto encode = get_encode_fn();
  if (!encode) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c * 2, (cuuint64_t)w * c * 2, (cuuint64_t)h * w * c * 2};
  cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)box_w, (cuuint32_t)box_h, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

int device_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

namespace {

template <int BLOCK_N, bool TRANSPOSED>
int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N, TRANSPOSED>;
  auto kern = gemm_bf16_tcgen05_kernel<BLOCK_N, TRANSPOSED>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  return launch_kernel(kern, dim3(grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, ta, tb, p);
}

template <bool TRANSPOSED>
int launch_bn(int block_n, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
              cudaStream_t stream) {
  switch (block_n) {
    case 16: return launch_cfg<16, TRANSPOSED>(ta, tb, p, grid, stream);
    case 32: return launch_cfg<32, TRANSPOSED>(ta, tb, p, grid, stream);
    case 64: return launch_cfg<64, TRANSPOSED>(ta, tb, p, grid, stream);
    case 128: return launch_cfg<128, TRANSPOSED>(ta, tb, p, grid, stream);
    case 256: return launch_cfg<256, TRANSPOSED>(ta, tb, p, grid, stream);
  }
  return -2;
}

}  // namespace

// 1 when a gate-up projection of this shape runs in the decode cluster kernel, whose epilogue can apply the gated
// activation (the same routing rule as in gemm_bf16_launch).
int gemm_bf16_gated_supported(int T, int N, int K) {
  return gemm_decode_cluster_supported(T) && (N + BM - 1) / BM <= 2 * device_sm_count() && (K + BK - 1) / BK >= 8 &&
         (N % 2) == 0;
}

int gemm_bf16_launch(const GemmArgs& a, cudaStream_t stream) {
  if (a.T <= 0 || a.N <= 0 || a.K <= 0) return 0;
  if ((a.K % 8) != 0 || (a.lda % 8) != 0 || (a.ldw % 8) != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.W) & 15)) return -3;
  const int sms = device_sm_count();

  int swapped = a.force_mode;
  if (a.scatter) {
    if (a.out_fp32 || a.residual || (a.N % 16) != 0 || (a.scatter->ld % 8) != 0) return -3;
    if (a.scatter->enabled == 1 && a.scatter->hd_total % 128 != 0) return -3;
    if (a.scatter->enabled == 2 && a.scatter->rows_per_rank <= 0) return -3;
    swapped = 0;
  }
  if (a.group_of_mtile) {
    if (a.scatter || a.groups <= 0 || a.bias || a.residual) return -3;
    swapped = 0;
  }
  if (a.conv_c > 0) {
    // implicit 3x3 convolution: tokens-as-M only; a 128-pixel tile is a run of one image row or whole rows
    const long hw = (long)a.conv_h * a.conv_w;
    if (a.scatter || a.group_of_mtile || a.ssq_in || a.ssq_out || (a.peer && a.peer->mode) || a.act >= SWB_ACT_SWIGLU_PAIRS)
      return -3;
    if (a.conv_n <= 0 || a.conv_h <= 0 || a.conv_w <= 0 || (a.conv_c % BK) != 0 || a.K != 9 * a.conv_c ||
        (long)a.T != hw * a.conv_n || (hw % BM) != 0 || !((a.conv_w % BM) == 0 || (BM % a.conv_w) == 0))
      return -3;
    swapped = 0;
  }
  if (swapped < 0) swapped = (a.T <= 256) ? 1 : 0;
  if (a.peer && a.peer->mode) {   // cross-rank sum in the epilogue: decode cluster kernel only, any K
    if (a.scatter || a.group_of_mtile || !gemm_decode_cluster_supported(a.T)) return -3;
    return gemm_decode_cluster_launch(a, a.force_mode == 2 ? a.force_ctas : 0, stream);
  }
  // decode-sized problems with at most two weight tiles per SM: the two-CTAs-per-SM cluster kernel (split-K over a
  // cluster with a DSMEM reduction when tiles are few, plain whole tiles otherwise)
  // the folded-norm chain lives in the decode cluster kernel only
  if ((a.ssq_out || a.ssq_in) && (a.scatter || a.group_of_mtile || a.force_mode == 0 || a.force_mode == 1 ||
                                  !gemm_bf16_gated_supported(a.T, a.N & ~1, a.K)))
    return -3;
  // gated-pair epilogues exist in the decode cluster kernel only (bf16 output, no residual)
  const bool pairs = a.act >= SWB_ACT_SWIGLU_PAIRS;
  if (pairs && (a.scatter || a.group_of_mtile || a.residual || a.out_fp32 || (a.N & 1) || a.force_mode == 0 ||
                a.force_mode == 1 || !gemm_bf16_gated_supported(a.T, a.N, a.K)))
    return -3;
  if (!a.scatter && !a.group_of_mtile && !a.conv_c && (a.force_mode == 2 || (a.force_mode < 0 && gemm_decode_cluster_supported(a.T) && (a.N + BM - 1) / BM <= 2 * sms &&
                            (a.K + BK - 1) / BK >= 8))) {
    if (!gemm_decode_cluster_supported(a.T)) return -4;
    return gemm_decode_cluster_launch(a, a.force_mode == 2 ? a.force_ctas : 0, stream);
  }
  if (swapped > 1) swapped = 1;

  GemmParams p{};
  p.K = a.K;
  p.kblocks_total = (a.K + BK - 1) / BK;
  p.ldd = a.ldd;
  p.out = a.D;
  p.out_fp32 = a.out_fp32;
  p.bias = reinterpret_cast<const bf16*>(a.bias);
  p.residual = reinterpret_cast<const bf16*>(a.residual);
  p.ld_res = a.ld_res;
  p.act = a.act;
  p.status = nullptr;
  if (a.scatter) {
    p.scatter = *a.scatter;
  }
  static const int staged_default = [] {
    const char* e = getenv("SWB_GEMM_STAGED");   // 0 restores the row-per-thread stores (comparison runs)
    return e ? atoi(e) : 1;
  }();
  p.staged_epilogue = staged_default;

  int block_n;
  CUtensorMap ta, tb;
  if (swapped) {
    if (a.T > 256) return -4;
    block_n = a.T <= 16 ? 16 : a.T <= 32 ? 32 : a.T <= 64 ? 64 : a.T <= 128 ? 128 : 256;
    if (a.force_block_n > 0) block_n = a.force_block_n;
    if (block_n < a.T) return -4;
    p.M = a.N;
    p.N = a.T;
    p.transposed = 1;
    p.stream_a = 1;
    p.tiles_m = (a.N + BM - 1) / BM;
    p.tiles_n = 1;
    int r = make_tmap_bf16_2d(&ta, a.W, a.N, a.K, a.ldw, BM);
    if (r) return r;
    r = make_tmap_bf16_2d(&tb, a.A, a.T, a.K, a.lda, block_n);
    if (r) return r;
    p.vec_ok = 0;
  } else {
    block_n = a.N >= 256 ? 256 : a.N >= 128 ? 128 : a.N >= 64 ? 64 : a.N >= 32 ? 32 : 16;
    if (block_n == 256) {
      // wave quantisation: with few row tiles a 128-wide tile can fill the SMs better than a 256-wide one does,
      // at roughly 0.85 of its per-SM rate
      const long tm = (a.T + BM - 1) / BM;
      auto fill = [&](int bn) {
        const long tiles = tm * ((a.N + bn - 1) / bn);
        const long waves = (tiles + sms - 1) / sms;
        return (double)tiles / (double)(waves * sms);
      };
      if (fill(128) * 0.85 > fill(256) * 1.02) block_n = 128;
    }
    if (a.force_block_n > 0) block_n = a.force_block_n;
    p.M = a.T;
    p.N = a.N;
    p.transposed = 0;
    p.stream_a = 0;
    p.tiles_m = (a.T + BM - 1) / BM;
    p.tiles_n = (a.N + block_n - 1) / block_n;
    int r;
    if (a.conv_c > 0) {
      const int box_w = a.conv_w >= BM ? BM : a.conv_w;
      r = make_tmap_bf16_nhwc(&ta, a.A, a.conv_n, a.conv_h, a.conv_w, a.conv_c, box_w, BM / box_w);
      p.conv_h = a.conv_h;
      p.conv_w = a.conv_w;
      p.conv_c = a.conv_c;
    } else {
      r = make_tmap_bf16_2d(&ta, a.A, a.T, a.K, a.lda, BM);
    }
    if (r) return r;
    r = make_tmap_bf16_2d(&tb, a.W, a.group_of_mtile ? a.groups * a.N : a.N, a.K, a.ldw, block_n);
    if (r) return r;
    p.group_of_mtile = a.group_of_mtile;
    p.group_rows = a.N;
    const size_t esz = a.out_fp32 ? 4 : 2;
    p.vec_ok = ((a.ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(a.D) & 15) == 0) &&
               (!a.bias || (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0) &&
               (!a.residual || (((reinterpret_cast<uintptr_t>(a.residual) & 15) == 0) && (a.ld_res % 8 == 0)));
    if (a.scatter && !p.vec_ok) return -3;
    if (!p.vec_ok || a.out_fp32 || (a.N % 16) != 0) p.staged_epilogue = 0;
  }

  const int tiles = p.tiles_m * p.tiles_n;
  const size_t counter_bytes = SWB_GEMM_COUNTER_BYTES;
  const size_t slot_bytes = (size_t)block_n * BM * sizeof(float);
  const long total_iters = (long)tiles * p.kblocks_total;
  // stream-K needs two partial slots per CTA and one counter per tile
  const bool ws_ok = a.workspace && a.workspace_bytes >= counter_bytes + (size_t)4 * sms * slot_bytes &&
                     tiles <= (int)(counter_bytes / sizeof(int));
  int grid;
  // decode-sized (swapped) problems are bandwidth bound and rarely fill a wave of whole tiles: balance them
  // exactly; large token counts keep whole tiles per CTA (no partial-tile reduction traffic)
  bool stream_k = ws_ok && a.force_ctas >= 0 && swapped && (tiles % sms != 0) && total_iters >= 2;
  if (a.force_ctas > 0 && ws_ok) stream_k = true;
  if (a.group_of_mtile) stream_k = false;   // whole tiles only: the skip table is indexed by row tile
  if (stream_k) {
    const int per_sm = 1;
    int want = a.force_ctas > 0 ? std::min(a.force_ctas, per_sm * sms) : per_sm * sms;
    // keep at least 4 k-blocks per CTA so the pipeline fill is amortised
    want = (int)std::max<long>(1, std::min<long>(want, total_iters / 4 > 0 ? total_iters / 4 : 1));
    const int per = (int)((total_iters + want - 1) / want);
    grid = (int)((total_iters + per - 1) / per);
    p.iters_per_cta = per;
    p.stream_k = 1;
  } else {
    grid = std::min(tiles, sms);
    p.iters_per_cta = p.kblocks_total;
    p.stream_k = 0;
  }
  p.counters = reinterpret_cast<int*>(a.workspace);
  p.workspace = a.workspace ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.workspace) + counter_bytes)
                            : nullptr;
  return swapped ? launch_bn<true>(block_n, ta, tb, p, grid, stream) : launch_bn<false>(block_n, ta, tb, p, grid, stream);
}

}  // namespace swb
