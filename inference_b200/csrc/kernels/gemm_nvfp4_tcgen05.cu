// NVFP4 x NVFP4 GEMM on the block-scaled tensor-core path (W4A4): D[T, N] = alpha * (Aq[T, K] . Wq[N, K]^T) + bias.
//
// Both operands are E2M1 codes, two per byte, K-major, with one unsigned E4M3 scale per 16 elements stored in
// 128-row x 4-scale atoms (512 bytes: row r of the atom at (r % 32) * 16 + (r / 32) * 4, atoms ordered row-atom
// fastest) and one fp32 scale per tensor; alpha is the product of the two tensor scales (the activation's lives on the
// device: it was produced by the quantiser that ran just before). The reference reaches this regime through
// cuBLASLt's FP4 matmul (candle-gen/src/quant/nvfp4_linear.rs, W4A4 lane); here it is one kernel:
//
//   warp 0   one thread: per stage two TMA tiles (128 rows x 256 K = 128 bytes per row, 128-byte swizzle) and two 3-D TMA
//            boxes of four scale atoms each (the atoms of one row-atom are strided in memory), all completing on the
//            stage's mbarrier
//   warp 1   one thread: per stage 8 tcgen05.cp (scale atoms -> tensor memory, the 32-lane x 128-bit shape replicated
//            to the four lane quarters) and 4 tcgen05.mma.kind::mxf4nvf4.block_scale (M 128, N 128, K 64 each) into one
//            of two 128-column fp32 accumulators; tcgen05.commit releases the stage / hands the accumulator over
//   warps 2..17 epilogue: four warps per lane quarter, each a quarter of the tile's columns: the slice is read from
//            tensor memory into registers in one go and the accumulator released at once; * alpha + bias, bf16 and
//            32-byte stores then overlap the next tile's main loop
//
// Persistent: one CTA per SM walks tiles (row-tile fastest, so concurrent CTAs share a weight tile in L2).
// Every wait is bounded (mbar_wait): on timeout the CTA raises the status word, drains its copies and frees its TMEM.
#include "common.cuh"
#include "gemm_tcgen05.cuh"

#include <algorithm>

namespace swb {

SWB_REGISTER_STATUS_UNIT(gemm_nvfp4);

namespace {

constexpr int FM = 128, FK = 256;                    // tile rows; FK elements = 128 bytes of codes per row
constexpr int F_EPI_WARPS = 16;                      // four per TMEM lane quarter
constexpr int F_THREADS = 64 + 32 * F_EPI_WARPS;     // TMA warp, MMA warp, epilogue warps
constexpr uint32_t F_TMEM_COLS = 512;

// FN = 128: two accumulators (the epilogue of a tile overlaps the next tile's main loop), 5 stages.
// FN = 256: one 256-column accumulator (two would leave no tensor memory for the scales), 4 stages; each MMA does twice
//           the work per A fetch and per scale copy.
template <int FN>
struct FCfg {
  static constexpr int ACCS = FN == 128 ? 2 : 1;
  static constexpr int STAGES = FN == 128 ? 5 : 4;
  static constexpr int B_ATOMS = FN / 128;                         // scale atoms of the B tile per 64 K
  static constexpr uint32_t A_BYTES = FM * (FK / 2);               // 16 KB
  static constexpr uint32_t B_BYTES = FN * (FK / 2);
  static constexpr uint32_t SFA_BYTES = 4 * 512;                   // four scale atoms (K 256 = 4 x 64)
  static constexpr uint32_t SFB_BYTES = 4 * 512 * B_ATOMS;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr uint32_t SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr uint32_t SFA_COL = ACCS * FN;                   // scale columns follow the accumulators
  static constexpr uint32_t SFB_COL = SFA_COL + 16;
};

struct FParams {
  const float* a_scale;   // device: activation tensor scale
  float w_scale;
  const bf16* bias;
  bf16* out;
  int ldd, T, N, kblocks, tiles_m, tiles_n;
};

// 32 rows x 16 bytes, rows contiguous: 8-row core matrices 128 bytes apart, no swizzle
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset: one 16-byte column only
  d |= (uint64_t)(128 >> 4) << 32;   // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// E2M1 x E2M1 with UE4M3 scales per 16, fp32 accumulate, both K-major
__host__ __device__ constexpr uint32_t idesc_nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (0u << 23) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                          uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

template <int FN>
__global__ void __launch_bounds__(F_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const FParams p) {
  using Cfg = FCfg<FN>;
  constexpr int F_STAGES = Cfg::STAGES;
  constexpr uint32_t F_STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + F_STAGES * F_STAGE_BYTES);
  uint64_t* bar_empty = bar_full + F_STAGES;
  uint64_t* bar_tfull = bar_empty + F_STAGES;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar_tfull[a], 1);
      mbar_init(&bar_tempty[a], F_EPI_WARPS);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, F_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  const int tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0, outstanding = 0, issue_phase_bits = 0;
      bool ok = true;
      pdl_wait(TL_GEMM_QUANT);
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          ok = mbar_wait(&bar_empty[stage], phase ^ 1, s_abort, 100 + stage);
          if (!ok) break;
          uint8_t* sa = smem + stage * F_STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          uint8_t* ssa = sb + Cfg::B_BYTES;
          uint8_t* ssb = ssa + Cfg::SFA_BYTES;
          mbar_arrive_expect_tx(&bar_full[stage], F_STAGE_BYTES);
          // x counts 16-bit words: 64 per stage; the B tile arrives as 128-row boxes
          tma_load_2d_hint(sa, &tmap_a, &bar_full[stage], kb * 64, tm * FM, pol);
#pragma unroll
          for (int h = 0; h < Cfg::B_ATOMS; ++h)
            tma_load_2d_hint(sb + h * Cfg::A_BYTES, &tmap_b, &bar_full[stage], kb * 64, tn * FN + h * 128, pol);
          // scale atoms: [k atom][row atom][128 words]; box = 128 words x 1 row atom x 4 k atoms
          tma_load_3d(ssa, &tmap_sfa, &bar_full[stage], 0, tm, kb * 4);
#pragma unroll
          for (int h = 0; h < Cfg::B_ATOMS; ++h)
            tma_load_3d(ssb + h * 2048, &tmap_sfb, &bar_full[stage], 0, tn * Cfg::B_ATOMS + h, kb * 4);
          outstanding |= 1u << stage;
          issue_phase_bits = (issue_phase_bits & ~(1u << stage)) | (phase << stage);
          if (++stage == F_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (*s_abort) {
        for (int s = 0; s < F_STAGES; ++s) {
          if (outstanding & (1u << s)) {
            const uint32_t par = (issue_phase_bits >> s) & 1u;
            for (int it = 0; it < (1 << 20); ++it)
              if (mbar_try_wait(&bar_full[s], par)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_nvf4(FM, FN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      pdl_wait(TL_GEMM_QUANT);
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        ok = mbar_wait(&bar_tempty[acc], acc_phase ^ 1, s_abort, 200 + acc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * FN);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          ok = mbar_wait(&bar_full[stage], phase, s_abort, 300 + stage);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * F_STAGE_BYTES);
          const uint32_t ssa = sa + Cfg::A_BYTES + Cfg::B_BYTES, ssb = ssa + Cfg::SFA_BYTES;
          const uint64_t adesc = umma_desc_kmajor_sw128(sa), bdesc = umma_desc_kmajor_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            tmem_cp_sf(tmem_base + Cfg::SFA_COL + 4 * q, sf_desc(ssa + q * 512));
#pragma unroll
            for (int h = 0; h < Cfg::B_ATOMS; ++h)
              tmem_cp_sf(tmem_base + Cfg::SFB_COL + (q * Cfg::B_ATOMS + h) * 4, sf_desc(ssb + h * 2048 + q * 512));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            // 64 codes = 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
            umma_nvf4(tmem_d, adesc + (uint64_t)(2 * q), bdesc + (uint64_t)(2 * q), idesc, (kb > 0 || q > 0) ? 1u : 0u,
                      tmem_base + Cfg::SFA_COL + 4 * q, tmem_base + Cfg::SFB_COL + 4 * q * Cfg::B_ATOMS);
          }
          umma_commit(&bar_empty[stage]);
          if (++stage == F_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&bar_tfull[acc]);
        if (++acc == Cfg::ACCS) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int quarter = warp & 3;                   // the TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;               // which slice of the tile's columns (four warps per quarter)
    constexpr int CHUNKS = FN / 16 / (F_EPI_WARPS / 4);   // 16-column chunks per warp: 4 (FN 256) or 2 (FN 128)
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    pdl_wait();
    const float alpha = __ldg(p.a_scale) * p.w_scale;
    for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      ok = mbar_wait(&bar_tfull[acc], acc_phase, s_abort, 400 + acc);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * FN) + (uint32_t)(part * CHUNKS * 16);
      const int row = tm * FM + row_in_tile;
      // the whole slice goes to registers first, so the accumulator is handed back after one TMEM read latency;
      // scaling, conversion and the global stores then overlap the next tile's main loop
      uint32_t r[CHUNKS][16];
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[ch][0]), "=r"(r[ch][1]), "=r"(r[ch][2]), "=r"(r[ch][3]), "=r"(r[ch][4]), "=r"(r[ch][5]), "=r"(r[ch][6]),
              "=r"(r[ch][7]), "=r"(r[ch][8]), "=r"(r[ch][9]), "=r"(r[ch][10]), "=r"(r[ch][11]), "=r"(r[ch][12]), "=r"(r[ch][13]),
              "=r"(r[ch][14]), "=r"(r[ch][15])
            : "r"(taddr + ch * 16)
            : "memory");
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_tempty[acc]);
#pragma unroll
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int col0 = tn * FN + (part * CHUNKS + ch) * 16;
        if (row < p.T && col0 < p.N) {
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float x0 = __uint_as_float(r[ch][2 * e]) * alpha, x1 = __uint_as_float(r[ch][2 * e + 1]) * alpha;
            if (p.bias) {
              x0 += __bfloat162float(p.bias[col0 + 2 * e]);
              x1 += __bfloat162float(p.bias[col0 + 2 * e + 1]);
            }
            __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
            o[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldd + col0);
          dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
          dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      if (++acc == Cfg::ACCS) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

}  // namespace
}  // namespace swb

extern "C" {

// D[T, N] (bf16, ldd) = a_scale[0] * w_scale * (Aq . Wq^T) + bias. Aq: [T, K / 2] code bytes; Wq: [N, K / 2]; sfa / sfb:
// scale atoms covering ceil(T / 128) / ceil(N / 128) row atoms x K / 64 column atoms; K % 256 == 0, N % 16 == 0,
// 16-byte aligned operands, ldd % 8 == 0.
int swb_gemm_nvfp4_w4a4(const void* Aq, const void* sfa, const void* a_scale, const void* Wq, const void* sfb, float w_scale,
                        void* D, int ldd, int T, int N, int K, const void* bias, void* stream) {
  using namespace swb;
  if (T <= 0 || N <= 0) return 0;
  auto mis = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
  if (K <= 0 || K % FK != 0 || N % 16 != 0 || ldd % 8 != 0 || mis(Aq) || mis(Wq) || mis(sfa) || mis(sfb) || mis(D) || !a_scale)
    return -3;
  FParams p{};
  p.a_scale = reinterpret_cast<const float*>(a_scale);
  p.w_scale = w_scale;
  p.bias = reinterpret_cast<const bf16*>(bias);
  p.out = reinterpret_cast<bf16*>(D);
  p.ldd = ldd;
  p.T = T;
  p.N = N;
  p.kblocks = K / FK;
  static const int forced_fn = [] { const char* e = getenv("SWB_NVFP4_FN"); return e ? atoi(e) : 0; }();
  const int FN = forced_fn == 128 || forced_fn == 256 ? forced_fn : ((N % 256 == 0 || N >= 2048) ? 256 : 128);
  p.tiles_m = (T + FM - 1) / FM;
  p.tiles_n = (N + FN - 1) / FN;
  CUtensorMap ta, tb;
  int rc = make_tmap_u16_2d(&ta, Aq, K / 4, T, K / 2, 64, FM, 1);
  if (rc) return rc;
  rc = make_tmap_u16_2d(&tb, Wq, K / 4, N, K / 2, 64, 128, 1);
  if (rc) return rc;
  CUtensorMap tsa, tsb;
  const unsigned box[3] = {128u, 1u, 4u};
  {
    const unsigned long long ma = (unsigned long long)(T + 127) / 128, mb = (unsigned long long)(N + 127) / 128;
    const unsigned long long da[3] = {128ull, ma, (unsigned long long)K / 64}, db[3] = {128ull, mb, (unsigned long long)K / 64};
    const unsigned long long sa[2] = {512ull, 512ull * ma}, sb[2] = {512ull, 512ull * mb};
    rc = make_tmap_u32_3d(&tsa, sfa, da, sa, box);
    if (rc) return rc;
    rc = make_tmap_u32_3d(&tsb, sfb, db, sb, box);
    if (rc) return rc;
  }
  const int grid = std::min(device_sm_count(), p.tiles_m * p.tiles_n);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int dev = 0;
  cudaGetDevice(&dev);
  if (FN == 256) {
    static bool configured[64] = {false};
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FCfg<256>::SMEM);
      if (e != cudaSuccess) return -(int)e;
      configured[dev] = true;
    }
    return launch_kernel(gemm_nvfp4_kernel<256>, dim3(grid), dim3(F_THREADS), FCfg<256>::SMEM, st, ta, tb, tsa, tsb, p);
  }
  static bool configured[64] = {false};
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FCfg<128>::SMEM);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  return launch_kernel(gemm_nvfp4_kernel<128>, dim3(grid), dim3(F_THREADS), FCfg<128>::SMEM, st, ta, tb, tsa, tsb, p);
}

}  // extern "C"
