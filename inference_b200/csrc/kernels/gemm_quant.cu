// Weight-only quantised GEMM for decode-sized token counts (T <= 64): D[T, N] = A[T, K] * dequant(Wq)[N, K]^T.
//
// The packed weights are the only large stream, so they move like one: a TMA thread copies raw 128-row x 256-K
// blocks of packed bytes into a 3-4 deep shared-memory ring (started before the programmatic dependency wait: weights
// are static). Sixteen dequantisation warps expand them (one 64-column group of one row per thread) to bf16 in the 128-byte-swizzled
// K-major layout tcgen05.mma reads; a second TMA thread brings the activations; one thread issues the MMAs
// (weights as the M operand) into a TMEM accumulator. K is split over CTAs; fp32 partial tiles meet in a workspace and
// the last CTA to arrive for a tile sums them in split order (deterministic).
// Integer -> float conversion uses the 2^23 mantissa trick (byte permute into 0x4B000000, subtract), not I2F.
//
// Formats: 0 GGUF Q4_K (144-byte super-blocks of 256, 6-bit sub-block scales / mins), 1 GGUF Q8_0 (34-byte blocks of
// 32), 2 / 3 group-affine 4 / 8 bit with 64-wide groups (packed uint32 + bf16 scales + bf16 biases, w = scale * q +
// bias; the MLX layout). They replace llama.cpp-derived MMVQ/MMQ kernels in the reference
// (candle-kernels/src/mmvq_gguf.cu, mmq_gguf/) and MLX's quantized_matmul (mlx-gen quant/mod.rs:518-571).
#include "common.cuh"
#include "gemm_tcgen05.cuh"

#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>

namespace swb {

bool gemv_q4k_accepts(int T, int K, int lda, const void* A, const void* Wq);      // gemv_q4k.cu
int gemv_q4k_launch(const void* A, int lda, const void* Wq, void* D, int ldd, int T, int N, int K, const void* bias,
                    cudaStream_t stream);

SWB_REGISTER_STATUS_UNIT(gemm_quant);

namespace {

constexpr int QBM = 128;        // features per tile
constexpr int QBK = 256;        // K per raw block
constexpr int QSK = 128;        // K per MMA stage (two stages per raw block)
constexpr int QTHREADS = 608;   // warp 0 raw TMA, warp 1 MMA, warp 2 activation TMA, warps 3..18 dequantise (+ epilogue)
constexpr uint32_t QA_BYTES = QBM * QSK * 2;   // 32 KB: two 64-column atoms of 16 KB
constexpr uint32_t QATOM = QBM * 128;          // 16 KB

struct QParams {
  const uint8_t* w;            // packed weights (dequant_rows reads them directly; the GEMM through TMA)
  const bf16* scales;          // group-affine only: [N, K/64]
  const bf16* biases;          // group-affine only: [N, K/64]
  long long row_bytes;         // bytes per packed weight row
  int N, K, T;
  int kblocks, splits, kb_per_split;
  bf16* out;
  int ldd;
  const bf16* bias;
  float* workspace;            // [tiles * splits][BLOCK_N * 128] fp32
  int* counters;               // [tiles]
  const uint8_t* sf;           // NVFP4 only: unsigned E4M3 block scales in 128 x 4 atoms (see DqNvfp4)
  int sf_m_atoms;              // NVFP4 only: row atoms of the scale tensor = ceil(N / 128)
  float gscale;                // NVFP4 only: per-tensor fp32 scale
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// byte I of x as a float, exactly: place it in the mantissa of 2^23 and subtract 2^23
template <int I>
__device__ __forceinline__ float byte_f(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650 | I)) - 8388608.f;
}
// four bytes of x -> 4 bf16 of (s * byte + m), packed as two 32-bit words
__device__ __forceinline__ void cvt4(uint32_t x, float s, float m, uint32_t& o0, uint32_t& o1) {
  o0 = pack2(fmaf(s, byte_f<0>(x), m), fmaf(s, byte_f<1>(x), m));
  o1 = pack2(fmaf(s, byte_f<2>(x), m), fmaf(s, byte_f<3>(x), m));
}

// Packed-pair arithmetic for 4-bit fields: (x & 0x000F000F) | 0x43004300 is the bf16 pair (128 + n0, 128 + n4) exactly
// (7-bit mantissa, exponent 2^7), one subtraction removes the 128 and one fused multiply-add applies scale and offset
// to both lanes; the scale and offset are rounded to bf16 first.
__device__ __forceinline__ uint32_t nib2(uint32_t x, uint32_t s2, uint32_t m2) {
  uint32_t v = (x & 0x000F000Fu) | 0x43004300u, r;
  asm("{\n.reg .b32 t;\nsub.bf16x2 t, %1, %4;\nfma.rn.bf16x2 %0, t, %2, %3;\n}" : "=r"(r) : "r"(v), "r"(s2), "r"(m2), "r"(0x43004300u));
  return r;
}
__device__ __forceinline__ uint32_t dup_bf16(float f) { return pack2(f, f); }

// Every functor expands one 64-column group `g` (0..3) of one row's 256-K raw block into 8 chunks of 8 bf16.
// `blk` points at the row's raw block (shared or global memory); SWZ: the block is a 128-byte row stored with the
// TMA 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
struct DqQ4K {
  static constexpr int RAW_ROW = 144, RAW_STAGES = 4, BOXES = 1;
  static constexpr bool SWIZZLED = false;
  template <bool SWZ>
  static __device__ __forceinline__ void run(const uint8_t* blk, int /*srow*/, const QParams&, int /*grow*/, int /*kb*/,
                                             int g, uint4* out) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
    const float d = __low2float(dd), dmin = __high2float(dd);
    auto sb = [&](int i) -> uint32_t {   // byte i (0..11) of the packed 6-bit scales / mins
      const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
      return (w >> ((i & 3) * 8)) & 0xFFu;
    };
    float s[2], m[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = g * 2 + e;
      uint32_t scv, mv;
      if (g < 2) {
        scv = sb(j) & 63u;
        mv = sb(j + 4) & 63u;
      } else {
        scv = (sb(j + 4) & 0xFu) | ((sb(j - 4) >> 6) << 4);
        mv = (sb(j + 4) >> 4) | ((sb(j) >> 6) << 4);
      }
      s[e] = d * (float)scv;
      m[e] = -dmin * (float)mv;
    }
    const uint32_t s2[2] = {dup_bf16(s[0]), dup_bf16(s[1])}, m2[2] = {dup_bf16(m[0]), dup_bf16(m[1])};
    // 32 bytes: low nibbles are weights 0..31 of the group (sub-block 2g), high nibbles weights 32..63 (2g + 1)
    const uint4* qs = reinterpret_cast<const uint4*>(blk + 16 + g * 32);
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const uint4 q = qs[v];
      const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t x = w4[c * 2 + u];
          // bytes b0..b3 of x: low nibbles are four consecutive weights of the low sub-block, high nibbles of the high
          const uint32_t a = nib2(x, s2[0], m2[0]), b = nib2(x >> 8, s2[0], m2[0]);     // (b0, b2), (b1, b3)
          const uint32_t cc = nib2(x >> 4, s2[1], m2[1]), dd2 = nib2(x >> 12, s2[1], m2[1]);
          lo[u * 2] = __byte_perm(a, b, 0x5410);
          lo[u * 2 + 1] = __byte_perm(a, b, 0x7632);
          hi[u * 2] = __byte_perm(cc, dd2, 0x5410);
          hi[u * 2 + 1] = __byte_perm(cc, dd2, 0x7632);
        }
        out[v * 2 + c] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        out[4 + v * 2 + c] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      }
    }
  }
};

struct DqQ80 {
  static constexpr int RAW_ROW = 272, RAW_STAGES = 3, BOXES = 1;
  static constexpr bool SWIZZLED = false;
  template <bool SWZ>
  static __device__ __forceinline__ void run(const uint8_t* blk, int, const QParams&, int, int, int g, uint4* out) {
    // two 34-byte blocks (fp16 scale + 32 int8) = 68 bytes, 4-byte aligned
    const uint32_t* src = reinterpret_cast<const uint32_t*>(blk + g * 68);
    uint32_t r[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) r[i] = src[i];
    // block 0: scale = low half of r[0], quants = bytes 2..33; block 1: scale = high half of r[8], quants = bytes 36..67
    const float d0 = __half2float(__ushort_as_half((unsigned short)(r[0] & 0xFFFF)));
    const float d1 = __half2float(__ushort_as_half((unsigned short)(r[8] >> 16)));
#pragma unroll
    for (int c = 0; c < 4; ++c) {   // 8 quants of block 0 start at byte 2 + 8c: straddle words -> funnel shift by 16
      const uint32_t a = __funnelshift_r(r[2 * c], r[2 * c + 1], 16) ^ 0x80808080u;
      const uint32_t b = __funnelshift_r(r[2 * c + 1], r[2 * c + 2], 16) ^ 0x80808080u;
      uint32_t o[4];
      cvt4(a, d0, -128.f * d0, o[0], o[1]);
      cvt4(b, d0, -128.f * d0, o[2], o[3]);
      out[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {   // block 1 quants start at byte 36 = word 9, aligned
      uint32_t o[4];
      cvt4(r[9 + 2 * c] ^ 0x80808080u, d1, -128.f * d1, o[0], o[1]);
      cvt4(r[10 + 2 * c] ^ 0x80808080u, d1, -128.f * d1, o[2], o[3]);
      out[4 + c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
};

template <int BITS>
struct DqAffine {   // groups of 64: packed uint32 little-endian fields, w = scale * q + bias
  static constexpr int RAW_ROW = BITS * 32, RAW_STAGES = BITS == 4 ? 4 : 3, BOXES = BITS / 4;   // 128-byte boxes
  static constexpr bool SWIZZLED = true;
  template <bool SWZ>
  static __device__ __forceinline__ void run(const uint8_t* blk, int srow, const QParams& p, int grow, int kb, int g,
                                             uint4* out) {
    const size_t gi = (size_t)grow * (p.K / 64) + (size_t)kb * 4 + g;
    const float s = __bfloat162float(p.scales[gi]), b = __bfloat162float(p.biases[gi]);
    const int x7 = SWZ ? (srow & 7) : 0;
    const uint32_t s2 = dup_bf16(s), b2 = dup_bf16(b);
    if (BITS == 4) {   // the group is 32 bytes: chunks 2g, 2g + 1 of the 128-byte row
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint4 q = *reinterpret_cast<const uint4*>(blk + (((2 * g + c) ^ x7) << 4));
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // one word = 8 weights: nibble i of the word is weight i
          const uint32_t x = w4[u];   // nibble i is weight i: nib2(x >> 4k) yields weights (k, k + 4)
          const uint32_t p0 = nib2(x, s2, b2), p1 = nib2(x >> 4, s2, b2), p2 = nib2(x >> 8, s2, b2),
                         p3 = nib2(x >> 12, s2, b2);
          out[c * 4 + u] = make_uint4(__byte_perm(p0, p1, 0x5410), __byte_perm(p2, p3, 0x5410),
                                      __byte_perm(p0, p1, 0x7632), __byte_perm(p2, p3, 0x7632));
        }
      }
    } else {           // 64 bytes: groups 0,1 live in the first 128-byte box, 2,3 in the second
      const uint8_t* base = blk + (SWZ ? (g >> 1) * (QBM * 128) : (g >> 1) * 128);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 q = *reinterpret_cast<const uint4*>(base + ((((g & 1) * 4 + c) ^ x7) << 4));
        uint32_t o[8];
        cvt4(q.x, s, b, o[0], o[1]);
        cvt4(q.y, s, b, o[2], o[3]);
        cvt4(q.z, s, b, o[4], o[5]);
        cvt4(q.w, s, b, o[6], o[7]);
        out[c * 2] = make_uint4(o[0], o[1], o[2], o[3]);
        out[c * 2 + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  }
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// NVFP4 (the reference's container: candle-gen/src/quant/nvfp4.rs:90-358): E2M1 codes, two per byte (even column in
// the low nibble), one unsigned E4M3 scale per 16 columns and one fp32 scale per tensor; w = e2m1 * e4m3 * global.
// The scale bytes sit in 128-row x 4-block atoms: atom (row / 128) + m_atoms * (block / 4), byte
// (row % 32) * 16 + (row % 128 / 32) * 4 + block % 4 - so the four scales of a 64-column group are one aligned word.
struct DqNvfp4 {
  static constexpr int RAW_ROW = 128, RAW_STAGES = 4, BOXES = 1;
  static constexpr bool SWIZZLED = true;
  // eight E2M1 codes (nibble i = column i) -> eight bf16 in column order, times the block scale. The magnitude bits
  // index two 8-byte tables (high and low bytes of 0, .5, 1, 1.5, 2, 3, 4, 6 in bf16) through prmt; the sign bits
  // reach bit 7 of each high byte through prmt's sign-replication mode.
  static __device__ __forceinline__ uint4 decode8(uint32_t x, uint32_t s2) {
    const uint32_t HL = 0x3F3F3F00u, HH = 0x40404040u, LL = 0xC0800000u, LH = 0xC0804000u;
    const uint32_t sel = x & 0x77777777u, selb = sel >> 16, xs = x << 4;
    uint32_t hiA = prmt(HL, HH, sel), loA = prmt(LL, LH, sel), hiB = prmt(HL, HH, selb), loB = prmt(LL, LH, selb);
    hiA |= prmt(xs, x, 0xD9C8u) & 0x80808080u;
    hiB |= prmt(xs, x, 0xFBEAu) & 0x80808080u;
    return make_uint4(mul_bf16x2(prmt(loA, hiA, 0x5140u), s2), mul_bf16x2(prmt(loA, hiA, 0x7362u), s2),
                      mul_bf16x2(prmt(loB, hiB, 0x5140u), s2), mul_bf16x2(prmt(loB, hiB, 0x7362u), s2));
  }
  template <bool SWZ>
  static __device__ __forceinline__ void run(const uint8_t* blk, int srow, const QParams& p, int grow, int kb, int g,
                                             uint4* out) {
    const size_t atom = (size_t)(grow >> 7) + (size_t)p.sf_m_atoms * (size_t)(kb * 4 + g);
    const uint32_t sfw = *reinterpret_cast<const uint32_t*>(p.sf + atom * 512 + (grow & 31) * 16 + ((grow & 127) >> 5) * 4);
    const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(sfw & 0xFFFFu), __NV_E4M3);
    const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(sfw >> 16), __NV_E4M3);
    const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
    const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
    const uint32_t s2[4] = {dup_bf16(f01.x * p.gscale), dup_bf16(f01.y * p.gscale), dup_bf16(f23.x * p.gscale),
                            dup_bf16(f23.y * p.gscale)};
    const int x7 = SWZ ? (srow & 7) : 0;
#pragma unroll
    for (int c = 0; c < 2; ++c) {   // the 64-column group is 32 bytes: chunks 2g, 2g + 1 of the 128-byte row
      const uint4 q = *reinterpret_cast<const uint4*>(blk + (((2 * g + c) ^ x7) << 4));
      out[c * 4 + 0] = decode8(q.x, s2[c * 2]);
      out[c * 4 + 1] = decode8(q.y, s2[c * 2]);
      out[c * 4 + 2] = decode8(q.z, s2[c * 2 + 1]);
      out[c * 4 + 3] = decode8(q.w, s2[c * 2 + 1]);
    }
  }
};

template <class DQ, int BLOCK_N>
struct QCfg {
  static constexpr int RS = DQ::RAW_STAGES;
  static constexpr int STAGES = (BLOCK_N == 64 && RS == 3) ? 2 : 3;
  static constexpr uint32_t RAW_BYTES = DQ::RAW_ROW * QBM;
  static constexpr uint32_t B_BYTES = BLOCK_N * QSK * 2;
  static constexpr uint32_t STAGE_BYTES = QA_BYTES + B_BYTES;
  static constexpr uint32_t OFF_RAW = STAGES * STAGE_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_RAW + RS * RAW_BYTES;
  static constexpr uint32_t TMEM_COLS = BLOCK_N < 32 ? 32 : BLOCK_N;
  static constexpr size_t SMEM_BYTES = (size_t)OFF_BAR + 256 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static_assert(STAGE_BYTES % 1024 == 0 && RAW_BYTES % 1024 == 0, "stage alignment");
};

template <class DQ, int BLOCK_N>
__global__ void __launch_bounds__(QTHREADS, 1)
gemm_quant_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_w,
                  const QParams p) {
  using Cfg = QCfg<DQ, BLOCK_N>;
  constexpr int STAGES = Cfg::STAGES, RS = Cfg::RS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full_a = bars;                      // [STAGES] 256 arrivals (dequantisation threads)
  uint64_t* full_b = bars + STAGES;             // [STAGES] TMA bytes
  uint64_t* empty = bars + 2 * STAGES;          // [STAGES] MMA commit
  uint64_t* raw_full = bars + 3 * STAGES;       // [RS] TMA bytes
  uint64_t* raw_empty = bars + 3 * STAGES + RS; // [RS] 512 arrivals
  uint64_t* acc_full = bars + 3 * STAGES + 2 * RS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.kblocks, kb0 + p.kb_per_split);
  const int n_sub = (kb1 - kb0) * 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_a[s], 256);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < RS; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 512);
    }
    mbar_init(acc_full, 1);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_act);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------------------------------------------------------- raw weight blocks (static: no dependency wait)
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_first();
      int issued = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        const int it = kb - kb0, s = it % RS;
        ok = mbar_wait(&raw_empty[s], ((it / RS) & 1) ^ 1, s_abort, 10);
        if (!ok) break;
        mbar_arrive_expect_tx(&raw_full[s], Cfg::RAW_BYTES);
        uint8_t* dst = smem + Cfg::OFF_RAW + s * Cfg::RAW_BYTES;
#pragma unroll
        for (int b = 0; b < DQ::BOXES; ++b)
          tma_load_2d_hint(dst + b * (Cfg::RAW_BYTES / DQ::BOXES), &tmap_w, &raw_full[s],
                           (kb * DQ::BOXES + b) * (DQ::RAW_ROW / DQ::BOXES / 2), tile * QBM, pol);
        issued = it + 1;
      }
      if (!ok) {
        volatile int never = 0;
        for (int it = max(0, issued - RS); it < issued; ++it) mbar_wait(&raw_full[it % RS], (it / RS) & 1, &never, 11);
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- activations
    if (lane == 0) {
      pdl_wait();
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < n_sub && ok; ++it) {
        const int s = it % STAGES;
        ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, s_abort, 12);
        if (!ok) break;
        mbar_arrive_expect_tx(&full_b[s], Cfg::B_BYTES);
        uint8_t* dst = smem + s * Cfg::STAGE_BYTES + QA_BYTES;
#pragma unroll
        for (int a = 0; a < 2; ++a)
          tma_load_2d(dst + a * (BLOCK_N * 128), &tmap_act, &full_b[s], kb0 * QBK + it * QSK + a * 64, 0);
        issued = it + 1;
      }
      if (!ok) {
        volatile int never = 0;
        for (int it = max(0, issued - STAGES); it < issued; ++it)
          mbar_wait(&full_b[it % STAGES], (it / STAGES) & 1, &never, 13);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(QBM, BLOCK_N);
      bool ok = true;
      for (int it = 0; it < n_sub && ok; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        ok = mbar_wait(&full_a[s], ph, s_abort, 20) && mbar_wait(&full_b[s], ph, s_abort, 21);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint32_t sb = sa + QA_BYTES;
#pragma unroll
        for (int k = 0; k < QSK / 16; ++k) {
          const uint64_t adesc = umma_desc_kmajor_sw128(sa + (k >> 2) * QATOM + (k & 3) * 32);
          const uint64_t bdesc = umma_desc_kmajor_sw128(sb + (k >> 2) * (BLOCK_N * 128) + (k & 3) * 32);
          umma_f16_ss(tmem, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
      }
      umma_commit(acc_full);
      if (!ok) {
        volatile int never = 0;
        mbar_wait(acc_full, 0, &never, 22);
      }
    }
  } else {
    // ------------------------------------------------- dequantise: thread = (K half of the raw block, atom, row)
    const int d = threadIdx.x - 96;            // 0..511
    const int row_in_tile = d & 127, q = (d >> 7) & 1, sub = d >> 8;
    const int grow = min(tile * QBM + row_in_tile, p.N - 1);
    bool ok = true;
    for (int kb = kb0; kb < kb1 && ok; ++kb) {
      const int itr = kb - kb0, rs = itr % RS;
      ok = mbar_wait(&raw_full[rs], (itr / RS) & 1, s_abort, 30);
      if (!ok) break;
      const uint8_t* rawblk = smem + Cfg::OFF_RAW + rs * Cfg::RAW_BYTES +
                              (DQ::SWIZZLED ? row_in_tile * 128 : row_in_tile * DQ::RAW_ROW);
      const int it = itr * 2 + sub, s = it % STAGES;
      uint4 chunk[8];
      DQ::template run<DQ::SWIZZLED>(rawblk, row_in_tile, p, grow, kb, sub * 2 + q, chunk);
      ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, s_abort, 31);
      if (!ok) break;
      uint8_t* a = smem + s * Cfg::STAGE_BYTES + q * QATOM + row_in_tile * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(a + ((j ^ (row_in_tile & 7)) << 4)) = chunk[j];
      fence_proxy_async_smem();                // generic-proxy stores -> visible to the tensor core's async proxy
      mbar_arrive(&full_a[s]);
      mbar_arrive(&raw_empty[rs]);
    }
    // ---------------------------------------------------------------- epilogue: warps 3..6 own TMEM lanes (warp & 3)
    if (warp < 7) {
      const int quarter = warp & 3;
      const int r_in_tile = quarter * 32 + lane;
      const int frow = tile * QBM + r_in_tile;
      if (ok) ok = mbar_wait(acc_full, 0, s_abort, 32);
      tc_fence_after_sync();
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16);
      if (p.splits == 1) {
        if (ok) {
          const float b = (p.bias && frow < p.N) ? __bfloat162float(p.bias[frow]) : 0.f;
#pragma unroll 1
          for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
            float v[16];
            tmem_ld_32x32b_x16(taddr + ch * 16, v);
            if (frow < p.N)
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int tok = ch * 16 + j;
                if (tok < p.T) p.out[(size_t)tok * p.ldd + frow] = __float2bfloat16(v[j] + b);
              }
          }
        }
      } else {
        // both named barriers are reached by all 128 epilogue threads whatever `ok` says
        if (ok) {
          float* ws = p.workspace + ((size_t)tile * p.splits + split) * (BLOCK_N * QBM);
#pragma unroll 1
          for (int ch = 0; ch < BLOCK_N / 16; ++ch) {
            float v[16];
            tmem_ld_32x32b_x16(taddr + ch * 16, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) __stcg(&ws[(ch * 16 + j) * QBM + r_in_tile], v[j]);
          }
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 3 && lane == 0) {
          int last = 0;
          if (*s_abort == 0) {
            const int old = atomicAdd(&p.counters[tile], 1);
            last = (old == p.splits - 1);
            if (last) p.counters[tile] = 0;
          }
          *s_last = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*s_last && frow < p.N) {
          __threadfence();
          const float b = p.bias ? __bfloat162float(p.bias[frow]) : 0.f;
          const float* base = p.workspace + (size_t)tile * p.splits * (BLOCK_N * QBM);
          for (int t0 = 0; t0 < p.T; t0 += 8) {   // eight independent load chains at a time, splits summed in order
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int sp = 0; sp < p.splits; ++sp) {
              const float* src = base + (size_t)sp * (BLOCK_N * QBM) + t0 * QBM + r_in_tile;
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] += (t0 + j < BLOCK_N) ? __ldcg(src + j * QBM) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (t0 + j < p.T) p.out[(size_t)(t0 + j) * p.ldd + frow] = __float2bfloat16(acc[j] + b);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// Expansion to dense bf16 [N, K] (prefill-sized token counts run the dense GEMM on the expanded weights).
template <class DQ>
__global__ void __launch_bounds__(256) dequant_rows_kernel(const QParams p, bf16* out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)p.N * p.kblocks * 4;
  if (i >= total) return;
  const int g = (int)(i & 3);
  const int kb = (int)((i >> 2) % p.kblocks);
  const int row = (int)((i >> 2) / p.kblocks);
  uint4 chunk[8];
  DQ::template run<false>(p.w + (size_t)row * p.row_bytes + (size_t)kb * DQ::RAW_ROW, 0, p, row, kb, g, chunk);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * p.K + (size_t)kb * QBK + g * 64);
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j] = chunk[j];
}

template <class DQ>
int launch_dequant(const QParams& p, bf16* out, cudaStream_t stream) {
  const long long total = (long long)p.N * p.kblocks * 4;
  return launch_kernel(dequant_rows_kernel<DQ>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, p, out);
}

template <class DQ, int BLOCK_N>
int launch_q(const CUtensorMap& ta, const QParams& p, int tiles, cudaStream_t stream) {
  using Cfg = QCfg<DQ, BLOCK_N>;
  auto kern = gemm_quant_kernel<DQ, BLOCK_N>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  CUtensorMap tw;
  int rc = make_tmap_u16_2d(&tw, p.w, p.row_bytes / 2, p.N, p.row_bytes, DQ::RAW_ROW / DQ::BOXES / 2, QBM,
                            DQ::SWIZZLED ? 1 : 0);
  if (rc) return rc;
  return launch_kernel(kern, dim3(tiles, p.splits), dim3(QTHREADS), Cfg::SMEM_BYTES, stream, ta, tw, p);
}

template <class DQ>
int launch_fmt(int block_n, const CUtensorMap& ta, const QParams& p, int tiles, cudaStream_t stream) {
  return block_n == 16 ? launch_q<DQ, 16>(ta, p, tiles, stream) : launch_q<DQ, 64>(ta, p, tiles, stream);
}

long long row_bytes_for(int fmt, int K) {
  return fmt == 0 ? (long long)K / 256 * 144 : fmt == 1 ? (long long)K / 32 * 34 : (fmt == 2 || fmt == 4) ? K / 2 : K;
}

}  // namespace
}  // namespace swb

extern "C" {

// Packed [N, K] weights (formats as for swb_gemm_quant) -> dense bf16 [N, K].
static int dequant_rows_impl(int fmt, const void* Wq, const void* scales, const void* biases, float gscale, void* out,
                             int N, int K, void* stream) {
  using namespace swb;
  if (N <= 0) return 0;
  if (K <= 0 || K % QBK != 0 || fmt < 0 || fmt > 4) return -3;
  QParams p{};
  p.sf = reinterpret_cast<const uint8_t*>(scales);
  p.sf_m_atoms = (N + 127) / 128;
  p.gscale = gscale;
  p.w = reinterpret_cast<const uint8_t*>(Wq);
  p.scales = reinterpret_cast<const bf16*>(scales);
  p.biases = reinterpret_cast<const bf16*>(biases);
  p.row_bytes = row_bytes_for(fmt, K);
  p.N = N;
  p.K = K;
  p.kblocks = K / QBK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  bf16* o = reinterpret_cast<bf16*>(out);
  switch (fmt) {
    case 0: return launch_dequant<DqQ4K>(p, o, s);
    case 1: return launch_dequant<DqQ80>(p, o, s);
    case 2: return launch_dequant<DqAffine<4>>(p, o, s);
    case 3: return launch_dequant<DqAffine<8>>(p, o, s);
    default: return launch_dequant<DqNvfp4>(p, o, s);
  }
}

int swb_dequant_rows(int fmt, const void* Wq, const void* scales, const void* biases, void* out, int N, int K,
                     void* stream) {
  if (fmt > 3) return -3;
  return dequant_rows_impl(fmt, Wq, scales, biases, 1.f, out, N, K, stream);
}

// NVFP4 weights -> dense bf16 [N, K]. packed: [N, K / 2] bytes; sf: swizzled unsigned E4M3 scales
// (ceil(N / 128) * 128 x ceil(K / 64) * 4 bytes, 16-byte aligned); global_scale: the tensor's fp32 scale.
int swb_dequant_nvfp4(const void* packed, const void* sf, float global_scale, void* out, int N, int K, void* stream) {
  if (!sf || (reinterpret_cast<uintptr_t>(sf) & 3)) return -3;
  return dequant_rows_impl(4, packed, sf, nullptr, global_scale, out, N, K, stream);
}

// fmt: 0 Q4_K, 1 Q8_0, 2 affine 4-bit (group 64), 3 affine 8-bit (group 64). A: bf16 [T <= 64, K] (lda elements);
// Wq: packed [N rows]; scales / biases: bf16 [N, K/64] for fmt 2 / 3 (null otherwise); D: bf16 [T, N] (ldd).
// K must be a multiple of 256. workspace: as for swb_gemm_bf16 (counters zeroed once, then fp32 partial tiles).
static int gemm_quant_impl(int fmt, const void* A, int lda, const void* Wq, const void* scales, const void* biases,
                           float gscale, void* D, int ldd, int T, int N, int K, const void* bias, void* workspace,
                           size_t workspace_bytes, int force_splits, void* stream) {
  using namespace swb;
  if (T <= 0 || N <= 0) return 0;
  if (T > 64 || K <= 0 || K % QBK != 0 || (lda % 8) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(Wq) & 15) || fmt < 0 || fmt > 4)
    return -3;
  if ((fmt == 2 || fmt == 3) && (!scales || !biases)) return -3;
  if (fmt == 4 && (!scales || (reinterpret_cast<uintptr_t>(scales) & 3))) return -3;
  // up to 8 tokens of Q4_K go to the integer matrix-vector kernel (force_splits < 0 keeps the tensor-core path)
  if (fmt == 0 && force_splits >= 0 && gemv_q4k_accepts(T, K, lda, A, Wq)) {
    static const bool off = [] { const char* e = getenv("SWB_Q4K_GEMV"); return e && e[0] == '0'; }();
    if (!off) return gemv_q4k_launch(A, lda, Wq, D, ldd, T, N, K, bias, reinterpret_cast<cudaStream_t>(stream));
  }
  if (force_splits < 0) force_splits = 0;
  QParams p{};
  p.sf = reinterpret_cast<const uint8_t*>(scales);
  p.sf_m_atoms = (N + 127) / 128;
  p.gscale = gscale;
  p.w = reinterpret_cast<const uint8_t*>(Wq);
  p.scales = reinterpret_cast<const bf16*>(scales);
  p.biases = reinterpret_cast<const bf16*>(biases);
  p.row_bytes = row_bytes_for(fmt, K);
  p.N = N;
  p.K = K;
  p.T = T;
  p.kblocks = K / QBK;
  p.out = reinterpret_cast<bf16*>(D);
  p.ldd = ldd;
  p.bias = reinterpret_cast<const bf16*>(bias);
  const int block_n = T <= 16 ? 16 : 64;
  const int tiles = (N + QBM - 1) / QBM;
  const int sms = device_sm_count();
  int splits = force_splits > 0 ? force_splits : std::max(1, sms / tiles);
  splits = std::min(splits, p.kblocks);
  const size_t need = SWB_GEMM_COUNTER_BYTES + (size_t)tiles * splits * block_n * QBM * sizeof(float);
  if (splits > 1 && (!workspace || workspace_bytes < need || tiles > (int)(SWB_GEMM_COUNTER_BYTES / sizeof(int)))) splits = 1;
  p.kb_per_split = (p.kblocks + splits - 1) / splits;
  p.splits = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;   // no empty splits
  p.counters = reinterpret_cast<int*>(workspace);
  p.workspace = workspace ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + SWB_GEMM_COUNTER_BYTES) : nullptr;
  CUtensorMap tm;
  int rc = make_tmap_bf16_2d(&tm, A, T, K, lda, block_n);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (fmt) {
    case 0: return launch_fmt<DqQ4K>(block_n, tm, p, tiles, s);
    case 1: return launch_fmt<DqQ80>(block_n, tm, p, tiles, s);
    case 2: return launch_fmt<DqAffine<4>>(block_n, tm, p, tiles, s);
    case 3: return launch_fmt<DqAffine<8>>(block_n, tm, p, tiles, s);
    default: return launch_fmt<DqNvfp4>(block_n, tm, p, tiles, s);
  }
}

int swb_gemm_quant(int fmt, const void* A, int lda, const void* Wq, const void* scales, const void* biases, void* D,
                   int ldd, int T, int N, int K, const void* bias, void* workspace, size_t workspace_bytes,
                   int force_splits, void* stream) {
  if (fmt > 3) return -3;
  return gemm_quant_impl(fmt, A, lda, Wq, scales, biases, 1.f, D, ldd, T, N, K, bias, workspace, workspace_bytes,
                         force_splits, stream);
}

// D[T <= 64, N] = A[T, K] * dequant(NVFP4 W[N, K])^T + bias: weight-only FP4 with bf16 activations (the reference's
// W4A16 regime, candle-gen/src/quant/nvfp4_linear.rs:80-88). Operands as for swb_dequant_nvfp4.
int swb_gemm_nvfp4(const void* A, int lda, const void* packed, const void* sf, float global_scale, void* D, int ldd,
                   int T, int N, int K, const void* bias, void* workspace, size_t workspace_bytes, int force_splits,
                   void* stream) {
  return gemm_quant_impl(4, A, lda, packed, sf, nullptr, global_scale, D, ldd, T, N, K, bias, workspace,
                         workspace_bytes, force_splits, stream);
}

}  // extern "C"
