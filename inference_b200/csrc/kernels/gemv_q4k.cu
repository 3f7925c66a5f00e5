// Q4_K matrix-vector kernel for 1..8 tokens: D[T, N] = A[T, K] * dequant(Wq)[N, K]^T (+ bias).
//
// At this size the packed weights are the only stream that matters (4.5 bits per weight) and the arithmetic must not
// cost more than their arrival. The weights are therefore never expanded: the activations are quantised to int8 per
// 32-element block inside the kernel (each CTA does all of them: K * T elements, a few microseconds at most, after
// the first weight loads have been issued), stored in shared memory in the order in which a super-block's nibbles lie,
// and the dot products run on packed-byte integer multiply-adds (dp4a), eight weights per instruction pair. This is the
// numerical scheme of the llama.cpp-derived kernels the reference uses (candle-kernels/src/mmvq_gguf.cu: q8_1
// activations against Q4_K weights), laid out for this machine: one persistent 512-thread CTA per SM, one output row
// per warp at a time, every lane owning one 16-byte piece of four consecutive super-blocks, the loads of the next
// 16-super-block slice in flight while the current one is consumed.
//
// Super-block (144 bytes, 256 weights): fp16 d, fp16 dmin, 12 bytes of 6-bit scales / mins for 8 sub-blocks of 32,
// 128 bytes of nibbles in four 32-byte chunks; in chunk j the low nibbles are weights 64j .. 64j+31 (sub-block 2j) and
// the high nibbles weights 64j+32 .. 64j+63 (sub-block 2j+1). w = d * sc * q - dmin * m.
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>

namespace swb {

int device_sm_count();   // gemm_tcgen05.cu

SWB_REGISTER_STATUS_UNIT(gemv_q4k);

namespace {

constexpr int GV_THREADS = 512;
constexpr int GV_WARPS = GV_THREADS / 32;
constexpr int GV_STEPS = 4;   // warp-steps (of 4 super-blocks) loaded before any is consumed

struct GvParams {
  const uint8_t* w;
  const bf16* a;
  bf16* out;
  const bf16* bias;
  long long row_bytes;
  int lda, ldd, N, K, kblocks;
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t u, int s, int acc) {   // unsigned bytes of u times signed bytes of s
  int r;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(u), "r"(s), "r"(acc));
  return r;
}

// Shared memory, per token t (strides in the comments are per token):
//   q_lo / q_hi  [K / 2] int8   quantised activations that meet low / high nibbles: super-block sb, piece i -> sb * 128 + i * 16
//   d_lo / d_hi  [K / 64] float block scale of the 32 activations of sub-block 2j / 2j + 1: sb * 4 + j
//   s_lo / s_hi  [K / 32] float scale * sum of the 16 quantised activations of piece i: sb * 8 + i
template <int T>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_q4k_kernel(const GvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = p.K, kb = p.kblocks;
  int8_t* q_lo = reinterpret_cast<int8_t*>(smem);
  int8_t* q_hi = q_lo + (size_t)T * (K / 2);
  float* d_lo = reinterpret_cast<float*>(q_hi + (size_t)T * (K / 2));
  float* d_hi = d_lo + T * (K / 64);
  float* s_lo = d_hi + T * (K / 64);
  float* s_hi = s_lo + T * (K / 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, piece = lane & 7;          // super-block within the warp-step, 16-byte piece within it
  const int total_warps = gridDim.x * GV_WARPS;
  int row = blockIdx.x * GV_WARPS + warp;

  // Work items are (row, slice of 16 super-blocks); two register buffers alternate so that the next item's bytes are
  // in flight while the current one is consumed. The first item starts moving before the activations exist.
  const int spr = (kb + GV_STEPS * 4 - 1) / (GV_STEPS * 4);
  uint4 hdrA[GV_STEPS], qsA[GV_STEPS], hdrB[GV_STEPS], qsB[GV_STEPS];
  auto issue = [&](uint4* hdr, uint4* qs, int r, int sl) {
    const uint8_t* rp = p.w + (size_t)r * p.row_bytes;
#pragma unroll
    for (int s = 0; s < GV_STEPS; ++s) {
      const int b = sl * (GV_STEPS * 4) + s * 4 + sub;
      if (b < kb) {
        const uint8_t* blk = rp + (size_t)b * 144;
        hdr[s] = ld_stream(blk);
        qs[s] = ld_stream(blk + 16 + piece * 16);
      }
    }
  };
  if (row < p.N) issue(hdrA, qsA, row, 0);

  pdl_wait(TL_GEMM_QUANT);
  // ---- quantise the activations: one thread per (token, 32-element block) ----
  const int nblk = K / 32;
  for (int idx = threadIdx.x; idx < T * nblk; idx += GV_THREADS) {
    const int t = idx / nblk, b = idx - t * nblk;
    const uint4* src = reinterpret_cast<const uint4*>(p.a + (size_t)t * p.lda + b * 32);
    float v[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 x = src[c];
      const uint32_t wds[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[c * 8 + e * 2] = __uint_as_float(wds[e] << 16);
        v[c * 8 + e * 2 + 1] = __uint_as_float(wds[e] & 0xFFFF0000u);
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(v[e]));
    const float d = amax * (1.f / 127.f), inv = amax > 0.f ? 127.f / amax : 0.f;
    // block b = sb * 8 + 2j + h: h = 0 meets low nibbles, h = 1 high nibbles of chunk j
    const int sb = b >> 3, j = (b >> 1) & 3, h = b & 1;
    int8_t* qd = (h ? q_hi : q_lo) + (size_t)t * (K / 2) + sb * 128 + j * 32;
    uint32_t packed[8];
    int sums[2] = {0, 0};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t wd = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int q = __float2int_rn(v[c * 4 + e] * inv);
        sums[c >> 2] += q;
        wd |= (uint32_t)(q & 0xFF) << (8 * e);
      }
      packed[c] = wd;
    }
    reinterpret_cast<uint4*>(qd)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    reinterpret_cast<uint4*>(qd)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    (h ? d_hi : d_lo)[t * (K / 64) + sb * 4 + j] = d;
    float* sd = (h ? s_hi : s_lo) + t * (K / 32) + sb * 8 + j * 2;
    sd[0] = d * (float)sums[0];
    sd[1] = d * (float)sums[1];
  }
  __syncthreads();
  pdl_launch_dependents();

  const int j = piece >> 1;   // chunk of this lane's piece: sub-blocks 2j (low nibbles) and 2j + 1 (high)
  float acc[T];
  auto consume = [&](const uint4* hdr, const uint4* qs, int r, int sl) {
    if (sl == 0) {
#pragma unroll
      for (int t = 0; t < T; ++t) acc[t] = 0.f;
    }
#pragma unroll
    for (int s = 0; s < GV_STEPS; ++s) {
      const int b = sl * (GV_STEPS * 4) + s * 4 + sub;
      if (b < kb) {
        const uint4 h4 = hdr[s], q = qs[s];
        const __half2 dd = *reinterpret_cast<const __half2*>(&h4.x);
        const float d = __low2float(dd), dmin = __high2float(dd);
        auto sbyte = [&](int i) -> uint32_t {
          const uint32_t wv = i < 4 ? h4.y : (i < 8 ? h4.z : h4.w);
          return (wv >> ((i & 3) * 8)) & 0xFFu;
        };
        float sc[2], mn[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int k = j * 2 + e;
          uint32_t scv, mv;
          if (j < 2) {
            scv = sbyte(k) & 63u;
            mv = sbyte(k + 4) & 63u;
          } else {
            scv = (sbyte(k + 4) & 0xFu) | ((sbyte(k - 4) >> 6) << 4);
            mv = (sbyte(k + 4) >> 4) | ((sbyte(k) >> 6) << 4);
          }
          sc[e] = d * (float)scv;
          mn[e] = dmin * (float)mv;
        }
        const uint32_t wq[4] = {q.x, q.y, q.z, q.w};
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          lo[c] = wq[c] & 0x0F0F0F0Fu;
          hi[c] = (wq[c] >> 4) & 0x0F0F0F0Fu;
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const int4 a0 = *reinterpret_cast<const int4*>(q_lo + (size_t)t * (K / 2) + b * 128 + piece * 16);
          const int4 a1 = *reinterpret_cast<const int4*>(q_hi + (size_t)t * (K / 2) + b * 128 + piece * 16);
          const int s0 = dp4a_us(lo[3], a0.w, dp4a_us(lo[2], a0.z, dp4a_us(lo[1], a0.y, dp4a_us(lo[0], a0.x, 0))));
          const int s1 = dp4a_us(hi[3], a1.w, dp4a_us(hi[2], a1.z, dp4a_us(hi[1], a1.y, dp4a_us(hi[0], a1.x, 0))));
          const float da0 = d_lo[t * (K / 64) + b * 4 + j], da1 = d_hi[t * (K / 64) + b * 4 + j];
          const float as0 = s_lo[t * (K / 32) + b * 8 + piece], as1 = s_hi[t * (K / 32) + b * 8 + piece];
          acc[t] = fmaf(sc[0] * da0, (float)s0, acc[t]);
          acc[t] = fmaf(sc[1] * da1, (float)s1, acc[t]);
          acc[t] = fmaf(-mn[0], as0, acc[t]);
          acc[t] = fmaf(-mn[1], as1, acc[t]);
        }
      }
    }
    if (sl == spr - 1) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        float v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (lane == t) {
          if (p.bias) v += __bfloat162float(p.bias[r]);
          p.out[(size_t)t * p.ldd + r] = __float2bfloat16(v);
        }
      }
    }
  };
  auto advance = [&](int& r, int& sl) {
    if (++sl == spr) {
      sl = 0;
      r += total_warps;
    }
  };
  int sl = 0;
  while (row < p.N) {
    int rn = row, sn = sl;
    advance(rn, sn);
    if (rn < p.N) issue(hdrB, qsB, rn, sn);
    consume(hdrA, qsA, row, sl);
    row = rn;
    sl = sn;
    if (row >= p.N) break;
    advance(rn, sn);
    if (rn < p.N) issue(hdrA, qsA, rn, sn);
    consume(hdrB, qsB, row, sl);
    row = rn;
    sl = sn;
  }
}

template <int T>
int launch_gv(const GvParams& p, cudaStream_t stream) {
  const size_t smem = (size_t)T * ((size_t)p.K + (size_t)(p.K / 64) * 8 + (size_t)(p.K / 32) * 8);
  auto kern = gemv_q4k_kernel<T>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  if (smem > 200 * 1024) return -3;
  const int ctas = std::min(device_sm_count(), (p.N + GV_WARPS - 1) / GV_WARPS);
  return launch_kernel(kern, dim3(ctas), dim3(GV_THREADS), smem, stream, p);
}

}  // namespace

// Whether the matrix-vector kernel takes this problem: T in 1..8, K a multiple of 256 whose activations fit in shared
// memory, 16-byte aligned operands.
bool gemv_q4k_accepts(int T, int K, int lda, const void* A, const void* Wq) {
  if (T < 1 || T > 8 || K <= 0 || K % 256 != 0 || lda % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(Wq) & 15)) return false;
  return (size_t)T * ((size_t)K + (size_t)(K / 64) * 8 + (size_t)(K / 32) * 8) <= 200 * 1024;
}

int gemv_q4k_launch(const void* A, int lda, const void* Wq, void* D, int ldd, int T, int N, int K, const void* bias,
                    cudaStream_t stream) {
  GvParams p{};
  p.w = reinterpret_cast<const uint8_t*>(Wq);
  p.a = reinterpret_cast<const bf16*>(A);
  p.out = reinterpret_cast<bf16*>(D);
  p.bias = reinterpret_cast<const bf16*>(bias);
  p.row_bytes = (long long)K / 256 * 144;
  p.lda = lda;
  p.ldd = ldd;
  p.N = N;
  p.K = K;
  p.kblocks = K / 256;
  cudaStream_t st = stream;
  switch (T) {
    case 1: return launch_gv<1>(p, st);
    case 2: return launch_gv<2>(p, st);
    case 3: return launch_gv<3>(p, st);
    case 4: return launch_gv<4>(p, st);
    case 5: return launch_gv<5>(p, st);
    case 6: return launch_gv<6>(p, st);
    case 7: return launch_gv<7>(p, st);
    case 8: return launch_gv<8>(p, st);
    default: return -3;
  }
}

}  // namespace swb
