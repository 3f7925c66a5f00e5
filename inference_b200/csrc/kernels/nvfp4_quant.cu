// NVFP4 quantiser on the device: fp32 / bf16 rows -> E2M1 codes, swizzled unsigned-E4M3 block scales and one fp32
// tensor scale, bit-identical to the host packer (`ops/nvfp4.py`, which restates candle-gen/src/quant/nvfp4.rs:150-260;
// the reference's device version is candle-gen/src/quant/nvfp4_quant.cu:80-156).
//   pass 1: one thread per 16-column block: block amax, and the tensor amax by atomicMax on the float's bit pattern
//           (non-negative floats order like unsigned integers);
//   pass 2: global = amax / (6 * 448); block scale = RNE-to-E4M3(block amax / (6 * global)); codes = nearest E2M1 of
//           x / (e4m3 * global) with ties to the even code; two codes per byte (even column in the low nibble);
//           scale bytes into the 128-row x 4-block atoms that block-scaled tensor-core instructions read.
#include "common.cuh"

#include <cuda_fp8.h>

#include <algorithm>

namespace swb {
namespace {

template <bool FP32>
__device__ __forceinline__ float load_elem(const void* x, size_t i) {
  if constexpr (FP32) return reinterpret_cast<const float*>(x)[i];
  return __bfloat162float(reinterpret_cast<const bf16*>(x)[i]);
}

// 16 consecutive elements of a block as floats; 16-byte vector loads when the block's address allows them
template <bool FP32>
__device__ __forceinline__ void load_block16(const void* x, size_t i0, float* v) {
  if constexpr (FP32) {
    const float* p = reinterpret_cast<const float*>(x) + i0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 f = reinterpret_cast<const float4*>(p)[c];
        v[4 * c] = f.x, v[4 * c + 1] = f.y, v[4 * c + 2] = f.z, v[4 * c + 3] = f.w;
      }
      return;
    }
  } else {
    const bf16* p = reinterpret_cast<const bf16*>(x) + i0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint4 u = reinterpret_cast<const uint4*>(p)[c];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[8 * c + 2 * e] = __uint_as_float(w[e] << 16);
          v[8 * c + 2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
        }
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = load_elem<FP32>(x, i0 + j);
}

template <bool FP32>
__global__ void __launch_bounds__(256) nvfp4_block_amax_kernel(const void* x, long long ld, int rows, int nb,
                                                              float* block_amax, unsigned int* tensor_amax_bits) {
  pdl_launch_dependents();
  pdl_wait();
  // grid-stride over 16-element blocks; one atomic per thread block on the tensor maximum
  __shared__ float red[8];
  const long long total = (long long)rows * nb;
  float a = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / nb), b = (int)(i % nb);
    float v[16];
    load_block16<FP32>(x, (size_t)r * ld + b * 16, v);
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(v[j]));
    if (block_amax) block_amax[i] = m;
    a = fmaxf(a, m);
  }
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x < 32) {
    a = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    for (int o = 4; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if (threadIdx.x == 0 && a > 0.f) atomicMax(tensor_amax_bits, __float_as_uint(a));
  }
}

__device__ __forceinline__ float e4m3_to_f32(unsigned char b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ unsigned e2m1_code(float q) {
  if (q != q) return 0u;
  const float m = fminf(fabsf(q), 6.f);
  const unsigned idx = (m > 0.25f) + (m >= 0.75f) + (m > 1.25f) + (m >= 1.75f) + (m > 2.5f) + (m >= 3.5f) + (m > 5.0f);
  return ((__float_as_uint(q) >> 31) << 3) | idx;
}

// FAST: codes by comparing |v| against the seven rounding boundaries scaled by the block's element scale (seven
// multiplies per block) instead of one IEEE division per element. A value within one rounding error of a boundary may
// land on the neighbouring code; the exact form reproduces the host packer bit for bit and is what weights use.
template <bool FP32, bool FAST>
__global__ void __launch_bounds__(256) nvfp4_pack_kernel(const void* x, long long ld, int rows, int nb,
                                                        const float* block_amax, const unsigned int* tensor_amax_bits,
                                                        unsigned char* packed, unsigned char* scales, int sf_rows,
                                                        float* global_scale_out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const float amax = __uint_as_float(*tensor_amax_bits);
  const float gs = amax > 0.f ? __fdiv_rn(amax, 2688.f) : 1.f;      // 6 * 448
  if (i == 0) *global_scale_out = gs;
  if (i >= (long long)rows * nb) return;
  const int r = (int)(i / nb), b = (int)(i % nb);
  float vals[16];
  load_block16<FP32>(x, (size_t)r * ld + b * 16, vals);
  float bmax = 0.f;
  if (block_amax) {
    bmax = block_amax[i];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) bmax = fmaxf(bmax, fabsf(vals[j]));
  }
  const float sf_real = __fdiv_rn(bmax, __fmul_rn(6.f, gs));
  const unsigned char sfb = sf_real > 0.f ? (unsigned char)__nv_cvt_float_to_fp8(sf_real, __NV_SATFINITE, __NV_E4M3) : 0;
  const int m_atoms = sf_rows >> 7;
  scales[((size_t)(r >> 7) + (size_t)m_atoms * (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)] = sfb;
  const float es = __fmul_rn(e4m3_to_f32(sfb), gs);
  unsigned long long bits = 0ull;
  if constexpr (FAST) {
    const float t0 = 0.25f * es, t1 = 0.75f * es, t2 = 1.25f * es, t3 = 1.75f * es, t4 = 2.5f * es, t5 = 3.5f * es, t6 = 5.0f * es;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float v = vals[j], m = fabsf(v);
      unsigned code = 0u;
      if (es > 0.f && v == v)
        code = ((__float_as_uint(v) >> 31) << 3) |
               ((m > t0) + (m >= t1) + (m > t2) + (m >= t3) + (m > t4) + (m >= t5) + (m > t6));
      bits |= (unsigned long long)code << (4 * j);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float v = vals[j];
      const unsigned code = es > 0.f ? e2m1_code(__fdiv_rn(v, es)) : 0u;
      bits |= (unsigned long long)code << (4 * j);
    }
  }
  *reinterpret_cast<unsigned long long*>(packed + ((size_t)r * nb + b) * 8) = bits;
}

}  // namespace
}  // namespace swb

extern "C" {

// x: [rows, cols] fp32 (is_fp32) or bf16, row stride ld elements, cols % 16 == 0. packed: [rows, cols / 2] bytes
// (8-byte aligned); scales: sf_rows * sf_cols bytes, zero-filled by the caller, sf_rows = ceil(rows / 128) * 128,
// sf_cols = ceil(cols / 64) * 4; block_amax: rows * cols / 16 floats of scratch, or null
// (each block's maximum is then recomputed by the packing kernel instead of being stored and re-read); tensor_amax_bits: one zeroed word;
// global_scale_out: one float on the device.
static int nvfp4_quantize_impl(const void* x, int is_fp32, long long ld, int rows, int cols, void* packed, void* scales,
                               int sf_rows, void* block_amax, void* tensor_amax_bits, void* global_scale_out, int fast,
                               void* stream) {
  using namespace swb;
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 16 != 0 || sf_rows % 128 != 0 || sf_rows < rows || (reinterpret_cast<uintptr_t>(packed) & 7)) return -3;
  const int nb = cols / 16;
  const long long n = (long long)rows * nb;
  const dim3 grid((unsigned)((n + 255) / 256)), block(256);
  const dim3 grid_amax((unsigned)std::min<long long>((n + 255) / 256, 148 * 16));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* ba = reinterpret_cast<float*>(block_amax);
  unsigned int* ta = reinterpret_cast<unsigned int*>(tensor_amax_bits);
  int rc;
  if (is_fp32) {
    rc = launch_kernel(nvfp4_block_amax_kernel<true>, grid_amax, block, 0, s, x, ld, rows, nb, ba, ta);
    if (rc) return rc;
    auto k = fast ? nvfp4_pack_kernel<true, true> : nvfp4_pack_kernel<true, false>;
    return launch_kernel(k, grid, block, 0, s, x, ld, rows, nb, (const float*)ba,
                         (const unsigned int*)ta, reinterpret_cast<unsigned char*>(packed),
                         reinterpret_cast<unsigned char*>(scales), sf_rows, reinterpret_cast<float*>(global_scale_out));
  }
  rc = launch_kernel(nvfp4_block_amax_kernel<false>, grid_amax, block, 0, s, x, ld, rows, nb, ba, ta);
  if (rc) return rc;
  auto k = fast ? nvfp4_pack_kernel<false, true> : nvfp4_pack_kernel<false, false>;
  return launch_kernel(k, grid, block, 0, s, x, ld, rows, nb, (const float*)ba,
                       (const unsigned int*)ta, reinterpret_cast<unsigned char*>(packed),
                       reinterpret_cast<unsigned char*>(scales), sf_rows, reinterpret_cast<float*>(global_scale_out));
}


int swb_nvfp4_quantize(const void* x, int is_fp32, long long ld, int rows, int cols, void* packed, void* scales,
                       int sf_rows, void* block_amax, void* tensor_amax_bits, void* global_scale_out, void* stream) {
  return nvfp4_quantize_impl(x, is_fp32, ld, rows, cols, packed, scales, sf_rows, block_amax, tensor_amax_bits,
                             global_scale_out, 0, stream);
}

// The activation-side variant: same outputs, codes chosen by boundary comparison (see nvfp4_pack_kernel).
int swb_nvfp4_quantize_fast(const void* x, int is_fp32, long long ld, int rows, int cols, void* packed, void* scales,
                            int sf_rows, void* tensor_amax_bits, void* global_scale_out, void* stream) {
  return nvfp4_quantize_impl(x, is_fp32, ld, rows, cols, packed, scales, sf_rows, nullptr, tensor_amax_bits,
                             global_scale_out, 1, stream);
}

}  // extern "C"
