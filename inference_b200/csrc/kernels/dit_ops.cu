// Bandwidth-bound media kernels for sm_100a: sampler axpy (the Euler flow-matching update x + dt * v and every
// other a*x + b*y of the sampler framework), GroupNorm(+SiLU) over NHWC activations, nearest 2x upsampling, row
// softmax and the final RGB8 quantisation. They replace chains of elementwise launches in the reference:
// candle-gen/src/sampler.rs:36-59 (scale / add / axpy), candle-gen-flux/src/vae/native.rs:163-222 (GroupNorm ->
// SiLU, nearest upsample) and candle-gen/src/lib.rs:56-62 (round_rgb8, nearest-even).
#include <algorithm>
#include "common.cuh"

namespace swb {
namespace {

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// out = a * x + b * y over n (multiple of 8) bf16 elements.
__global__ void __launch_bounds__(256) axpy_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                                       bf16* out, long long n8, float a, float b) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float fx[8], fy[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(x)[i], fx);
  unpack8(reinterpret_cast<const uint4*>(y)[i], fy);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = a * fx[j] + b * fy[j];
  reinterpret_cast<uint4*>(out)[i] = pack8(o);
}

__global__ void __launch_bounds__(256) axpy_f32_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                      float* out, long long n, float a, float b) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a * x[i] + b * y[i];
}

// GroupNorm statistics over NHWC bf16: one CTA per (sample, group, chunk of pixels); partial sum / sum of squares are
// accumulated with atomics into stats[n][g][2] (zeroed by the caller).
__global__ void __launch_bounds__(256) groupnorm_stats_kernel(const bf16* __restrict__ x, float* stats, int HW, int C,
                                                             int G, int chunk) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[2][8];
  const int n = blockIdx.z, g = blockIdx.y;
  const int cpg = C / G;
  const int p0 = blockIdx.x * chunk;
  const int p1 = min(HW, p0 + chunk);
  float s = 0.f, ss = 0.f;
  const int per_pixel = cpg / 8;  // uint4 loads per pixel (cpg multiple of 8)
  const long long total = (long long)(p1 - p0) * per_pixel;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const int p = p0 + (int)(i / per_pixel);
    const int v = (int)(i % per_pixel);
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + ((size_t)n * HW + p) * C + g * cpg + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s += f[j];
      ss += f[j] * f[j];
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red[0][warp] = s;
    red[1][warp] = ss;
  }
  __syncthreads();
  if (warp == 0) {
    s = lane < 8 ? red[0][lane] : 0.f;
    ss = lane < 8 ? red[1][lane] : 0.f;
    s = warp_sum(s);
    ss = warp_sum(ss);
    if (lane == 0) {
      atomicAdd(&stats[((size_t)n * G + g) * 2], s);
      atomicAdd(&stats[((size_t)n * G + g) * 2 + 1], ss);
    }
  }
}

// Row-coalesced statistics: one CTA covers `chunk` pixels of one sample over all channels; thread t owns vector column
// t % (C/8) and walks pixels with stride 256 / (C/8), so a warp reads whole contiguous pixel rows. Groups may be narrower
// than a 16-byte vector (C / G in {1, 2, 4}: the vector spans several groups) or a multiple of it (the vector's eight
// channels fall in one group). Requires C/8 to divide 256 and G <= 512.
__global__ void __launch_bounds__(256) groupnorm_stats_narrow_kernel(const bf16* __restrict__ x, float* stats, int HW,
                                                                    int C, int G, int chunk) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float acc[2 * 512];
  for (int i = threadIdx.x; i < 2 * G; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int n = blockIdx.y;
  const int c8 = C / 8, cpg = C / G;
  const int v = threadIdx.x % c8, lane_p = threadIdx.x / c8, stride_p = 256 / c8;
  const int p0 = blockIdx.x * chunk, p1 = min(HW, p0 + chunk);
  float s[8], ss[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = ss[j] = 0.f;
  for (int p = p0 + lane_p; p < p1; p += stride_p) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + ((size_t)n * HW + p) * C + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j] += f[j];
      ss[j] += f[j] * f[j];
    }
  }
  if (cpg >= 8) {
    float st = 0.f, sst = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      st += s[j];
      sst += ss[j];
    }
    const int g = (v * 8) / cpg;
    atomicAdd(&acc[2 * g], st);
    atomicAdd(&acc[2 * g + 1], sst);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int g = (v * 8 + j) / cpg;
      atomicAdd(&acc[2 * g], s[j]);
      atomicAdd(&acc[2 * g + 1], ss[j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * G; i += blockDim.x) atomicAdd(&stats[(size_t)n * G * 2 + i], acc[i]);
}

// y = silu?((x - mean) * rstd * gamma + beta), NHWC bf16. A thread owns one 8-channel vector column (C / 8 divides the
// CTA's 256 threads) and walks pixels with a grid stride, so the per-channel scale and shift (folded from the group
// statistics and gamma / beta) are computed once per sample instead of once per element, and the index arithmetic is
// 32-bit. Launch with a grid whose thread count is a multiple of C / 8.
__global__ void __launch_bounds__(256) groupnorm_apply_kernel(const bf16* __restrict__ x, const float* __restrict__ stats,
                                                             const bf16* __restrict__ gamma,
                                                             const bf16* __restrict__ beta, bf16* out, int N, int HW,
                                                             int C, int G, float eps, int silu) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned c8 = C / 8, cpg = C / G;
  const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x, threads = gridDim.x * blockDim.x;
  const unsigned v = tid % c8, c = v * 8;
  const unsigned pix_step = threads / c8;
  const float cnt = (float)HW * cpg;
  float ga[8], be[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(gamma + c)), ga);
  unpack8(__ldg(reinterpret_cast<const uint4*>(beta + c)), be);
  for (int n = 0; n < N; ++n) {
    float sc[8], sh[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned g = (c + j) / cpg;
      const float mean = stats[((size_t)n * G + g) * 2] / cnt;
      const float var = fmaxf(stats[((size_t)n * G + g) * 2 + 1] / cnt - mean * mean, 0.f);
      const float rstd = rsqrtf(var + eps);
      sc[j] = rstd * ga[j];
      sh[j] = be[j] - mean * sc[j];
    }
    const uint4* xin = reinterpret_cast<const uint4*>(x) + (size_t)n * HW * c8 + v;
    uint4* yout = reinterpret_cast<uint4*>(out) + (size_t)n * HW * c8 + v;
    for (unsigned p = tid / c8; p < (unsigned)HW; p += pix_step) {
      float f[8], o[8];
      unpack8(xin[(size_t)p * c8], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float t = fmaf(f[j], sc[j], sh[j]);
        o[j] = silu ? silu_f(t) : t;
      }
      yout[(size_t)p * c8] = pack8(o);
    }
  }
}

// Fallback for channel counts whose vector columns do not divide the CTA: one 8-channel vector per thread.
__global__ void __launch_bounds__(256) groupnorm_apply_any_kernel(const bf16* __restrict__ x, const float* __restrict__ stats,
                                                                 const bf16* __restrict__ gamma,
                                                                 const bf16* __restrict__ beta, bf16* out, long long n8,
                                                                 int HW, int C, int G, float eps, int silu) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const int c8 = C / 8;
  const int c = (int)(i % c8) * 8;
  const long long pix = i / c8;
  const int n = (int)(pix / HW);
  const int cpg = C / G;
  const float cnt = (float)HW * cpg;
  float f[8], ga[8], be[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(x)[i], f);
  unpack8(__ldg(reinterpret_cast<const uint4*>(gamma + c)), ga);
  unpack8(__ldg(reinterpret_cast<const uint4*>(beta + c)), be);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = (c + j) / cpg;
    const float mean = stats[((size_t)n * G + g) * 2] / cnt;
    const float var = fmaxf(stats[((size_t)n * G + g) * 2 + 1] / cnt - mean * mean, 0.f);
    const float t = (f[j] - mean) * rsqrtf(var + eps) * ga[j] + be[j];
    o[j] = silu ? silu_f(t) : t;
  }
  reinterpret_cast<uint4*>(out)[i] = pack8(o);
}

// Nearest-neighbour 2x upsampling, NHWC bf16: out[n, 2h+a, 2w+b, :] = x[n, h, w, :].
__global__ void __launch_bounds__(256) upsample2x_kernel(const bf16* __restrict__ x, bf16* out, int N, int H, int W,
                                                        int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int c8 = C / 8;
  const long long total = (long long)N * (2 * H) * (2 * W) * c8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int v = (int)(i % c8);
  long long p = i / c8;
  const int ow = (int)(p % (2 * W));
  p /= (2 * W);
  const int oh = (int)(p % (2 * H));
  const int n = (int)(p / (2 * H));
  reinterpret_cast<uint4*>(out)[i] =
      reinterpret_cast<const uint4*>(x)[(((size_t)n * H + oh / 2) * W + ow / 2) * c8 + v];
}

// Row softmax of fp32 scores scaled by `scale`, written as bf16 probabilities (one CTA per row).
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float* __restrict__ s, bf16* out, int cols,
                                                          long long ld_in, long long ld_out, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  const float* row = s + (size_t)blockIdx.x * ld_in;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, row[i] * scale);
  mx = warp_max(mx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) sum += __expf(row[i] * scale - mx);
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) sum += red[w];
  const float inv = 1.f / sum;
  bf16* o = out + (size_t)blockIdx.x * ld_out;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) o[i] = __float2bfloat16(__expf(row[i] * scale - mx) * inv);
}

// NHWC bf16 image in [-1, 1] -> RGB8: clamp, (x + 1) * 127.5, round half to even.
__global__ void __launch_bounds__(256) rgb8_kernel(const bf16* __restrict__ x, uint8_t* out, long long npix, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= npix * 3) return;
  const long long p = i / 3;
  const int c = (int)(i % 3);
  float v = __bfloat162float(x[p * C + c]);
  v = fminf(fmaxf(v, -1.f), 1.f);
  out[i] = (uint8_t)__float2int_rn((v + 1.f) * 127.5f);
}

// 3x3, stride 1, zero-padding 1 patch gather over NHWC bf16: out[(n, h, w), (kh, kw, c)] = x[n, h+kh-1, w+kw-1, c].
// The result feeds the tcgen05 GEMM against weights laid out [C_out, (kh, kw, c)].
__global__ void __launch_bounds__(256) im2col3x3_kernel(const bf16* __restrict__ x, bf16* out, int N, int H, int W,
                                                       int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int c8 = C / 8;
  const long long total = (long long)N * H * W * 9 * c8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int v = (int)(i % c8);
  long long r = i / c8;
  const int tap = (int)(r % 9);
  r /= 9;
  const int w = (int)(r % W);
  r /= W;
  const int h = (int)(r % H);
  const int n = (int)(r / H);
  const int ih = h + tap / 3 - 1, iw = w + tap % 3 - 1;
  uint4 val = make_uint4(0, 0, 0, 0);
  if (ih >= 0 && ih < H && iw >= 0 && iw < W)
    val = reinterpret_cast<const uint4*>(x)[(((size_t)n * H + ih) * W + iw) * c8 + v];
  reinterpret_cast<uint4*>(out)[i] = val;
}

inline int blocks_for(long long n) { return (int)((n + 255) / 256); }

}  // namespace
}  // namespace swb

extern "C" {

int swb_axpy(const void* x, const void* y, void* out, long long n, float a, float b, int is_fp32, void* stream) {
  using namespace swb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_fp32)
    return launch_kernel(axpy_f32_kernel, dim3(blocks_for(n)), dim3(256), 0, s, reinterpret_cast<const float*>(x),
                         reinterpret_cast<const float*>(y), reinterpret_cast<float*>(out), n, a, b);
  if (n % 8) return -3;
  return launch_kernel(axpy_bf16_kernel, dim3(blocks_for(n / 8)), dim3(256), 0, s, reinterpret_cast<const bf16*>(x),
                       reinterpret_cast<const bf16*>(y), reinterpret_cast<bf16*>(out), n / 8, a, b);
}

// stats: fp32 [N, G, 2] scratch. x, out: NHWC bf16 [N, H*W, C]; C / G a multiple of 8, or one of 1, 2, 4 (then
// C/8 must divide 256 and G <= 512).
int swb_groupnorm(const void* x, void* stats, const void* gamma, const void* beta, void* out, int N, int HW, int C,
                  int G, float eps, int silu, void* stream) {
  using namespace swb;
  if (N <= 0 || HW <= 0) return 0;
  if (C % G != 0 || C % 8 != 0) return -3;
  const int cpg = C / G;
  const bool rows_ok = 256 % (C / 8) == 0 && G <= 512 && (cpg % 8 == 0 || 8 % cpg == 0);
  const bool narrow = cpg % 8 != 0 || rows_ok;      // the row-coalesced kernel whenever the shape allows it
  if (cpg % 8 != 0 && !rows_ok) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(stats, 0, (size_t)N * G * 2 * sizeof(float), s);
  if (e != cudaSuccess) return -(int)e;
  // enough CTAs to cover the SMs twice on small feature maps, at most 1024 pixels per CTA on large ones
  const int chunk = narrow ? std::max(64, std::min(1024, (HW + 295) / 296)) : 1024;
  dim3 grid((HW + chunk - 1) / chunk, G, N);
  int rc = narrow ? launch_kernel(groupnorm_stats_narrow_kernel, dim3((HW + chunk - 1) / chunk, N), dim3(256), 0, s,
                                  reinterpret_cast<const bf16*>(x), reinterpret_cast<float*>(stats), HW, C, G, chunk)
                  : launch_kernel(groupnorm_stats_kernel, grid, dim3(256), 0, s, reinterpret_cast<const bf16*>(x),
                                  reinterpret_cast<float*>(stats), HW, C, G, chunk);
  if (rc) return rc;
  const long long n8 = (long long)N * HW * C / 8;
  if (256 % (C / 8) == 0) {
    // about four vectors per thread, at most eight CTAs per SM's worth of blocks
    const long long per_sample = (long long)HW * (C / 8);
    const int blocks = (int)std::max<long long>(1, std::min<long long>((per_sample + 1023) / 1024, 148 * 8));
    return launch_kernel(groupnorm_apply_kernel, dim3(blocks), dim3(256), 0, s, reinterpret_cast<const bf16*>(x),
                         reinterpret_cast<const float*>(stats), reinterpret_cast<const bf16*>(gamma),
                         reinterpret_cast<const bf16*>(beta), reinterpret_cast<bf16*>(out), N, HW, C, G, eps, silu);
  }
  return launch_kernel(groupnorm_apply_any_kernel, dim3(blocks_for(n8)), dim3(256), 0, s, reinterpret_cast<const bf16*>(x),
                       reinterpret_cast<const float*>(stats), reinterpret_cast<const bf16*>(gamma),
                       reinterpret_cast<const bf16*>(beta), reinterpret_cast<bf16*>(out), n8, HW, C, G, eps, silu);
}

int swb_upsample2x(const void* x, void* out, int N, int H, int W, int C, void* stream) {
  using namespace swb;
  if (C % 8) return -3;
  const long long total = (long long)N * 4 * H * W * (C / 8);
  return launch_kernel(upsample2x_kernel, dim3(blocks_for(total)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(out), N, H, W, C);
}

int swb_im2col3x3(const void* x, void* out, int N, int H, int W, int C, void* stream) {
  using namespace swb;
  if (C % 8) return -3;
  const long long total = (long long)N * H * W * 9 * (C / 8);
  if (total <= 0) return 0;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return -4;
  return launch_kernel(im2col3x3_kernel, dim3((unsigned)blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(out), N, H, W, C);
}

int swb_softmax_rows(const void* scores, void* out, int rows, int cols, long long ld_in, long long ld_out, float scale,
                     void* stream) {
  using namespace swb;
  if (rows <= 0) return 0;
  return launch_kernel(softmax_rows_kernel, dim3(rows), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const float*>(scores), reinterpret_cast<bf16*>(out), cols, ld_in, ld_out, scale);
}

int swb_rgb8(const void* x, void* out, long long npix, int C, void* stream) {
  using namespace swb;
  if (npix <= 0) return 0;
  return launch_kernel(rgb8_kernel, dim3(blocks_for(npix * 3)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                       reinterpret_cast<const bf16*>(x), reinterpret_cast<uint8_t*>(out), npix, C);
}

}  // extern "C"
