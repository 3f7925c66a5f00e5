// Bandwidth-bound LLM glue kernels for sm_100a: fused residual-add + RMSNorm, fused QK-norm + RoPE +
// paged-KV write, gated-activation multiply, embedding gather, LayerNorm/adaLN modulation.
//
// They replace chains of small kernels in the reference: rms_norm (candle-llm/src/primitives/nn.rs:22-31,
// six launches), apply_rope + transpose + contiguous (models/llama.rs:1084-1090), KV concat-grow /
// scatter_set (primitives/kv_cache.rs:107-117, paged_kv_cache.rs:269-283), SwiGLU (models/llama.rs:1386-1391).
#include "common.cuh"

namespace swb {

SWB_REGISTER_STATUS_UNIT(llm_ops);
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

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// out = rmsnorm(x (+ residual)) * w ; when residual != nullptr it is updated in place to x + residual.
// One CTA per row; H % 8 == 0; the row is kept in registers between the two passes (H <= 8 * 8 * THREADS).
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) rmsnorm_kernel(const bf16* __restrict__ x, int ldx, bf16* residual,
                                                         int ldr, const bf16* __restrict__ w, bf16* out, int ldo,
                                                         int H, float eps, float w_offset, const uint8_t* pf_ptr,
                                                         long long pf_bytes) {
  pdl_launch_dependents();
  pdl_wait(TL_RMSNORM);
  // The weights of the GEMM that consumes this norm do not depend on anything in flight: ask L2 for them now, so the
  // memory system works through the norm and the GEMM's prologue instead of idling (decode steps are bandwidth bound).
  if (pf_ptr) {
    constexpr long long CHUNK = 4096;
    const long long n_chunks = (pf_bytes + CHUNK - 1) / CHUNK;
    for (long long c = (long long)blockIdx.x * THREADS + threadIdx.x; c < n_chunks; c += (long long)gridDim.x * THREADS) {
      const long long off = c * CHUNK;
      const unsigned bytes = (unsigned)min(CHUNK, pf_bytes - off) & ~15u;
      if (bytes) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf_ptr + off), "r"(bytes) : "memory");
    }
  }
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = H / 8;
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      uint4 u = *reinterpret_cast<const uint4*>(x + (size_t)row * ldx + v * 8);
      unpack8(u, vals[i]);
      if (residual) {
        uint4 r = *reinterpret_cast<const uint4*>(residual + (size_t)row * ldr + v * 8);
        float rf[8];
        unpack8(r, rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] += rf[j];
        uint4 s = pack8(vals[i]);
        *reinterpret_cast<uint4*>(residual + (size_t)row * ldr + v * 8) = s;
        unpack8(s, vals[i]);  // normalise exactly what was stored (bf16-rounded residual stream)
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  ss = block_sum<THREADS>(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      uint4 wu = __ldg(reinterpret_cast<const uint4*>(w + v * 8));
      float wf[8], o[8];
      unpack8(wu, wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * (wf[j] + w_offset);
      *reinterpret_cast<uint4*>(out + (size_t)row * ldo + v * 8) = pack8(o);
    }
  }
}

// LayerNorm without affine followed by adaLN modulation: out = LN(x) * (1 + scale) + shift, where
// scale/shift are per-batch vectors (row / rows_per_batch selects the batch).
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) layernorm_mod_kernel(const bf16* __restrict__ x, int ldx,
                                                               const bf16* __restrict__ scale,
                                                               const bf16* __restrict__ shift, int ld_mod,
                                                               int rows_per_batch, const bf16* __restrict__ gamma,
                                                               const bf16* __restrict__ beta, bf16* out, int ldo, int H,
                                                               float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = H / 8;
  float vals[VPT][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      unpack8(*reinterpret_cast<const uint4*>(x + (size_t)row * ldx + v * 8), vals[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += vals[i][j];
    }
  }
  const float mean = block_sum<THREADS>(s, red) / (float)H;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = vals[i][j] - mean;
        ss += d * d;
      }
    }
  }
  const float inv = rsqrtf(block_sum<THREADS>(ss, red) / (float)H + eps);
  const int b = rows_per_batch > 0 ? row / rows_per_batch : 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (vals[i][j] - mean) * inv;
      if (gamma) {
        float g[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(gamma + v * 8)), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= g[j];
      }
      if (beta) {
        float g[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(beta + v * 8)), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += g[j];
      }
      if (scale) {
        float sc[8];
        unpack8(*reinterpret_cast<const uint4*>(scale + (size_t)b * ld_mod + v * 8), sc);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= (1.f + sc[j]);
      }
      if (shift) {
        float sh[8];
        unpack8(*reinterpret_cast<const uint4*>(shift + (size_t)b * ld_mod + v * 8), sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += sh[j];
      }
      *reinterpret_cast<uint4*>(out + (size_t)row * ldo + v * 8) = pack8(o);
    }
  }
}

// Per (token, head) warp: optional per-head RMSNorm (q_norm / k_norm), rotary embedding from a
// precomputed fp32 cos/sin table [max_pos, rot_dim/2], then: q heads are written back in place, k and v
// heads are written into the paged cache (layout [block, kv_head, block_size, head_dim]) at slot_mapping[t].
// interleaved = 0: NeoX half-split pairs (i, i + rot_dim/2); 1: GPT-J pairs (2i, 2i+1).
__global__ void __launch_bounds__(256) rope_kv_write_kernel(
    bf16* qkv, int ld_qkv, const int* __restrict__ positions, const long long* __restrict__ slot_mapping,
    const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_dim, int interleaved,
    const bf16* __restrict__ q_norm_w, const bf16* __restrict__ k_norm_w, float norm_eps, float norm_w_offset,
    bf16* kcache, bf16* vcache, int block_size, int T, int Hq, int Hkv, int D) {
  pdl_launch_dependents();
  pdl_wait(TL_ROPE_KV);
  __shared__ float rope_smem[8 * 256];
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int heads = Hq + 2 * Hkv;
  if (gw >= (long long)T * heads) return;
  const int t = (int)(gw / heads);
  const int h = (int)(gw % heads);
  bf16* src = qkv + (size_t)t * ld_qkv + (size_t)h * D;
  const bool is_q = h < Hq;
  const bool is_k = !is_q && h < Hq + Hkv;
  const int pos = positions[t];
  const int epl = (D + 31) / 32;  // elements per lane, <= 8 (D <= 256)
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = lane + i * 32;
    v[i] = (i < epl && d < D) ? __bfloat162float(src[d]) : 0.f;
  }
  bf16* dst = src;
  if (!is_q && (is_k ? kcache : vcache) != nullptr) {
    // with a cache the k / v heads go to their slot (in-place otherwise: dense attention reads qkv directly)
    const long long slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot < 0) {
      dst = nullptr;  // padding token: nothing to cache
    } else {
      const long long blk = slot / block_size;
      const int off = (int)(slot % block_size);
      const int kvh = is_k ? (h - Hq) : (h - Hq - Hkv);
      bf16* base = is_k ? kcache : vcache;
      dst = base + (((size_t)blk * Hkv + kvh) * block_size + off) * (size_t)D;
    }
  }
  if (is_q || is_k) {
    const bf16* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + norm_eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = lane + i * 32;
        if (i < epl && d < D) {
          // round through bf16 like an unfused norm would before the rotation
          v[i] = __bfloat162float(__float2bfloat16(v[i] * inv * (__bfloat162float(nw[d]) + norm_w_offset)));
        }
      }
    }
    const int half = rot_dim / 2;
    const float* cs = cos_tab + (size_t)pos * half;
    const float* sn = sin_tab + (size_t)pos * half;
    if (!interleaved) {
      // partner of element d (< rot_dim) is d +/- half; exchange through this warp's shared-memory row
      float* row = rope_smem + (threadIdx.x >> 5) * 256;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = lane + i * 32;
        if (i < epl && d < D) row[d] = v[i];
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = lane + i * 32;
        if (i < epl && d < rot_dim) {
          const bool lo = d < half;
          const float partner = row[lo ? d + half : d - half];
          const int fi = lo ? d : d - half;
          const float c = cs[fi], sgn = sn[fi];
          v[i] = lo ? (v[i] * c - partner * sgn) : (v[i] * c + partner * sgn);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = lane + i * 32;
        const float partner = __shfl_xor_sync(0xffffffffu, v[i], 1);
        if (i < epl && d < rot_dim) {
          const int fi = d >> 1;
          const float c = cs[fi], sgn = sn[fi];
          v[i] = (d & 1) ? (v[i] * c + partner * sgn) : (v[i] * c - partner * sgn);
        }
      }
    }
  }
  if (dst) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane + i * 32;
      if (i < epl && d < D) dst[d] = __float2bfloat16(v[i]);
    }
  }
  if (is_k && dst != src) {   // the rotated key also stays in the projection buffer
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane + i * 32;
      if (i < epl && d < D) src[d] = __float2bfloat16(v[i]);
    }
  }
}

// Head dim 128 with full rotary width: every lane owns four elements so that both members of each rotation pair are
// lane-local (interleaved: elements 4l..4l+3; half-split: 2l, 2l+1, 64+2l, 65+2l) and all accesses are 4- or 8-byte
// vectors. V heads are only touched when they have to be copied into a cache.
template <bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_kv_write_d128_kernel(
    bf16* qkv, int ld_qkv, const int* __restrict__ positions, const long long* __restrict__ slot_mapping,
    const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, const bf16* __restrict__ q_norm_w,
    const bf16* __restrict__ k_norm_w, float norm_eps, float norm_w_offset, bf16* kcache, bf16* vcache, int block_size,
    int T, int Hq, int Hkv, int heads_active) {
  pdl_launch_dependents();
  pdl_wait(TL_ROPE_KV);
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)T * heads_active) return;
  const int t = (int)(gw / heads_active);
  const int h = (int)(gw % heads_active);
  bf16* src = qkv + (size_t)t * ld_qkv + (size_t)h * D;
  const bool is_q = h < Hq;
  const bool is_k = !is_q && h < Hq + Hkv;
  const int e0 = INTERLEAVED ? 4 * lane : 2 * lane;         // first element of the low pair block
  const int e1 = INTERLEAVED ? 4 * lane + 2 : 64 + 2 * lane;  // first element of the second block
  float v[4];
  {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + e0));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + e1));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  }
  bf16* dst = src;
  if (!is_q && (is_k ? kcache : vcache) != nullptr) {
    const long long slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot < 0) {
      dst = nullptr;
    } else {
      const long long blk = slot / block_size;
      const int off = (int)(slot % block_size);
      const int kvh = is_k ? (h - Hq) : (h - Hq - Hkv);
      dst = (is_k ? kcache : vcache) + (((size_t)blk * Hkv + kvh) * block_size + off) * (size_t)D;
    }
  }
  if (is_q || is_k) {
    const bf16* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + norm_eps);
      const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + e0));
      const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + e1));
      // round through bf16 like an unfused norm would before the rotation
      v[0] = __bfloat162float(__float2bfloat16(v[0] * inv * (wa.x + norm_w_offset)));
      v[1] = __bfloat162float(__float2bfloat16(v[1] * inv * (wa.y + norm_w_offset)));
      v[2] = __bfloat162float(__float2bfloat16(v[2] * inv * (wb.x + norm_w_offset)));
      v[3] = __bfloat162float(__float2bfloat16(v[3] * inv * (wb.y + norm_w_offset)));
    }
    const int pos = positions[t];
    const float2 c = *reinterpret_cast<const float2*>(cos_tab + (size_t)pos * 64 + 2 * lane);
    const float2 sn = *reinterpret_cast<const float2*>(sin_tab + (size_t)pos * 64 + 2 * lane);
    float o[4];
    if (INTERLEAVED) {   // pairs (v0, v1) with angle 2l and (v2, v3) with angle 2l + 1
      o[0] = v[0] * c.x - v[1] * sn.x;
      o[1] = v[1] * c.x + v[0] * sn.x;
      o[2] = v[2] * c.y - v[3] * sn.y;
      o[3] = v[3] * c.y + v[2] * sn.y;
    } else {             // pairs (v0, v2) with angle 2l and (v1, v3) with angle 2l + 1
      o[0] = v[0] * c.x - v[2] * sn.x;
      o[2] = v[2] * c.x + v[0] * sn.x;
      o[1] = v[1] * c.y - v[3] * sn.y;
      o[3] = v[3] * c.y + v[1] * sn.y;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = o[i];
  }
  if (dst) {
    *reinterpret_cast<__nv_bfloat162*>(dst + e0) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + e1) = __floats2bfloat162_rn(v[2], v[3]);
  }
  if (is_k && dst != src) {   // the rotated key also stays in the projection buffer (prefill attention reads it there)
    *reinterpret_cast<__nv_bfloat162*>(src + e0) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(src + e1) = __floats2bfloat162_rn(v[2], v[3]);
  }
}

// out[t, f] = act(gu[t, f]) * gu[t, F + f]; act 1 = SiLU (SwiGLU), 2 = tanh-GELU (GeGLU). act 3 / 4: the same two
// activations on a pair-interleaved projection output, out[t, f] = act(gu[t, 2f]) * gu[t, 2f + 1].
__global__ void __launch_bounds__(256) gated_act_mul_kernel(const bf16* __restrict__ gu, int ld_gu, bf16* out,
                                                           int ldo, int T, int F, int act) {
  pdl_launch_dependents();
  pdl_wait(TL_GATED_ACT);
  const int nvec = F / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * nvec) return;
  const int t = (int)(idx / nvec);
  const int v = (int)(idx % nvec);
  float g[8], u[8], o[8];
  if (act >= 3) {
    float lo[8], hi[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + (size_t)t * ld_gu + v * 16), lo);
    unpack8(*reinterpret_cast<const uint4*>(gu + (size_t)t * ld_gu + v * 16 + 8), hi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      g[j] = lo[2 * j];
      u[j] = lo[2 * j + 1];
      g[4 + j] = hi[2 * j];
      u[4 + j] = hi[2 * j + 1];
    }
  } else {
    unpack8(*reinterpret_cast<const uint4*>(gu + (size_t)t * ld_gu + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + (size_t)t * ld_gu + F + v * 8), u);
  }
  const bool gelu = act == 2 || act == 4;
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = (gelu ? gelu_tanh_f(g[j]) : silu_f(g[j])) * u[j];
  *reinterpret_cast<uint4*>(out + (size_t)t * ldo + v * 8) = pack8(o);
}

__global__ void __launch_bounds__(256) embedding_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table,
                                                       bf16* out, int T, int H, int vocab_start, int vocab_end,
                                                       float scale) {
  pdl_launch_dependents();
  pdl_wait(TL_EMBED);
  const int nvec = H / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * nvec) return;
  const int t = (int)(idx / nvec);
  const int v = (int)(idx % nvec);
  const long long id = ids[t];
  uint4 u = make_uint4(0, 0, 0, 0);
  if (id >= vocab_start && id < vocab_end) {
    u = __ldg(reinterpret_cast<const uint4*>(table + (size_t)(id - vocab_start) * H + v * 8));
    if (scale != 1.f) {
      float f[8];
      unpack8(u, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= scale;
      u = pack8(f);
    }
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * H + v * 8) = u;
}

// out = a + gate * b (gate per batch row-vector), or out = a + b when gate == nullptr.
__global__ void __launch_bounds__(256) gated_residual_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                            const bf16* __restrict__ gate, int ld_gate,
                                                            int rows_per_batch, bf16* out, int T, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int nvec = H / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * nvec) return;
  const int t = (int)(idx / nvec);
  const int v = (int)(idx % nvec);
  float fa[8], fb[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(a + (size_t)t * H + v * 8), fa);
  unpack8(*reinterpret_cast<const uint4*>(b + (size_t)t * H + v * 8), fb);
  if (gate) {
    float g[8];
    const int bi = rows_per_batch > 0 ? t / rows_per_batch : 0;
    unpack8(*reinterpret_cast<const uint4*>(gate + (size_t)bi * ld_gate + v * 8), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fa[j] + g[j] * fb[j];
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fa[j] + fb[j];
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * H + v * 8) = pack8(o);
}

template <typename F>
int launch_norm(int H, F&& f) {
  const int nvec = H / 8;
  if (nvec <= 128) return f(std::integral_constant<int, 128>{}, std::integral_constant<int, 1>{});
  if (nvec <= 256) return f(std::integral_constant<int, 256>{}, std::integral_constant<int, 1>{});
  if (nvec <= 512) return f(std::integral_constant<int, 256>{}, std::integral_constant<int, 2>{});
  if (nvec <= 1024) return f(std::integral_constant<int, 256>{}, std::integral_constant<int, 4>{});
  if (nvec <= 2048) return f(std::integral_constant<int, 512>{}, std::integral_constant<int, 4>{});
  return -3;
}

static thread_local int launch_rc = 0;
inline int last_err() { return launch_rc; }

}  // namespace
}  // namespace swb

extern "C" {

int swb_rmsnorm_prefetch(const void* x, int ldx, void* residual, int ldr, const void* w, void* out, int ldo, int T,
                         int H, float eps, float w_offset, const void* prefetch_ptr, long long prefetch_bytes,
                         void* stream);

int swb_rmsnorm(const void* x, int ldx, void* residual, int ldr, const void* w, void* out, int ldo, int T, int H,
                float eps, float w_offset, void* stream) {
  return swb_rmsnorm_prefetch(x, ldx, residual, ldr, w, out, ldo, T, H, eps, w_offset, nullptr, 0, stream);
}

// As swb_rmsnorm; additionally asks L2 to fetch prefetch_bytes (16-byte aligned start) of the next kernel's weights.
int swb_rmsnorm_prefetch(const void* x, int ldx, void* residual, int ldr, const void* w, void* out, int ldo, int T,
                         int H, float eps, float w_offset, const void* prefetch_ptr, long long prefetch_bytes,
                         void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0 || (residual && ldr % 8 != 0)) return -3;
  if (prefetch_ptr && ((reinterpret_cast<uintptr_t>(prefetch_ptr) & 15) || prefetch_bytes < 0)) return -3;
  const uint8_t* pf = prefetch_bytes > 0 ? reinterpret_cast<const uint8_t*>(prefetch_ptr) : nullptr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return launch_norm(H, [&](auto TH, auto VP) {
    constexpr int THREADS = decltype(TH)::value, VPT = decltype(VP)::value;
    launch_rc = launch_kernel(rmsnorm_kernel<THREADS, VPT>, dim3(T), dim3(THREADS), 0, s, reinterpret_cast<const bf16*>(x), ldx,
                                                        reinterpret_cast<bf16*>(residual), ldr,
                                                        reinterpret_cast<const bf16*>(w), reinterpret_cast<bf16*>(out),
                                                        ldo, H, eps, w_offset, pf, prefetch_bytes);
    return last_err();
  });
}

int swb_layernorm_mod(const void* x, int ldx, const void* scale, const void* shift, int ld_mod, int rows_per_batch,
                      const void* gamma, const void* beta, void* out, int ldo, int T, int H, float eps,
                      void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0 || ld_mod % 8 != 0) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return launch_norm(H, [&](auto TH, auto VP) {
    constexpr int THREADS = decltype(TH)::value, VPT = decltype(VP)::value;
    launch_rc = launch_kernel(layernorm_mod_kernel<THREADS, VPT>, dim3(T), dim3(THREADS), 0, s, reinterpret_cast<const bf16*>(x), ldx, reinterpret_cast<const bf16*>(scale),
        reinterpret_cast<const bf16*>(shift), ld_mod, rows_per_batch, reinterpret_cast<const bf16*>(gamma),
        reinterpret_cast<const bf16*>(beta), reinterpret_cast<bf16*>(out), ldo, H, eps);
    return last_err();
  });
}

int swb_rope_kv_write(void* qkv, int ld_qkv, const int* positions, const long long* slot_mapping,
                      const float* cos_tab, const float* sin_tab, int rot_dim, int interleaved, const void* q_norm_w,
                      const void* k_norm_w, float norm_eps, float norm_w_offset, void* kcache, void* vcache,
                      int block_size, int T, int Hq, int Hkv, int D, void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (D > 256 || rot_dim > D || (rot_dim & 1)) return -3;
  const int wpb = 8;
  if (D == 128 && rot_dim == 128 && (ld_qkv % 2) == 0 && (reinterpret_cast<uintptr_t>(qkv) & 3) == 0) {
    const int heads_active = Hq + Hkv + (vcache ? Hkv : 0);   // V stays where it is unless it goes to a cache
    const long long nblk = ((long long)T * heads_active + wpb - 1) / wpb;
    auto kern = interleaved ? rope_kv_write_d128_kernel<true> : rope_kv_write_d128_kernel<false>;
    launch_rc = launch_kernel(kern, dim3((unsigned)nblk), dim3(wpb * 32), 0, reinterpret_cast<cudaStream_t>(stream),
                              reinterpret_cast<bf16*>(qkv), ld_qkv, positions, slot_mapping, cos_tab, sin_tab,
                              reinterpret_cast<const bf16*>(q_norm_w), reinterpret_cast<const bf16*>(k_norm_w),
                              norm_eps, norm_w_offset, reinterpret_cast<bf16*>(kcache), reinterpret_cast<bf16*>(vcache),
                              block_size, T, Hq, Hkv, heads_active);
    return last_err();
  }
  const long long warps = (long long)T * (Hq + 2 * Hkv);
  const long long blocks = (warps + wpb - 1) / wpb;
  launch_rc = launch_kernel(rope_kv_write_kernel, dim3((unsigned)blocks), dim3(wpb * 32), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<bf16*>(qkv), ld_qkv, positions, slot_mapping, cos_tab, sin_tab, rot_dim, interleaved,
      reinterpret_cast<const bf16*>(q_norm_w), reinterpret_cast<const bf16*>(k_norm_w), norm_eps, norm_w_offset,
      reinterpret_cast<bf16*>(kcache), reinterpret_cast<bf16*>(vcache), block_size, T, Hq, Hkv, D);
  return last_err();
}

int swb_gated_act_mul(const void* gate_up, int ld_gu, void* out, int ldo, int T, int F, int act, void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (F % 8 != 0 || ld_gu % 8 != 0 || ldo % 8 != 0) return -3;
  const long long n = (long long)T * (F / 8);
  launch_rc = launch_kernel(gated_act_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const bf16*>(gate_up), ld_gu, reinterpret_cast<bf16*>(out), ldo, T, F, act);
  return last_err();
}

int swb_embedding(const long long* ids, const void* table, void* out, int T, int H, int vocab_start, int vocab_end,
                  float scale, void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (H % 8 != 0) return -3;
  const long long n = (long long)T * (H / 8);
  launch_rc = launch_kernel(embedding_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), ids, reinterpret_cast<const bf16*>(table), reinterpret_cast<bf16*>(out), T, H, vocab_start, vocab_end, scale);
  return last_err();
}

int swb_gated_residual(const void* a, const void* b, const void* gate, int ld_gate, int rows_per_batch, void* out,
                       int T, int H, void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (H % 8 != 0 || (gate && ld_gate % 8 != 0)) return -3;
  const long long n = (long long)T * (H / 8);
  launch_rc = launch_kernel(gated_residual_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const bf16*>(a), reinterpret_cast<const bf16*>(b), reinterpret_cast<const bf16*>(gate), ld_gate,
      rows_per_batch, reinterpret_cast<bf16*>(out), T, H);
  return last_err();
}

}  // extern "C"
