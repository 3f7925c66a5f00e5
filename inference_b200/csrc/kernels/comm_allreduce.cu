// One-shot all-reduce over NVLink peer memory fused with residual add and RMSNorm (tensor-parallel decode).
//
// Every rank's row-parallel GEMM writes its partial [T, H] tile straight into a symmetric-memory buffer. This
// kernel then (1) runs a flag barrier with every peer (release store of an epoch into the peer's flag word,
// bounded acquire spin on its own), (2) pulls the P partial rows with 16-byte peer loads, sums them in fp32 in
// rank order (so every rank produces bit-identical results), (3) adds the residual stream and writes it back,
// (4) applies RMSNorm and writes the normalised activations for the next column-parallel GEMM.
// It replaces ncclAllReduce + residual add + rms_norm (the reference has no collective at all: its only
// multi-GPU path copies the hidden state between devices, candle-llm/src/models/llama.rs:690-707).
// Buffers are double-buffered by the caller, so no trailing barrier is needed: a buffer is rewritten only after
// the next call's leading barrier proved that every peer finished reading it.
// Waits are bounded: on expiry the CTA records {where, rank, peer} in the status word and skips the reduction.
#include "common.cuh"

#include <type_traits>

namespace swb {

SWB_REGISTER_STATUS_UNIT(comm_allreduce);

namespace {

constexpr int MAX_RANKS = 8;
constexpr int MAX_CTAS = 256;

struct ArParams {
  const bf16* peer_data[MAX_RANKS];
  uint32_t* peer_flags[MAX_RANKS];  // [MAX_CTAS][MAX_RANKS] per rank
  uint32_t* epochs;                 // local, [MAX_CTAS]
  int rank, world, T, H, ld_data;
  bf16* residual;
  int ldr;
  const bf16* weight;
  float eps, w_offset;
  bf16* out;
  int ldo;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
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

// Flag barrier of CTA `blockIdx.x` with the same CTA on every peer. Returns false on timeout.
__device__ __forceinline__ bool peer_barrier(const ArParams& p, uint32_t epoch, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    // The release store alone orders everything this rank wrote before the barrier: earlier kernels' writes are
    // visible to this thread at the kernel boundary and a system-scope release is cumulative over them.
    st_release_sys(p.peer_flags[peer] + (size_t)blockIdx.x * MAX_RANKS + p.rank, epoch);
    const uint32_t* mine = p.peer_flags[p.rank] + (size_t)blockIdx.x * MAX_RANKS + peer;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) break;
      if ((it & 0x3F) == 0x3F) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > g_wait_limit_ns) {
          report_error(SWB_ERR_PEER_TIMEOUT, 1000 + (int)blockIdx.x, p.rank, peer);
          *s_ok = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) allreduce_rmsnorm_kernel(const ArParams p) {
  pdl_launch_dependents();
  pdl_wait(TL_PEER);
  __shared__ float red[32];
  __shared__ int s_ok;
  const uint32_t epoch = p.epochs[blockIdx.x] + 1u;
  const bool ok = peer_barrier(p, epoch, &s_ok);
  if (threadIdx.x == 0) p.epochs[blockIdx.x] = epoch;
  if (!ok) return;

  const int nvec = p.H / 8;
  for (int row = blockIdx.x; row < p.T; row += gridDim.x) {
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
        uint4 part[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < p.world) part[r] = ld_peer16(p.peer_data[r] + (size_t)row * p.ld_data + v * 8);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) {
          if (r < p.world) {
            float f[8];
            unpack8(part[r], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] += f[j];
          }
        }
        if (p.residual) {
          float rf[8];
          unpack8(*reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ldr + v * 8), rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += rf[j];
          uint4 s = pack8(vals[i]);
          *reinterpret_cast<uint4*>(p.residual + (size_t)row * p.ldr + v * 8) = s;
          unpack8(s, vals[i]);
        } else if (p.weight) {
          uint4 s = pack8(vals[i]);  // normalise the bf16-rounded sum, like a separate all-reduce would
          unpack8(s, vals[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    float inv = 1.f;
    if (p.weight) {
      ss = warp_sum(ss);
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      float t = (lane < THREADS / 32) ? red[lane] : 0.f;
      t = warp_sum(t);
      __syncthreads();
      inv = rsqrtf(t / (float)p.H + p.eps);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
        float o[8];
        if (p.weight) {
          float wf[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.weight + v * 8)), wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * (wf[j] + p.w_offset);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j];
        }
        *reinterpret_cast<uint4*>(p.out + (size_t)row * p.ldo + v * 8) = pack8(o);
      }
    }
  }
}

// Second half of the fused reduce-scatter, joined with the all-gather that feeds the next column-parallel GEMM
// (sequence-parallel tensor parallelism for prefill). This rank owns `rows` token rows. Peers' row-parallel GEMM
// epilogues have stored their bf16 partial sums into the local slot buffer [world, rows_per_rank, H]. Per row:
// barrier (first), fp32 sum over the slots in rank order (+ the local residual shard, which is updated in place),
// RMSNorm, and the normed row is stored into EVERY rank's gathered activation buffer at its global row.
// n_src == 0 skips the slots (first layer: norm of the residual only).
struct RsAgParams {
  ArParams ar;                 // peer_flags / epochs / rank / world / H / residual / weight / eps ... (data unused)
  const bf16* slots;           // local [world, rows_per_rank, H]
  bf16* gather[MAX_RANKS];     // every rank's [T, ld_gather] buffer
  int n_src, rows, rows_per_rank, row_offset, ld_gather;
};

template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) reduce_norm_gather_kernel(const RsAgParams q) {
  pdl_launch_dependents();
  pdl_wait();
  const ArParams& p = q.ar;
  __shared__ float red[32];
  __shared__ int s_ok;
  const uint32_t epoch = p.epochs[blockIdx.x] + 1u;
  const bool ok = peer_barrier(p, epoch, &s_ok);
  if (threadIdx.x == 0) p.epochs[blockIdx.x] = epoch;
  if (!ok) return;
  const int nvec = p.H / 8;
  for (int row = blockIdx.x; row < q.rows; row += gridDim.x) {
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
        for (int r = 0; r < q.n_src; ++r) {
          float f[8];
          unpack8(__ldcg(reinterpret_cast<const uint4*>(q.slots + ((size_t)r * q.rows_per_rank + row) * p.H + v * 8)), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += f[j];
        }
        if (p.residual) {
          uint4* rp = reinterpret_cast<uint4*>(p.residual + (size_t)row * p.ldr + v * 8);
          if (q.n_src > 0) {
            float rf[8];
            unpack8(*rp, rf);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] += rf[j];
            const uint4 s = pack8(vals[i]);
            *rp = s;
            unpack8(s, vals[i]);
          } else {
            unpack8(*rp, vals[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    ss = warp_sum(ss);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float t = (lane < THREADS / 32) ? red[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    const float inv = rsqrtf(t / (float)p.H + p.eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
        float o[8], wf[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.weight + v * 8)), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * (wf[j] + p.w_offset);
        const uint4 packed = pack8(o);
        const size_t off = (size_t)(q.row_offset + row) * q.ld_gather + v * 8;
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < p.world) *reinterpret_cast<uint4*>(q.gather[r] + off) = packed;
      }
    }
  }
}

struct PairParams {
  const float* vals[MAX_RANKS];          // per rank: [rows] best value of its vocabulary shard
  const long long* ids[MAX_RANKS];       // per rank: [rows] index inside the shard
  long long* out;                        // [rows] global token ids
  int rows, vocab_local;
};

// One CTA: flag barrier (flag row 0, like peer_barrier_kernel), then thread = row pulls `world` candidates.
__global__ void __launch_bounds__(128) argmax_peer_merge_kernel(const ArParams p, const PairParams q) {
  pdl_launch_dependents();
  pdl_wait(TL_PEER);
  __shared__ int s_ok;
  const uint32_t epoch = p.epochs[0] + 1u;
  const bool ok = peer_barrier(p, epoch, &s_ok);
  if (threadIdx.x == 0) p.epochs[0] = epoch;
  if (!ok) return;
  for (int row = threadIdx.x; row < q.rows; row += blockDim.x) {
    float best = 0.f;
    long long best_id = 0;
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < p.world) {
        uint32_t vb;
        unsigned long long ib;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(vb) : "l"(q.vals[r] + row) : "memory");
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(ib) : "l"(q.ids[r] + row) : "memory");
        const float v = __uint_as_float(vb);
        if (r == 0 || v > best) {
          best = v;
          best_id = (long long)ib + (long long)r * q.vocab_local;
        }
      }
    }
    q.out[row] = best_id;
  }
}

// Barrier across ranks between two kernels of a stream (everything this rank's earlier kernels wrote to peers is
// visible to a peer once that peer's barrier returns). One CTA; flag row `blockIdx.x` = 0 of its own flag pad.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const ArParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  const uint32_t epoch = p.epochs[0] + 1u;
  peer_barrier(p, epoch, &s_ok);
  if (threadIdx.x == 0) p.epochs[0] = epoch;
}

// A stand-alone wait used by the timeout test: spins on one local flag word that nothing sets.
__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t expected, int* result) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(ld_acquire_sys(flag) - expected) >= 0) {
      *result = 1;
      return;
    }
    if ((it & 0x3F) == 0x3F) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > g_wait_limit_ns) {
        report_error(SWB_ERR_PEER_TIMEOUT, 2000, 0, 0);
        *result = 0;
        return;
      }
    }
  }
}

}  // namespace
}  // namespace swb

extern "C" {

int swb_comm_max_ctas(void) { return swb::MAX_CTAS; }
int swb_comm_flag_words(void) { return swb::MAX_CTAS * swb::MAX_RANKS; }

// out = rmsnorm(sum_r data_r [+ residual]) * (weight + w_offset); residual (if given) becomes the sum.
// weight == null: out = sum (+ residual). peer_data / peer_flags: `world` device pointers each.
int swb_allreduce_rmsnorm(const void* const* peer_data, void* const* peer_flags, void* epochs, int rank, int world,
                          int T, int H, int ld_data, void* residual, int ldr, const void* weight, float eps,
                          float w_offset, void* out, int ldo, void* stream) {
  using namespace swb;
  if (T <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || H % 8 != 0 || ld_data % 8 != 0 || ldo % 8 != 0) return -3;
  ArParams p{};
  for (int r = 0; r < world; ++r) {
    p.peer_data[r] = reinterpret_cast<const bf16*>(peer_data[r]);
    p.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
  }
  p.epochs = reinterpret_cast<uint32_t*>(epochs);
  p.rank = rank;
  p.world = world;
  p.T = T;
  p.H = H;
  p.ld_data = ld_data;
  p.residual = reinterpret_cast<bf16*>(residual);
  p.ldr = ldr;
  p.weight = reinterpret_cast<const bf16*>(weight);
  p.eps = eps;
  p.w_offset = w_offset;
  p.out = reinterpret_cast<bf16*>(out);
  p.ldo = ldo;
  const int grid = T < MAX_CTAS ? T : MAX_CTAS;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nvec = H / 8;
  if (nvec <= 128) return launch_kernel(allreduce_rmsnorm_kernel<128, 1>, dim3(grid), dim3(128), 0, s, p);
  if (nvec <= 256) return launch_kernel(allreduce_rmsnorm_kernel<256, 1>, dim3(grid), dim3(256), 0, s, p);
  if (nvec <= 512) return launch_kernel(allreduce_rmsnorm_kernel<512, 1>, dim3(grid), dim3(512), 0, s, p);
  if (nvec <= 1024) return launch_kernel(allreduce_rmsnorm_kernel<512, 2>, dim3(grid), dim3(512), 0, s, p);
  if (nvec <= 2048) return launch_kernel(allreduce_rmsnorm_kernel<512, 4>, dim3(grid), dim3(512), 0, s, p);
  return -3;
}

// See reduce_norm_gather_kernel. slots: local [world, rows_per_rank, H]; gather: `world` pointers to [T, ld_gather];
// residual: local [rows, ldr] (updated in place when n_src > 0); rows: rows this rank owns (may be 0: the rank still
// takes part in the barrier). peer_flags as for swb_allreduce_rmsnorm (pads of MAX_CTAS * MAX_RANKS words).
int swb_reduce_norm_gather(const void* slots, int n_src, void* residual, int ldr, const void* weight, float eps,
                           float w_offset, void* const* gather, int ld_gather, int row_offset, int rows,
                           int rows_per_rank, int H, void* const* peer_flags, void* epochs, int rank, int world,
                           void* stream) {
  using namespace swb;
  if (world < 1 || world > MAX_RANKS || H % 8 != 0 || ld_gather % 8 != 0 || !weight || !residual) return -3;
  RsAgParams q{};
  for (int r = 0; r < world; ++r) {
    q.ar.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
    q.gather[r] = reinterpret_cast<bf16*>(gather[r]);
  }
  q.ar.epochs = reinterpret_cast<uint32_t*>(epochs);
  q.ar.rank = rank;
  q.ar.world = world;
  q.ar.H = H;
  q.ar.residual = reinterpret_cast<bf16*>(residual);
  q.ar.ldr = ldr;
  q.ar.weight = reinterpret_cast<const bf16*>(weight);
  q.ar.eps = eps;
  q.ar.w_offset = w_offset;
  q.slots = reinterpret_cast<const bf16*>(slots);
  q.n_src = n_src;
  q.rows = rows;
  q.rows_per_rank = rows_per_rank;
  q.row_offset = row_offset;
  q.ld_gather = ld_gather;
  // every rank launches the same grid so that CTA b meets CTA b of its peers at the barrier
  const int grid = rows_per_rank < MAX_CTAS ? (rows_per_rank > 0 ? rows_per_rank : 1) : MAX_CTAS;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nvec = H / 8;
  if (nvec <= 256) return launch_kernel(reduce_norm_gather_kernel<256, 1>, dim3(grid), dim3(256), 0, s, q);
  if (nvec <= 512) return launch_kernel(reduce_norm_gather_kernel<512, 1>, dim3(grid), dim3(512), 0, s, q);
  if (nvec <= 1024) return launch_kernel(reduce_norm_gather_kernel<512, 2>, dim3(grid), dim3(512), 0, s, q);
  if (nvec <= 2048) return launch_kernel(reduce_norm_gather_kernel<512, 4>, dim3(grid), dim3(512), 0, s, q);
  return -3;
}

// Distributed argmax of a vocabulary-parallel output head: every rank has written its shard's best (value, local
// index) per row into its own symmetric buffers; after the flag barrier each rank pulls all shards' candidates over
// NVLink and keeps the largest value (ties: lowest rank = lowest global index, like a single-device argmax).
int swb_argmax_peer_merge(const void* const* peer_vals, const void* const* peer_ids, void* const* peer_flags,
                          void* epochs, int rank, int world, int rows, int vocab_local, long long* out_ids,
                          void* stream) {
  using namespace swb;
  if (world < 1 || world > MAX_RANKS || rows < 0) return -3;
  if (rows == 0) return 0;
  ArParams p{};
  PairParams q{};
  for (int r = 0; r < world; ++r) {
    p.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
    q.vals[r] = reinterpret_cast<const float*>(peer_vals[r]);
    q.ids[r] = reinterpret_cast<const long long*>(peer_ids[r]);
  }
  p.epochs = reinterpret_cast<uint32_t*>(epochs);
  p.rank = rank;
  p.world = world;
  q.rows = rows;
  q.vocab_local = vocab_local;
  q.out = out_ids;
  return launch_kernel(argmax_peer_merge_kernel, dim3(1), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), p, q);
}

// peer_flags: `world` pointers to flag pads of at least MAX_RANKS words; epochs: one local word.
int swb_peer_barrier(void* const* peer_flags, void* epochs, int rank, int world, void* stream) {
  using namespace swb;
  if (world < 1 || world > MAX_RANKS) return -3;
  ArParams p{};
  for (int r = 0; r < world; ++r) p.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
  p.epochs = reinterpret_cast<uint32_t*>(epochs);
  p.rank = rank;
  p.world = world;
  return launch_kernel(peer_barrier_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), p);
}

// Bounded wait on a flag nothing sets (health / timeout self-test): result[0] = 1 if the flag reached
// `expected`, 0 if the wait budget ran out (the status word then holds SWB_ERR_PEER_TIMEOUT).
int swb_flag_wait(const void* flag, unsigned expected, int* result, void* stream) {
  swb::flag_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(flag), expected, result);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

}  // extern "C"
