// Decode-sized bf16 GEMM (tokens <= 64) as a thread-block-cluster split-K kernel for sm_100a.
//
// out[T, N] = act(x[T, K] * W[N, K]^T + bias) + residual with T <= 64 is pure weight streaming: the
// roofline is HBM bandwidth, and one 128-row weight tile per CTA leaves most SMs idle (N = 4096 gives 32
// tiles for 148 SMs). Here a cluster of 2/4/8 CTAs shares one weight tile and splits K between its
// members; each member streams its K range by TMA into a small ring (two CTAs fit per SM), accumulates
// with tcgen05.mma into TMEM (weights as the M = 128 operand, tokens as N), then the partial tiles are
// reduce-scattered through distributed shared memory: member r receives every member's rows
// [r * R, (r + 1) * R), R = ceil(128 / C), by st.shared::cluster, sums them in a fixed order
// (deterministic) and runs the fused epilogue for its slice. No global workspace, atomics or fences.
// The weight operand does not depend on the preceding kernel, so its first stages are requested before
// the programmatic-dependent-launch wait.
#include "common.cuh"
#include "gemm_tcgen05.cuh"

#include <algorithm>
#include <cstdlib>

namespace swb {

SWB_REGISTER_STATUS_UNIT(gemm_decode_cluster);

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int EPI_WARPS = 8;                 // two warps per TMEM lane quarter: each takes half of the token columns
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int THREADS = 64 + EPI_THREADS;

// STAGES_ = 4: two CTAs per SM (large weights: bytes in flight across the whole GPU); STAGES_ = 8: one CTA per SM with
// a ring deep enough to hold most or all of a small projection's k-range, requested before the dependency on the
// previous kernel resolves (decode steps are a chain of small dependent kernels: whatever is already in shared memory
// when the activations arrive is off the critical path). The receive buffer of the cluster reduction aliases the ring:
// partial tiles are exchanged only after every member's last MMA has read its ring.
template <int BLOCK_N, int STAGES_>
struct DecCfg {
  static constexpr int STAGES = STAGES_;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BLOCK_N * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t RECV_BYTES = (BM + 16) * BLOCK_N * 4;  // CLUSTER slots of [BLOCK_N][rows per member] fp32
  static constexpr uint32_t RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr uint32_t DATA_BYTES = RING_BYTES > RECV_BYTES ? RING_BYTES : RECV_BYTES;
  static constexpr uint32_t TMEM_COLS = BLOCK_N < 32 ? 32 : BLOCK_N;
  static constexpr size_t SMEM_BYTES = (size_t)DATA_BYTES + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void st_cluster_f32x2(uint32_t addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}

// barrier of the epilogue warps (threads 64 ..) only
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory"); }

// Flag-in-data lines for the cross-rank sum: 16 bytes = {data, epoch, data, epoch}. Each 8-byte half is written
// atomically, so a reader that sees both epochs has both data words; no fence or separate flag is needed and a row
// crosses NVLink in one hop. (The same idea as the low-latency protocol of collective libraries.)
__device__ __forceinline__ void st_line(uint4* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Bounded spin until both lines at `src` carry `epoch`; returns their four data words in `out`. On expiry records
// {where, rank, peer} in the status word and returns false.
__device__ __forceinline__ bool ld_lines(const uint4* src, uint32_t epoch, uint4& out, int where, int rank, int peer) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    const uint4 a = ld_line(src), b = ld_line(src + 1);
    if (a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch) {
      out = make_uint4(a.x, a.z, b.x, b.z);
      return true;
    }
    if ((it & 0x3F) == 0x3F) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > g_wait_limit_ns) {
        report_error(SWB_ERR_PEER_TIMEOUT, where, rank, peer);
        return false;
      }
    }
  }
}
// Batched form for the rank that sums: the lines of four peers for one 16-byte group are requested together, so the
// wait costs one memory round trip per four peers once the data has landed instead of one per peer. `bases[r]` is the
// first line of peer first_peer + r (unused where bit r of `need` is clear); the data words land in u[r].
__device__ __forceinline__ bool ld_lines_all(const uint4* const* bases, uint32_t need, uint32_t epoch, uint4* u, int where,
                                             int rank, int first_peer) {
  uint64_t t0 = 0;
  uint32_t pending = need;
  for (uint32_t it = 0; pending; ++it) {
    uint4 a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (pending & (1u << r)) {
        a[r] = ld_line(bases[r]);
        b[r] = ld_line(bases[r] + 1);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if ((pending & (1u << r)) && a[r].y == epoch && a[r].w == epoch && b[r].y == epoch && b[r].w == epoch) {
        u[r] = make_uint4(a[r].x, a[r].z, b[r].x, b[r].z);
        pending &= ~(1u << r);
      }
    }
    if (pending && (it & 0x3F) == 0x3F) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > g_wait_limit_ns) {
        report_error(SWB_ERR_PEER_TIMEOUT, where, rank, first_peer + __ffs(pending) - 1);
        return false;
      }
    }
  }
  return true;
}
// sum of squares -> 2^-24 fixed point (integer accumulation is order independent, so every rank and every replay
// gets the same bits)
__device__ __forceinline__ unsigned long long ssq_fixed(float ss) {
  return __float2ull_rn(fminf(ss, 5.0e11f) * 16777216.f);
}

__device__ __forceinline__ float act_apply(float x, int act) {
  if (act == SWB_ACT_SILU) return silu_f(x);
  if (act == SWB_ACT_GELU_TANH) return gelu_tanh_f(x);
  return x;
}

// PEER instantiates the cross-rank epilogue (its batched peer loads need more registers than the plain store path).
template <int BLOCK_N, int CLUSTER, int STAGES_, bool PEER>
__global__ void __launch_bounds__(THREADS, STAGES_ > 4 ? 1 : 2)
gemm_decode_cluster_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                           const GemmParams p) {
  using Cfg = DecCfg<BLOCK_N, STAGES_>;
  constexpr int STAGES = Cfg::STAGES;
  // output-feature rows owned by each cluster member, rounded up to 8 so the final store is 16-byte vectors
  constexpr int R = (((BM + CLUSTER - 1) / CLUSTER) + 7) / 8 * 8;
  static_assert(CLUSTER * R * BLOCK_N * 4 <= (int)Cfg::RECV_BYTES, "receive buffer too small for this cluster size");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  float* recv = reinterpret_cast<float*>(smem);      // aliases the ring (free once every member's MMAs are done)
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + Cfg::DATA_BYTES);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_tfull = bar_empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tfull + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float s_rstd[64];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* tr = p.trace ? p.trace + (size_t)blockIdx.x * 16 : nullptr;   // [0..7] globaltimer, [8..15] SM clock
  if (tr && threadIdx.x == 0) tr[0] = global_timer_ns();
  const uint32_t crank = CLUSTER > 1 ? cluster_ctarank() : 0u;
  const int tile_m = (int)blockIdx.x / CLUSTER;
  const int kps = (p.kblocks_total + CLUSTER - 1) / CLUSTER;
  const int kb0 = (int)crank * kps;
  const int kb1 = min(p.kblocks_total, kb0 + kps);
  const int nkb = max(0, kb1 - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    mbar_init(bar_tfull, 1);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
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
  if (tr && threadIdx.x == 0) tr[1] = global_timer_ns();   // setup done

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const int pre = min(STAGES, nkb);
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&bar_full[i], Cfg::STAGE_BYTES);
        tma_load_2d_hint(smem + i * Cfg::STAGE_BYTES, &tmap_w, &bar_full[i], (kb0 + i) * BK, tile_m * BM, pol_w);
      }
      pdl_wait(TL_GEMM_DECODE);
      if (tr) tr[2] = global_timer_ns();                   // dependency satisfied
      int stage = 0;
      uint32_t phase = 0;
      uint32_t outstanding = (pre >= 32) ? 0xffffffffu : ((1u << pre) - 1u);
      uint32_t issue_phase_bits = 0;
      for (int i = 0; i < nkb; ++i) {
        uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
        uint8_t* sb = sa + Cfg::A_BYTES;
        if (i >= pre) {
          if (!mbar_wait(&bar_empty[stage], phase ^ 1, s_abort, 700 + stage)) break;
          mbar_arrive_expect_tx(&bar_full[stage], Cfg::STAGE_BYTES);
          tma_load_2d_hint(sa, &tmap_w, &bar_full[stage], (kb0 + i) * BK, tile_m * BM, pol_w);
          outstanding |= 1u << stage;
          issue_phase_bits = (issue_phase_bits & ~(1u << stage)) | (phase << stage);
        }
        tma_load_2d_hint(sb, &tmap_x, &bar_full[stage], (kb0 + i) * BK, 0, pol_x);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (*s_abort) {
        for (int s = 0; s < STAGES; ++s)
          if (outstanding & (1u << s))
            for (int it = 0; it < (1 << 20); ++it)
              if (mbar_try_wait(&bar_full[s], (issue_phase_bits >> s) & 1u)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        ok = mbar_wait(&bar_full[stage], phase, s_abort, 800 + stage);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
        const uint64_t adesc = umma_desc_kmajor_sw128(sa);
        const uint64_t bdesc = umma_desc_kmajor_sw128(sa + Cfg::A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_f16_ss(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&bar_empty[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && nkb > 0) umma_commit(bar_tfull);
    }
  }

  // ---- phase 1 of the cluster exchange: a member arrives once its accumulator is complete (its ring is then free to
  // receive partial tiles); nobody stores remotely before every member has arrived ----
  if (warp < 2) {
    __syncwarp();
    if (CLUSTER > 1) {
      cluster_arrive();
      cluster_wait();
    }
  }

  if (warp >= 2) {
    pdl_wait();
    if (p.ssq_in) {
      // per-token 1 / rms of the residual stream: the producer accumulated every token's sum of squares in 2^-24 fixed
      // point (integer adds: the order of the CTAs cannot change the result), one load per token
      const int tok = (warp - 2) * 32 + lane;
      if (tok < BLOCK_N && tok < 64) {
        const unsigned long long acc = __ldcg(p.ssq_in + tok);
        s_rstd[tok] = rsqrtf((float)acc * (1.f / 16777216.f) / (float)p.norm_dim + p.norm_eps);
      }
    }
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    bool have = nkb > 0;
    if (have) have = mbar_wait(bar_tfull, 0, s_abort, 900);
    have = __all_sync(0xffffffffu, have);   // warp-uniform: tcgen05.ld is warp-collective
    if (tr && threadIdx.x == 64) { tr[3] = global_timer_ns(); tr[12] = clock64(); }  // accumulator complete
    if (CLUSTER > 1) {
      cluster_arrive();
      cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t recv_local = smem_u32(recv);
    const uint32_t owner = (uint32_t)(row / R);
    const int lr = row - (int)owner * R;
    // slot `crank` of the owner's receive buffer, laid out [token][R rows] fp32: a warp's 32 consecutive rows
    // store 128 contiguous bytes per token, and the owner later reads 8 consecutive rows as two float4
    const uint32_t col_base = recv_local + (uint32_t)((crank * BLOCK_N * R + lr) * 4);
    const uint32_t remote = CLUSTER > 1 ? map_to_cta(col_base, owner) : col_base;
    constexpr int NCH = BLOCK_N / 16;
    const int half = (warp - 2) >> 2;                       // which half of the token chunks this warp moves
    const int ch0 = half == 0 ? 0 : (NCH + 1) / 2;
    const int ch1 = half == 0 ? (NCH + 1) / 2 : NCH;
#pragma unroll 1
    for (int ch = ch0; ch < ch1; ++ch) {
      float v[16];
      if (have) {
        tmem_ld_32x32b_x16(taddr + ch * 16, v);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (ch * 16 + j < p.N)   // tokens past the batch are never read back
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((ch * 16 + j) * R * 4)), "f"(v[j])
                       : "memory");
      }
    }
    tc_fence_before_sync();
    if (tr && threadIdx.x == 64) { tr[4] = global_timer_ns(); tr[13] = clock64(); }  // partials delivered
  }

  // ---- phase 2: every partial slice has been delivered ----
  // Each epilogue thread finishes ITEMS 16-byte groups (8 features of one token). Their residual values do not
  // depend on the cluster, so they are requested between the barrier's arrive and wait.
  constexpr int R8 = R / 8;
  constexpr int ITEMS = (R8 * BLOCK_N + EPI_THREADS - 1) / EPI_THREADS;
  constexpr bool PREFETCH_RES = ITEMS <= 4;     // (more items would not stay in registers)
  uint4 resv[PREFETCH_RES ? ITEMS : 1];
  __syncwarp();
  if (CLUSTER > 1) cluster_arrive();
  if (PREFETCH_RES && warp >= 2 && p.residual && p.vec_ok && (p.ld_res & 7) == 0) {
    const int et = (warp - 2) * 32 + lane;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int idx = et + it * EPI_THREADS;
      const int f8 = idx % R8, tok = idx / R8;
      const int row = (int)crank * R + f8 * 8;
      const int feat = tile_m * BM + row;
      resv[PREFETCH_RES ? it : 0] = make_uint4(0u, 0u, 0u, 0u);
      if (idx < R8 * BLOCK_N && row < BM && feat + 8 <= p.M && tok < p.N)
        resv[PREFETCH_RES ? it : 0] = *reinterpret_cast<const uint4*>(p.residual + (size_t)tok * p.ld_res + feat);
    }
  }
  if (CLUSTER > 1) {
    cluster_wait();
  } else {
    __syncthreads();
  }

  if (tr && threadIdx.x == 64) { tr[5] = global_timer_ns(); tr[8] = clock64(); }    // cluster barrier passed
  if (warp >= 2 && p.ssq_zero && blockIdx.x == 0) {
    // the chain's other accumulator: its consumer finished before this kernel's dependency resolved, its producer
    // starts after this kernel ends
    const int e = (warp - 2) * 32 + lane;
    if (e < 64) p.ssq_zero[e] = 0ull;
  }
  if (PEER && warp >= 2) {
    // ---- cross-rank sum over peer memory, flag-in-data lines: no barrier, no fence, one NVLink hop per shot ----
    const int et = (warp - 2) * 32 + lane;  // 0 .. EPI_THREADS - 1
    const GemmPeerReduce& q = p.peer;
    const int pmode = q.mode;
    const int owner_rank = pmode == 2 ? tile_m % q.world : q.rank;   // two-shot: who finishes this weight tile's rows
    const bool i_finish = pmode != 2 || owner_rank == q.rank;
    const uint32_t counter = q.epochs[blockIdx.x] + 1u;
    // unique per (launch, CTA): a line left behind by another CTA of an earlier launch shape never matches
    const uint32_t epoch = (counter << 9) | ((uint32_t)blockIdx.x & 511u);
    const int ld8 = q.ld >> 3;
    uint4 own[ITEMS];
    // pass 1: deliver this CTA's partial rows (cluster-reduced, rounded to bf16) to the rank(s) that sum them
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int idx = et + it * EPI_THREADS;
      const int f8 = idx % R8, tok = idx / R8;
      const int row = (int)crank * R + f8 * 8;
      const int feat = tile_m * BM + row;
      own[it] = make_uint4(0u, 0u, 0u, 0u);
      if (idx >= R8 * BLOCK_N || row >= BM || feat >= p.M || tok >= p.N) continue;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int src = 0; src < CLUSTER; ++src) {
        const float4* rp = reinterpret_cast<const float4*>(recv + ((size_t)src * BLOCK_N + tok) * R + f8 * 8);
        const float4 a0 = rp[0], a1 = rp[1];
        acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
        acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
      }
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&own[it]);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      const size_t line = (((size_t)q.rank * q.cap + tok) * ld8 + (feat >> 3)) * 2;
      const uint4 l0 = make_uint4(own[it].x, epoch, own[it].y, epoch);
      const uint4 l1 = make_uint4(own[it].z, epoch, own[it].w, epoch);
      if (pmode == 2) {
        if (!i_finish) {
          st_line(q.slots[owner_rank] + line, l0);
          st_line(q.slots[owner_rank] + line + 1, l1);
        }
      } else {
#pragma unroll
        for (int r = 1; r < 8; ++r) {
          if (r < q.world) {
            uint4* dst = q.slots[(q.rank + r) % q.world] + line;
            st_line(dst, l0);
            st_line(dst + 1, l1);
          }
        }
      }
    }
    // pass 2: sum in rank order (bit-identical on every rank), add the residual, store; or take the owner's rows
    bool failed = false;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int idx = et + it * EPI_THREADS;
      const int f8 = idx % R8, tok = idx / R8;
      const int row = (int)crank * R + f8 * 8;
      const int feat = tile_m * BM + row;
      float ss = 0.f;
      const bool valid = !(idx >= R8 * BLOCK_N || row >= BM || feat >= p.M || tok >= p.N);
      if (valid && !failed) {
        const size_t off = (size_t)tok * p.ldd + feat;
        uint4 o;
        if (i_finish) {
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {        // peers 0-3, then 4-7: the sum runs in rank order on every rank
            if (h * 4 < q.world && !failed) {
              uint4 u[4];
              const uint4* bases[4];
              uint32_t need = 0;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int r = h * 4 + k;
                bases[k] = q.slots[q.rank] + (((size_t)r * q.cap + tok) * ld8 + (feat >> 3)) * 2;
                if (r < q.world && r != q.rank) need |= 1u << k;
              }
              failed = !ld_lines_all(bases, need, epoch, u, 1100, q.rank, h * 4);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int r = h * 4 + k;
                if (r < q.world && !failed) {
                  const uint4 v = (r == q.rank) ? own[it] : u[k];
                  const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 t = __bfloat1622float2(uh[j]);
                    acc[2 * j] += t.x;
                    acc[2 * j + 1] += t.y;
                  }
                }
              }
            }
          }
          if (p.residual) {
            const uint4 rr = PREFETCH_RES ? resv[PREFETCH_RES ? it : 0]
                                          : *reinterpret_cast<const uint4*>(p.residual + (size_t)tok * p.ld_res + feat);
            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = __bfloat1622float2(rh[j]);
              acc[2 * j] += t.x;
              acc[2 * j + 1] += t.y;
            }
          }
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          if (pmode == 2 && !failed) {
            const size_t line = ((size_t)tok * ld8 + (feat >> 3)) * 2;
            const uint4 l0 = make_uint4(o.x, epoch, o.y, epoch);
            const uint4 l1 = make_uint4(o.z, epoch, o.w, epoch);
#pragma unroll
            for (int r = 1; r < 8; ++r) {
              if (r < q.world) {
                uint4* dst = q.result[(q.rank + r) % q.world] + line;
                st_line(dst, l0);
                st_line(dst + 1, l1);
              }
            }
          }
        } else {
          failed = !ld_lines(q.result[q.rank] + ((size_t)tok * ld8 + (feat >> 3)) * 2, epoch, o, 1200, q.rank, owner_rank);
        }
        if (!failed) {
          *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + off) = o;
          const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 t = __bfloat1622float2(oh[j]);
            ss += t.x * t.x + t.y * t.y;
          }
        }
      }
      if (p.ssq_out && idx < R8 * BLOCK_N) {   // warp-uniform (R8 * BLOCK_N is a multiple of 32)
        for (int o2 = 1; o2 < R8; o2 <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
        if (f8 == 0 && valid) atomicAdd(p.ssq_out + tok, ssq_fixed(ss));
      }
    }
    epi_bar_sync();     // every thread has read its epoch
    if (et == 0) q.epochs[blockIdx.x] = counter;
  } else if (warp >= 2) {
    const int et = (warp - 2) * 32 + lane;  // 0 .. EPI_THREADS - 1
    const bool res_vec = PREFETCH_RES && p.residual && p.vec_ok && (p.ld_res & 7) == 0;
#pragma unroll(ITEMS < 4 ? ITEMS : 4)
    for (int it = 0; it < ITEMS; ++it) {
      const int idx = et + it * EPI_THREADS;
      const int f8 = idx % R8;         // consecutive threads -> consecutive 16-byte feature groups of one token
      const int tok = idx / R8;
      const int row = (int)crank * R + f8 * 8;
      const int feat = tile_m * BM + row;
      float ss = 0.f;
      const bool valid = idx < R8 * BLOCK_N && row < BM && feat < p.M && tok < p.N;
      if (valid) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int src = 0; src < CLUSTER; ++src) {
          const float4* rp = reinterpret_cast<const float4*>(recv + ((size_t)src * BLOCK_N + tok) * R + f8 * 8);
          const float4 a0 = rp[0], a1 = rp[1];
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
          acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
        }
        if (p.ssq_in) {
          const float rs = s_rstd[tok];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] *= rs;
        }
        if (tr && threadIdx.x == 64 && it == 0) tr[9] = clock64();    // first item summed
        const int nvalid = min(8, p.M - feat);
        const size_t off = (size_t)tok * p.ldd + feat;
        const bool vec = p.vec_ok && nvalid == 8 && ((p.ldd & 7) == 0) && ((feat & 7) == 0) && (!p.residual || (p.ld_res & 7) == 0);   // gated pairs: ldd % 8 == 0 keeps the 8-byte stores aligned
        if (vec) {
          if (p.bias) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + feat));
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = __bfloat1622float2(bh[j]);
              acc[2 * j] += t.x;
              acc[2 * j + 1] += t.y;
            }
          }
          if (p.act >= SWB_ACT_SWIGLU_PAIRS) {
            // rows come in (gate, up) pairs: four gated outputs, one 8-byte store
            const int a1 = p.act == SWB_ACT_SWIGLU_PAIRS ? SWB_ACT_SILU : SWB_ACT_GELU_TANH;
            uint2 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
            oh[0] = __floats2bfloat162_rn(act_apply(acc[0], a1) * acc[1], act_apply(acc[2], a1) * acc[3]);
            oh[1] = __floats2bfloat162_rn(act_apply(acc[4], a1) * acc[5], act_apply(acc[6], a1) * acc[7]);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (size_t)tok * p.ldd + (feat >> 1)) = o;
          } else {
            if (p.act != SWB_ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = act_apply(acc[j], p.act);
            }
            if (p.residual) {
              const uint4 r = res_vec ? resv[PREFETCH_RES ? it : 0]
                                      : *reinterpret_cast<const uint4*>(p.residual + (size_t)tok * p.ld_res + feat);
              const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 t = __bfloat1622float2(rh[j]);
                acc[2 * j] += t.x;
                acc[2 * j + 1] += t.y;
              }
            }
            if (p.out_fp32) {
              float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off);
              op[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
              op[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            } else {
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
              *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + off) = o;
              if (p.ssq_out) {   // sum of squares of exactly what was stored (bf16-rounded)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 t = __bfloat1622float2(oh[j]);
                  ss += t.x * t.x + t.y * t.y;
                }
              }
            }
          }
        } else if (p.act >= SWB_ACT_SWIGLU_PAIRS) {
          const int a1 = p.act == SWB_ACT_SWIGLU_PAIRS ? SWB_ACT_SILU : SWB_ACT_GELU_TANH;
          for (int j = 0; j + 1 < nvalid; j += 2) {
            const float gte = acc[j] + (p.bias ? __bfloat162float(p.bias[feat + j]) : 0.f);
            const float up = acc[j + 1] + (p.bias ? __bfloat162float(p.bias[feat + j + 1]) : 0.f);
            reinterpret_cast<bf16*>(p.out)[(size_t)tok * p.ldd + ((feat + j) >> 1)] = __float2bfloat16(act_apply(gte, a1) * up);
          }
        } else {
          for (int j = 0; j < nvalid; ++j) {
            float x = act_apply(acc[j] + (p.bias ? __bfloat162float(p.bias[feat + j]) : 0.f), p.act);
            if (p.residual) x += __bfloat162float(p.residual[(size_t)tok * p.ld_res + feat + j]);
            if (p.out_fp32)
              reinterpret_cast<float*>(p.out)[off + j] = x;
            else
              reinterpret_cast<bf16*>(p.out)[off + j] = __float2bfloat16(x);
          }
        }
      }
      if (tr && threadIdx.x == 64 && it == 0) tr[10] = clock64();     // first item stored
      if (p.ssq_out && idx < R8 * BLOCK_N) {   // warp-uniform (R8 * BLOCK_N is a multiple of 32)
        for (int o2 = 1; o2 < R8; o2 <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
        if (f8 == 0 && valid) atomicAdd(p.ssq_out + tok, ssq_fixed(ss));
      }
      if (tr && threadIdx.x == 64 && it == 0) tr[14] = clock64();     // first item's sum of squares sent
    }
  }

  if (tr && threadIdx.x == 64) { tr[6] = global_timer_ns(); tr[11] = clock64(); }    // outputs stored
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (tr && threadIdx.x == 0) tr[7] = global_timer_ns();
}

template <int BLOCK_N, int CLUSTER, int STAGES_, bool PEER>
int launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  using Cfg = DecCfg<BLOCK_N, STAGES_>;
  auto kern = gemm_decode_cluster_kernel<BLOCK_N, CLUSTER, STAGES_, PEER>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.tiles_m * CLUSTER);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (CLUSTER > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = CLUSTER;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return e == cudaSuccess ? 0 : -(int)e;
}

template <int BLOCK_N, int STAGES_>
int launch_cluster(int cluster, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t s) {
  if (p.peer.mode) {          // the cross-rank epilogue runs with 1, 2, 4 or 8 members (see the launch checks)
    switch (cluster) {
      case 1: return launch_one<BLOCK_N, 1, STAGES_, true>(tw, tx, p, s);
      case 2: return launch_one<BLOCK_N, 2, STAGES_, true>(tw, tx, p, s);
      case 4: return launch_one<BLOCK_N, 4, STAGES_, true>(tw, tx, p, s);
      case 8: return launch_one<BLOCK_N, 8, STAGES_, true>(tw, tx, p, s);
    }
    return -2;
  }
  switch (cluster) {
    case 1: return launch_one<BLOCK_N, 1, STAGES_, false>(tw, tx, p, s);
    case 2: return launch_one<BLOCK_N, 2, STAGES_, false>(tw, tx, p, s);
    case 3: return launch_one<BLOCK_N, 3, STAGES_, false>(tw, tx, p, s);
    case 4: return launch_one<BLOCK_N, 4, STAGES_, false>(tw, tx, p, s);
    case 6: return launch_one<BLOCK_N, 6, STAGES_, false>(tw, tx, p, s);
    case 8: return launch_one<BLOCK_N, 8, STAGES_, false>(tw, tx, p, s);
  }
  return -2;
}
template <int BLOCK_N>
int launch_stages(bool deep, int cluster, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p,
                  cudaStream_t s) {
  return deep ? launch_cluster<BLOCK_N, 8>(cluster, tw, tx, p, s) : launch_cluster<BLOCK_N, 4>(cluster, tw, tx, p, s);
}

}  // namespace

// Returns 1 when the cluster kernel takes this problem (T <= 64), 0 when the caller should use the general kernel.
int gemm_decode_cluster_supported(int T) { return T >= 1 && T <= 64; }

int gemm_decode_cluster_launch(const GemmArgs& a, int force_cluster, cudaStream_t stream) {
  const int sms = device_sm_count();
  const int block_n = a.T <= 16 ? 16 : a.T <= 32 ? 32 : 64;
  GemmParams p{};
  p.M = a.N;
  p.N = a.T;
  p.K = a.K;
  p.kblocks_total = (a.K + BK - 1) / BK;
  p.tiles_m = (a.N + BM - 1) / BM;
  p.tiles_n = 1;
  p.transposed = 1;
  p.stream_a = 1;
  p.ldd = a.ldd;
  p.out = a.D;
  p.out_fp32 = a.out_fp32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ld_res = a.ld_res;
  p.act = a.act;
  p.ssq_out = reinterpret_cast<unsigned long long*>(a.ssq_out);
  p.ssq_in = reinterpret_cast<const unsigned long long*>(a.ssq_in);
  p.ssq_zero = reinterpret_cast<unsigned long long*>(a.ssq_zero);
  p.norm_dim = a.norm_dim;
  p.norm_eps = a.norm_eps;
  p.trace = gemm_trace_buffer();
  if (a.peer && a.peer->mode) p.peer = *a.peer;
  p.vec_ok = ((reinterpret_cast<uintptr_t>(a.D) & 15) == 0) && (!a.bias || (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0) &&
             (!a.residual || (reinterpret_cast<uintptr_t>(a.residual) & 15) == 0) && (!a.out_fp32 || (a.ldd % 4) == 0);
  // Two CTAs can be resident per SM. Measured on B200 over Llama-3-8B projections: the fastest member count is
  // the largest one that keeps the grid under ~1.75 CTAs per SM with at least 6 k-blocks per member.
  int cluster = 1;
  // Small projections (default: up to 24 MB of weights): as many members per cluster as keep the grid within one CTA
  // per SM; up to 16 MB with the 8-stage ring. Larger ones: two CTAs per SM, grid under ~1.75 CTAs per SM, 4 stages.
  // Measured on Llama-3-8B decode steps (batch 64): the 8-stage ring fills the SM, so the next kernel's CTAs cannot
  // become resident and request their own weights before this kernel ends; that costs more than the deeper ring
  // gains once a projection streams tens of megabytes (unsharded step 5.06 ms with 4 stages, 5.40 ms with 8 stages
  // on the 50 MB qkv projection), and gains about 5 % on the shard shapes of 8-way tensor parallelism.
  static const long deep_mb = [] {
    const char* e = getenv("SWB_DEC_DEEP_MB");
    return e ? atol(e) : 24L;
  }();
  static const long stages8_mb = [] {
    const char* e = getenv("SWB_DEC_STAGES8_MB");
    return e ? atol(e) : 16L;
  }();
  const long wbytes = (long)a.N * a.K * 2;
  const bool one_per_sm = wbytes <= deep_mb * (1L << 20) && p.tiles_m <= sms;
  bool deep = one_per_sm && wbytes <= stages8_mb * (1L << 20);
  for (int c : {2, 3, 4, 6, 8}) {
    if (one_per_sm ? (long)p.tiles_m * c > sms : (long)p.tiles_m * c * 4 > 7L * sms) break;
    if (p.kblocks_total / c < 4 && c > 2) break;
    if (p.kblocks_total / c < 2) break;
    cluster = c;
  }
  if (force_cluster > 0) {
    cluster = std::min(8, force_cluster);
    deep = deep && (long)p.tiles_m * cluster <= sms;
  }
  if (cluster == 5) cluster = 4;
  if (cluster == 7) cluster = 6;
  if (p.peer.mode) {
    // the cross-rank sum moves whole 16-byte groups of a full 128-row tile grid, bf16 in and out, nothing else fused;
    // at most 4 members per cluster keep a token's run of peer stores at 64 bytes or more
    const GemmPeerReduce& q = p.peer;
    if (q.world < 2 || q.world > 8 || q.rank < 0 || q.rank >= q.world || (q.mode != 1 && q.mode != 2)) return -3;
    if (a.bias || a.act != SWB_ACT_NONE || a.out_fp32 || a.ssq_in || !p.vec_ok || (a.ldd & 7) || (a.N % BM) ||
        (q.ld & 7) || (a.residual && (a.ld_res & 7)))
      return -3;
    if (q.mode == 2 && p.tiles_m < q.world) p.peer.mode = 1;   // every rank must own a tile for the lines to order buffer reuse
    if (a.T > q.cap) return -3;
    if (cluster == 3) cluster = 2;
    if (cluster == 6) cluster = 4;
    if (p.tiles_m * cluster > SWB_PEER_MAX_CTAS) return -3;
  }
  if (a.ssq_out) {
    // the per-token reduction in the producer's epilogue pairs lanes by xor: rows per member / 8 must be a power of two
    if (cluster == 3) cluster = 2;
    if (cluster == 6) cluster = 4;
    if (a.N % BM != 0 || a.out_fp32) return -3;
  }
  if ((a.ssq_out || a.ssq_in) && (!p.vec_ok || (a.ldd & 7) != 0)) return -3;
  CUtensorMap tw, tx;
  int r = make_tmap_bf16_2d(&tw, a.W, a.N, a.K, a.ldw, BM);
  if (r) return r;
  r = make_tmap_bf16_2d(&tx, a.A, a.T, a.K, a.lda, block_n);
  if (r) return r;
  switch (block_n) {
    case 16: return launch_stages<16>(deep, cluster, tw, tx, p, stream);
    case 32: return launch_stages<32>(deep, cluster, tw, tx, p, stream);
    default: return launch_stages<64>(deep, cluster, tw, tx, p, stream);
  }
}

}  // namespace swb
