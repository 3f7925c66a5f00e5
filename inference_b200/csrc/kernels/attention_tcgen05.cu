// Dense (non-causal) flash attention on the 5th-generation tensor cores, head dim 128, bf16 in / bf16 out.
//
// One CTA owns 256 query rows of one head (two 128-row tiles, "q0" and "q1") and walks the keys in tiles of 128.
//   warp 8 (one lane)   TMA producer: Q once, then K and V tiles through two 2-stage rings (4-D tensor maps over
//                       [d, head, token, batch], 64-column boxes, 128-byte swizzle).
//   warp 9 (one lane)   tcgen05.mma issuer. S_q = Q_q K^T accumulates into TMEM; O_q += P_q V reads P from TMEM
//                       (P overwrites the first half of S in place as packed bf16) and V from shared memory as an
//                       MN-major operand, so V needs no transpose. Issue order
//                           S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) ...
//                       keeps the tensor pipe busy with one tile's MMAs while the other tile is in softmax.
//   warps 0-3 / 4-7     softmax warpgroups for q0 / q1: thread = row. tcgen05.ld the S row, running max with lazy
//                       rescale (O is only rescaled when the max grew by more than 2^8), exp2, tcgen05.st of P.
// TMEM map (512 columns): [0,128) S0/P0, [128,256) O0, [256,384) S1/P1, [384,512) O1.
// It replaces the mma.sync kernel for the FLUX joint attention (reference: candle-gen-flux/src/ip_dit.rs:64-85 runs
// SDPA through cuBLAS matmuls + softmax, or FlashAttention-2 sm80 kernels).
// Every wait is bounded; on expiry the CTA raises its abort flag, drains its own copies, frees TMEM and returns.
#include "attention_common.cuh"
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

namespace swb {

SWB_REGISTER_STATUS_UNIT(attention_tcgen05);

namespace {

constexpr int BM = 128;          // query rows per tile (two tiles per CTA)
constexpr int BN = 128;          // keys per tile
constexpr int KV_STAGES = 2;
constexpr int THREADS = 320;
constexpr uint32_t ATOM_BYTES = BM * 64 * 2;       // 16 KB: 128 rows of one 64-column swizzle atom
// Head dim 128 (two swizzle atoms per tile) or 64 (one atom: half the shared memory and half the MMA work of the padded path).
template <int HD>
struct FaCfg {
  static_assert(HD == 64 || HD == 128, "head dim 64 or 128");
  static constexpr int ATOMS = HD / 64;
  static constexpr uint32_t TILE_BYTES = BM * HD * 2;
  static constexpr uint32_t SMEM_Q = 0;                                   // 2 tiles
  static constexpr uint32_t SMEM_K = 2 * TILE_BYTES;                      // KV_STAGES tiles
  static constexpr uint32_t SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
  static constexpr uint32_t SMEM_BAR = SMEM_V + KV_STAGES * TILE_BYTES;
  static constexpr size_t SMEM_BYTES = SMEM_BAR + 256 + 1024 /*alignment slack*/;
  static constexpr int ROW_BYTES = HD * 2;                                // one output row of one head
  static constexpr int CHUNKS = ROW_BYTES / 16;                           // 16-byte chunks per row
};
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S0 = 0, COL_O0 = 128, COL_S1 = 256, COL_O1 = 384;
constexpr float RESCALE_THRESHOLD = 8.f;           // in log2 units

// Sequence-parallel return path: query row g (global token index, batch 1) belongs to rank
// (g < split ? g / n0 : (g - split) / n1) at local row (g < split ? g % n0 : n0 + (g - split) % n1); the output row is
// stored straight into that rank's buffer at column col_offset + head * 128.
struct OutScatter {
  bf16* peer[8];
  int enabled, split, n0, n1, col_offset;
};

struct FaParams {
  OutScatter scatter;
  bf16* out;
  long long out_stride_tok;   // elements; token index = b * q_len + s
  int q_len, kv_len, Hq, Hkv;
  float scale_log2;
  int tiles;   // query tiles per CTA: 2 (MMAs of one tile overlap the softmax of the other) or 1 (twice the CTAs)
  int causal;  // key j attends to query i only if j <= i (sequences start at position 0: fresh prefill)
  const int* cu_q;   // optional [num_seqs + 1] token offsets: blockIdx.z is then a sequence of a packed batch
  // Paged keys / values (prefill on top of earlier context): tmap_k / tmap_v then describe the page pool
  // [page, kv head, row in page, d]; sequence z owns pages block_table[z * max_blocks + i] and kv_lens[z] keys, and
  // its queries are the last q_len of those positions (bottom-right aligned causal mask). Needs cu_q.
  const int* kv_lens;
  const int* block_table;
  int max_blocks, block_size;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// D[tmem] (+)= A[tmem, packed bf16] * B[smem desc]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// V tile as the B operand of O += P V: rows are keys (the MMA K dimension), 64 head-dim columns per 128-byte row
// (MN-major), 8-key groups 1024 bytes apart, the second 64-column block one atom (16 KB) further.
__device__ __forceinline__ uint64_t umma_desc_mnmajor_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(ATOM_BYTES >> 4) << 16;   // leading byte offset: next 64-element block along N
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset: next 8-row group along K
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// 32 consecutive 32-bit columns of this thread's TMEM lane (no wait inside).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2];   // MMA -> softmax q: S_q of the current key tile is complete
  uint64_t p_full[2];   // softmax q -> MMA: P_q is in TMEM (128 arrivals)
  uint64_t o_final;     // every MMA of the CTA has completed
  uint32_t tmem_base;
  int abort;
};

// 168 registers per thread is the cap for ten warps: two of the four scheduler partitions hold three warps, and a
// partition's file is 16 K registers (a build with 200 registers per thread does not launch).
template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_dense_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using C = FaCfg<HD>;
  constexpr uint32_t TILE_BYTES = C::TILE_BYTES, SMEM_Q = C::SMEM_Q, SMEM_K = C::SMEM_K, SMEM_V = C::SMEM_V, SMEM_BAR = C::SMEM_BAR;
  constexpr int ATOMS = C::ATOMS, ROW_BYTES = C::ROW_BYTES, CHUNKS = C::CHUNKS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + SMEM_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_base = blockIdx.x * (p.tiles * BM);
  const int head = blockIdx.y;
  // packed variable-length batch: this CTA's sequence covers tokens [tok0, tok0 + q_len) of one flat token axis
  const int tok0 = p.cu_q ? p.cu_q[blockIdx.z] : 0;
  const int q_len = p.cu_q ? p.cu_q[blockIdx.z + 1] - tok0 : p.q_len;
  const bool paged = p.block_table != nullptr;
  const int kv_len = paged ? p.kv_lens[blockIdx.z] : (p.cu_q ? q_len : p.kv_len);
  const int coff = paged ? max(kv_len - q_len, 0) : 0;   // position of query 0 among the sequence's keys
  const int batch = p.cu_q ? 0 : blockIdx.z;
  if (q_base >= q_len || kv_len <= 0) return;   // uniform for the whole CTA, before any barrier or TMEM allocation
  const int kv_head = head / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(kv_len, q_base + p.tiles * BM + coff) : kv_len;
  const int n_tiles = (kv_end + BN - 1) / BN;
  volatile int* abort_flag = &bars->abort;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&bars->s_full[q], 1);
      mbar_init(&bars->p_full[q], BM);
    }
    mbar_init(&bars->o_final, 1);
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->q_full, p.tiles * TILE_BYTES);
      for (int q = 0; q < p.tiles; ++q)
        for (int a = 0; a < ATOMS; ++a)
          tma_load_4d(smem + SMEM_Q + q * TILE_BYTES + a * ATOM_BYTES, &tmap_q, &bars->q_full, a * 64, head,
                      tok0 + q_base + q * BM, batch);
      bool ok = true;
      int issued_k = 0, issued_v = 0;
      // paged: a tile is BN / block_size pages, each a box of block_size rows that lands at its place in the swizzled
      // tile (a page is a whole number of 8-row swizzle groups); tiles past the last page repeat it, masked below
      const int* pages = paged ? p.block_table + (long long)blockIdx.z * p.max_blocks : nullptr;
      const int per_tile = paged ? BN / p.block_size : 1, last_page = paged ? (kv_len - 1) / p.block_size : 0;
      const uint32_t page_bytes = paged ? (uint32_t)p.block_size * 128u : 0u;
      auto load_tile = [&](uint32_t dst_off, const CUtensorMap* map, uint64_t* bar, int j) {
        if (!paged) {
          for (int a = 0; a < ATOMS; ++a)
            tma_load_4d(smem + dst_off + a * ATOM_BYTES, map, bar, a * 64, kv_head, tok0 + j * BN, batch);
          return;
        }
        for (int g = 0; g < per_tile; ++g) {
          const int page = pages[min(j * per_tile + g, last_page)];
          for (int a = 0; a < ATOMS; ++a)
            tma_load_4d(smem + dst_off + a * ATOM_BYTES + g * page_bytes, map, bar, a * 64, 0, kv_head, page);
        }
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        ok = mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, 10);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->k_full[s], TILE_BYTES);
        load_tile(SMEM_K + s * TILE_BYTES, &tmap_k, &bars->k_full[s], j);
        issued_k = j + 1;
        ok = mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, 11);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars->v_full[s], TILE_BYTES);
        load_tile(SMEM_V + s * TILE_BYTES, &tmap_v, &bars->v_full[s], j);
        issued_v = j + 1;
      }
      if (!ok) {
        // drain: every copy this thread started must land before the CTA's shared memory is released
        volatile int never = 0;
        mbar_wait(&bars->q_full, 0, &never, 12);
        for (int j = max(0, issued_k - KV_STAGES); j < issued_k; ++j)
          mbar_wait(&bars->k_full[j % KV_STAGES], (j / KV_STAGES) & 1, &never, 13);
        for (int j = max(0, issued_v - KV_STAGES); j < issued_v; ++j)
          mbar_wait(&bars->v_full[j % KV_STAGES], (j / KV_STAGES) & 1, &never, 14);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16_f32(BM, BN);
      constexpr uint32_t IDESC_PV = umma_idesc_bf16_f32(BM, HD) | (1u << 16);   // B is MN-major
      const uint32_t col_s[2] = {COL_S0, COL_S1}, col_o[2] = {COL_O0, COL_O1};
      const uint32_t q_addr = smem_u32(smem + SMEM_Q), k_addr = smem_u32(smem + SMEM_K),
                     v_addr = smem_u32(smem + SMEM_V);
      auto issue_qk = [&](int q, int s) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM_BYTES + (k & 3) * 32;
          umma_f16_ss(tmem + col_s[q], umma_desc_kmajor_sw128(q_addr + q * TILE_BYTES + off),
                      umma_desc_kmajor_sw128(k_addr + s * TILE_BYTES + off), IDESC_QK, k > 0);
        }
        umma_commit(&bars->s_full[q]);
      };
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, 20);
      if (ok) ok = mbar_wait(&bars->k_full[0], 0, abort_flag, 21);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0, 0);
        if (p.tiles == 2) issue_qk(1, 0);
        umma_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % KV_STAGES, sn = (j + 1) % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1, phn = ((j + 1) / KV_STAGES) & 1;
        ok = mbar_wait(&bars->v_full[s], ph, abort_flag, 22);
        if (ok && j + 1 < n_tiles) ok = mbar_wait(&bars->k_full[sn], phn, abort_flag, 23);
        for (int q = 0; q < p.tiles && ok; ++q) {
          ok = mbar_wait(&bars->p_full[q], j & 1, abort_flag, 24 + q);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            umma_f16_ts(tmem + col_o[q], tmem + col_s[q] + k * 8,
                        umma_desc_mnmajor_sw128(v_addr + s * TILE_BYTES + k * 2048), IDESC_PV, (j > 0) || (k > 0));
          const bool last_q = (q == p.tiles - 1);
          if (last_q) umma_commit(&bars->v_empty[s]);
          if (j + 1 < n_tiles) {
            issue_qk(q, sn);
            if (last_q) umma_commit(&bars->k_empty[sn]);
          }
        }
      }
      umma_commit(&bars->o_final);   // also on the abort path: it only tracks MMAs already issued
      if (!ok) {                     // TMEM must not be freed under MMAs that are still running
        volatile int never = 0;
        mbar_wait(&bars->o_final, 0, &never, 27);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups (thread = query row)
    const int q = warp >> 2;
    const int my_tiles = (q < p.tiles) ? n_tiles : 0;   // the second warpgroup idles in one-tile mode
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + (q ? COL_S1 : COL_S0);
    const uint32_t t_o = tmem + lane_base + (q ? COL_O1 : COL_O0);
    const int row = q_base + q * BM + (warp & 3) * 32 + lane;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_tiles; ++j) {
      ok = mbar_wait(&bars->s_full[q], j & 1, abort_flag, 30 + q);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld_x32(t_s + c * 32, s + c * 32);
      tmem_ld_wait();
      // keys past the sequence (zero fill, or the next sequence of a packed batch) and, when causal, keys after the
      // query position never contribute
      if ((j + 1) * BN > kv_len || (p.causal && (j + 1) * BN > q_base + q * BM + coff)) {
        const int last_key = p.causal ? min(kv_len - 1, row + coff) : kv_len - 1;
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if (j * BN + i > last_key) s[i] = __float_as_uint(-INFINITY);
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(s[i]));
        mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(s[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
      }
      const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m_used);
      const bool grow = (m_new - m_used) * p.scale_log2 > RESCALE_THRESHOLD;   // true on the first tile (m_used = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float f = grow ? ex2((m_used - m_new) * p.scale_log2) : 1.f;      // -inf -> 0 on the first tile
        if (grow) {
          l *= f;
          m_used = m_new;
        }
        if (j > 0) {   // O holds nothing before the first PV
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_x32(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st_x32(t_o + c * 32, o);
          }
        }
      }
      const float neg_m = -m_used * p.scale_log2;
      float l0 = 0.f, l1 = 0.f;
      // (Measured alternatives for this loop, all slower on B200: every 4th / 2nd exponential as a cubic on the FMA pipe
      // -8 % / -17 %; pairs of exponentials as one bf16x2 special-function operation -6 %; three-input max with
      // two-lane fp32 multiply-add and add -30 %, from register-pair moves and spills. The loop is issue-bound.)
#pragma unroll
      for (int i = 0; i < BN; i += 2) {   // packed P overwrites the row in place (index i/2 <= i)
        const float e0 = ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, neg_m));
        const float e1 = ex2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, neg_m));
        l0 += e0;
        l1 += e1;
        s[i >> 1] = pack_bf16x2(e0, e1);
      }
      l += l0 + l1;
      tmem_st_x32(t_s, s);
      tmem_st_x32(t_s + 32, s + 32);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars->p_full[q]);
    }
    if (ok && my_tiles > 0) ok = mbar_wait(&bars->o_final, 0, abort_flag, 32 + q);
    if (ok && my_tiles > 0) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      // Stage this warp's 32 rows x HD columns in the (now idle) Q region, then write every row's HD * 2 bytes with
      // HD / 8 lanes x 16 bytes: contiguous runs for local stores and for stores that cross NVLink alike.
      // 16-byte chunk c of row r sits at c ^ (r & 7).
      uint8_t* slab = smem + SMEM_Q + warp * (32 * ROW_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(t_o + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
          u.y = pack_bf16x2(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
          u.z = pack_bf16x2(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
          u.w = pack_bf16x2(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(slab + lane * ROW_BYTES + (((c * 4 + v) ^ (lane & 7)) << 4)) = u;
        }
      }
      __syncwarp();
      const int row0 = q_base + q * BM + (warp & 3) * 32;
#pragma unroll 4
      for (int it = 0; it < CHUNKS; ++it) {            // CHUNKS lanes write one row: 32 / CHUNKS rows per pass
        const int r = (32 / CHUNKS) * it + lane / CHUNKS, ch = lane % CHUNKS;
        const int grow = row0 + r;
        if (grow < q_len) {
          const uint4 val = *reinterpret_cast<const uint4*>(slab + r * ROW_BYTES + ((ch ^ (r & 7)) << 4));
          bf16* dst = p.out + ((long long)batch * p.q_len + tok0 + grow) * p.out_stride_tok + (long long)head * HD;
          if (p.scatter.enabled) {
            const OutScatter& sc = p.scatter;
            const int g2 = grow - sc.split;
            const int rk = grow < sc.split ? grow / sc.n0 : g2 / sc.n1;
            const int local = grow < sc.split ? grow % sc.n0 : sc.n0 + g2 % sc.n1;
            dst = sc.peer[rk] + (long long)local * p.out_stride_tok + sc.col_offset + head * HD;
          }
          *reinterpret_cast<uint4*>(dst + ch * 8) = val;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct Map4Key {
  const void* ptr;
  long long s1, s2, s3;
  int d1, d2, d3;
  bool operator==(const Map4Key& o) const {
    return ptr == o.ptr && s1 == o.s1 && s2 == o.s2 && s3 == o.s3 && d1 == o.d1 && d2 == o.d2 && d3 == o.d3;
  }
};
struct Map4Hash {
  size_t operator()(const Map4Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    for (long long v : {k.s1, k.s2, k.s3, (long long)k.d1, (long long)k.d2, (long long)k.d3}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// bf16 [batch, tokens, heads, 128] with element strides (tok, head, batch): dims (128, heads, tokens, batch),
// box (64, 1, 128, 1), 128-byte swizzle, zero fill outside.
// With page_rows > 0 the tensor is a page pool [batch = pages, heads, page_rows, 128] (contiguous): dims
// (128, page_rows, heads, pages), box (64, page_rows, 1, 1); `tokens` and the strides are then unused.
int make_tmap_heads(CUtensorMap* out, const void* ptr, int hd, int heads, int tokens, int batch, long long stride_head,
                    long long stride_tok, long long stride_batch, int page_rows = 0) {
  static std::mutex mu;
  static std::unordered_map<Map4Key, CUtensorMap, Map4Hash> cache;
  if (page_rows > 0) {
    tokens = -page_rows;
    stride_head = (long long)page_rows * hd;
    stride_tok = hd;
    stride_batch = (long long)heads * page_rows * hd;
  }
  Map4Key key{ptr, stride_head, stride_tok, stride_batch, heads * 1024 + hd, tokens, batch};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)tokens, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_tok * 2, (cuuint64_t)stride_batch * 2};
  cuuint32_t box[4] = {64u, 1u, (cuuint32_t)BM, 1u};
  if (page_rows > 0) {
    dims[1] = (cuuint64_t)page_rows;
    dims[2] = (cuuint64_t)heads;
    strides[0] = (cuuint64_t)stride_tok * 2;
    strides[1] = (cuuint64_t)stride_head * 2;
    box[1] = (cuuint32_t)page_rows;
    box[2] = 1u;
  }
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 1000;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace

int g_force_tiles = 0;   // 0: choose per problem; 1 / 2: fixed query tiles per CTA (comparison runs)
void attn_dense_tcgen05_set_tiles(int tiles) { g_force_tiles = tiles; }

// Returns 1 when the tcgen05 kernel handles this problem, 0 otherwise.
int attn_dense_tcgen05_supported(const void* q, const void* k, const void* v, long long q_stride_tok, int q_stride_head,
                                 long long kv_stride_tok, int kv_stride_head, long long out_stride_tok, int D,
                                 int causal) {
  if (D != 128 && D != 64) return 0;
  (void)causal;   // causal problems are supported when queries and keys cover the same positions (checked by callers)
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return 0;
  if ((q_stride_tok | q_stride_head | kv_stride_tok | kv_stride_head | out_stride_tok) % 8) return 0;
  return 1;
}

int attn_dense_tcgen05_launch(const void* q, long long q_stride_tok, int q_stride_head, const void* k, const void* v,
                              long long kv_stride_tok, int kv_stride_head, void* out, long long out_stride_tok,
                              int batch, int q_len, int kv_len, int Hq, int Hkv, float scale, cudaStream_t stream,
                              void* const* peers, int world, int split, int n0, int n1, int col_offset, int causal,
                              const int* cu_q, int total_tokens, int head_dim, const int* kv_lens,
                              const int* block_table, int max_blocks, int block_size, int num_blocks) {
  if (head_dim != 64 && head_dim != 128) return -3;
  const bool paged = block_table != nullptr;
  if (paged && (head_dim != 128 || !cu_q || !kv_lens || block_size < 8 || block_size % 8 || BN % block_size ||
                num_blocks <= 0 || max_blocks <= 0 || peers))
    return -3;
  CUtensorMap tq, tk, tv;
  // packed batches address one flat token axis (batch = the number of sequences only sizes the grid)
  const int map_q_tokens = cu_q ? total_tokens : q_len, map_kv_tokens = cu_q ? total_tokens : kv_len;
  const int map_batch = cu_q ? 1 : batch;
  int rc = make_tmap_heads(&tq, q, head_dim, Hq, map_q_tokens, map_batch, q_stride_head, q_stride_tok, q_stride_tok * map_q_tokens);
  if (rc) return rc;
  rc = make_tmap_heads(&tk, k, head_dim, Hkv, map_kv_tokens, paged ? num_blocks : map_batch, kv_stride_head,
                       kv_stride_tok, kv_stride_tok * map_kv_tokens, paged ? block_size : 0);
  if (rc) return rc;
  rc = make_tmap_heads(&tv, v, head_dim, Hkv, map_kv_tokens, paged ? num_blocks : map_batch, kv_stride_head,
                       kv_stride_tok, kv_stride_tok * map_kv_tokens, paged ? block_size : 0);
  if (rc) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_dense_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)FaCfg<128>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_dense_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)FaCfg<64>::SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured[dev] = true;
  }
  FaParams p{};
  p.out = reinterpret_cast<bf16*>(out);
  p.out_stride_tok = out_stride_tok;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.cu_q = cu_q;
  p.kv_lens = kv_lens;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  if (cu_q) p.q_len = 0;   // rows are addressed by their flat token index
  if (peers) {
    if (world < 1 || world > 8 || batch != 1 || n1 <= 0 || (split > 0 && n0 <= 0) || (col_offset % 8) != 0) return -3;
    for (int r = 0; r < world; ++r) p.scatter.peer[r] = reinterpret_cast<bf16*>(peers[r]);
    p.scatter.enabled = 1;
    p.scatter.split = split;
    p.scatter.n0 = n0 > 0 ? n0 : 1;
    p.scatter.n1 = n1;
    p.scatter.col_offset = col_offset;
  }
  // one-tile CTAs when that shortens the schedule: a one-tile CTA takes ~0.85 of a two-tile CTA's time (measured)
  const int sms = 148;
  const long c2 = (long)((q_len + 2 * BM - 1) / (2 * BM)) * Hq * batch, c1 = (long)((q_len + BM - 1) / BM) * Hq * batch;
  const double t2 = (double)((c2 + sms - 1) / sms), t1 = 0.85 * (double)((c1 + sms - 1) / sms);
  p.tiles = (g_force_tiles == 1 || g_force_tiles == 2) ? g_force_tiles : (t1 < t2 ? 1 : 2);
  dim3 grid((q_len + p.tiles * BM - 1) / (p.tiles * BM), Hq, batch);
  if (head_dim == 64)
    return launch_kernel(attn_dense_tcgen05_kernel<64>, grid, dim3(THREADS), FaCfg<64>::SMEM_BYTES, stream, tq, tk, tv, p);
  return launch_kernel(attn_dense_tcgen05_kernel<128>, grid, dim3(THREADS), FaCfg<128>::SMEM_BYTES, stream, tq, tk, tv, p);
}

}  // namespace swb
