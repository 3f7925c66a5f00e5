// Shared device-side primitives for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers,
// bounded waits and the library-wide status word.
//
// Every wait in this library is bounded: a spin that exceeds its budget records where it gave up in
// the status word and returns false so the kernel can drain and exit with the context intact.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace swb {

using bf16 = __nv_bfloat16;

// ---------------------------------------------------------------------------------------------
// Status word (device global, read back by swb_status_read()).
//   [0] sticky error code (0 = ok)   [1] detail a   [2] detail b   [3] detail c
// ---------------------------------------------------------------------------------------------
enum StatusCode : int {
  SWB_OK = 0,
  SWB_ERR_WAIT_TIMEOUT = 1,   // an mbarrier / flag wait ran out of budget
  SWB_ERR_BAD_ARGS = 2,
  SWB_ERR_PEER_TIMEOUT = 3,   // a wait on another rank's flag ran out of budget
};

// One copy per translation unit (no relocatable device code is used); each unit that can time out
// registers its copy with the host-side registry so swb_status_read() can aggregate them.
static __device__ int g_status[8] = {0, 0, 0, 0, 0, 0, 0, 0};
static __device__ unsigned long long g_wait_limit_ns = 2000000000ULL;
// Optional launch timeline (profiling aid, null = off): [0] = records written, [1] = capacity, records of four
// words from word 8 on: {kernel id, globaltimer before the dependency wait, after it, gridDim.x}. Written by thread 0
// of block 0 inside pdl_wait(), so the "after" stamp of launch k + 1 is the moment launch k had completely finished.
static __device__ unsigned long long* g_timeline = nullptr;

struct StatusUnit {
  const char* name;
  int (*read)(int* out8);
  int (*clear)();
  int (*set_limit)(unsigned long long ns);
  int (*set_timeline)(unsigned long long* buf);
};
void register_status_unit(const StatusUnit& u);

static int tu_status_read(int* out8) {
  return (int)cudaMemcpyFromSymbol(out8, g_status, 8 * sizeof(int));
}
static int tu_status_clear() {
  int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_status, z, sizeof(z));
}
static int tu_status_set_limit(unsigned long long ns) {
  return (int)cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns));
}
static int tu_set_timeline(unsigned long long* buf) {
  return (int)cudaMemcpyToSymbol(g_timeline, &buf, sizeof(buf));
}
struct StatusRegistrar {
  explicit StatusRegistrar(const char* name) {
    register_status_unit(StatusUnit{name, tu_status_read, tu_status_clear, tu_status_set_limit, tu_set_timeline});
  }
};
#define SWB_REGISTER_STATUS_UNIT(name) static ::swb::StatusRegistrar swb_status_registrar_##name(#name)

__device__ __forceinline__ void report_error(int code, int a, int b, int c) {
  if (atomicCAS(&g_status[0], 0, code) == 0) {
    g_status[1] = a;
    g_status[2] = b;
    g_status[3] = c;
    __threadfence();
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor
// in the stream is still running; it must call pdl_wait() before touching anything the predecessor
// produces (or anything the predecessor still reads and this kernel overwrites). pdl_launch_dependents()
// lets the successor begin launching. Both are no-ops for a normally launched kernel.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// kernel ids of the launch timeline
enum TimelineId : int {
  TL_OTHER = 0, TL_EMBED = 1, TL_RMSNORM = 2, TL_GEMM_DECODE = 3, TL_ROPE_KV = 4, TL_ATTN_DECODE = 5, TL_ATTN_MERGE = 6,
  TL_GEMM = 7, TL_ARGMAX = 8, TL_ARGMAX_MERGE = 9, TL_META = 10, TL_TAIL = 11, TL_PEER = 12, TL_GATED_ACT = 13,
  TL_ATTN_PREFILL = 14, TL_GEMM_QUANT = 15,
};

__device__ __forceinline__ void pdl_wait(int timeline_id = TL_OTHER) {
  unsigned long long* tl = g_timeline;
  if (tl != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    const unsigned long long slot = atomicAdd(tl, 1ull);
    const unsigned long long t0 = global_timer_ns();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (slot < tl[1]) {
      unsigned long long* rec = tl + 8 + slot * 4;
      rec[0] = (unsigned long long)timeline_id;
      rec[1] = t0;
      rec[2] = global_timer_ns();
      rec[3] = gridDim.x;
    }
    return;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();  // host: process-wide switch (env SWB_PDL=0 disables), defined in status.cu

template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return e == cudaSuccess ? 0 : -(int)e;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` is a CTA-shared int: once any role sets it every other role's wait
// returns false on its next slow-path check, so the whole CTA drains.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
#pragma unroll 1
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xFF) == 0) {
      if (*abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > g_wait_limit_ns) {
        *abort_flag = 1;
        report_error(SWB_ERR_WAIT_TIMEOUT, where, (int)blockIdx.x, (int)parity);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// TMA (non-multicast tiled bulk tensor copies only)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, "
      "%3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2,
                                                 int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, "
      "%3, %4, %5}], [%6], %7;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16/fp16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all previously issued tcgen05.mma of this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 consecutive fp32 columns: thread i of the warp reads TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// UMMA shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 64 bf16 x R rows with SWIZZLE_128B produces): 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused for swizzled K-major.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                         // leading byte offset (ignored) = 1
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset = 1024 B
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                         // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
  return (1u << 4)                       // D format fp32
         | (1u << 7)                     // A format bf16
         | (1u << 10)                    // B format bf16
         | ((uint32_t)(n >> 3) << 17)    // N / 8
         | ((uint32_t)(m >> 4) << 24);   // M / 16
}

// ---------------------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace swb
