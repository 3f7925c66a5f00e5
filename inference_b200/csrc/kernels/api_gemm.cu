// extern "C" entry points for the dense GEMM.
#include "gemm_tcgen05.cuh"

namespace swb {
namespace {
unsigned long long* g_trace = nullptr;
}
unsigned long long* gemm_trace_buffer() { return g_trace; }
}  // namespace swb

extern "C" {

// Profiling aid: when set to a device buffer of at least grid * 16 uint64, decode GEMM CTAs record per CTA eight
// globaltimer stamps of their phases (start, setup done, dependency satisfied, accumulator complete, partials
// delivered, cluster barrier passed, outputs stored, end) followed by eight SM-clock stamps of the epilogue
// ([8] barrier passed, [9] first group summed, [10] first group stored, [11] all stored, [12] accumulator complete,
// [13] partials delivered, [14] first group's sum of squares sent). Pass null to switch it off.
void swb_gemm_set_trace(void* device_buffer) { swb::g_trace = reinterpret_cast<unsigned long long*>(device_buffer); }

int swb_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* D, int ldd, int T, int N, int K,
                  const void* bias, const void* residual, int ld_res, int act, int out_fp32, void* workspace,
                  size_t workspace_bytes, int force_mode, int force_block_n, int force_ctas, void* stream) {
  swb::GemmArgs a;
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = D;
  a.ldd = ldd;
  a.T = T;
  a.N = N;
  a.K = K;
  a.bias = bias;
  a.residual = residual;
  a.ld_res = ld_res;
  a.act = act;
  a.out_fp32 = out_fp32;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.force_mode = force_mode;
  a.force_block_n = force_block_n;
  a.force_ctas = force_ctas;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// 3x3 convolution, stride 1, zero padding 1, over an NHWC bf16 activation x [n, h, w, c] as an implicit GEMM on the
// tcgen05 kernel: no patch matrix is written; each reduction block is one window tap over one 64-channel slab, fetched
// by a 4-D TMA box at the tile's pixel origin shifted by the tap (zero fill outside the image is the padding).
// W [cout, (ky, kx, cin)] bf16 rows of 9 c; out [n h w, cout] bf16 (= NHWC); optional bias [cout] and residual
// [n h w, cout]. Needs c % 64 == 0, h w % 128 == 0 and w a multiple or a divisor of 128; returns -3 otherwise.
int swb_conv3x3_nhwc(const void* x, int n, int h, int w, int c, const void* W, int ldw, int cout, void* out, int ldd,
                     const void* bias, const void* residual, int ld_res, int act, void* stream) {
  swb::GemmArgs a;
  a.A = x;
  a.lda = c;
  a.W = W;
  a.ldw = ldw;
  a.D = out;
  a.ldd = ldd;
  a.T = n * h * w;
  a.N = cout;
  a.K = 9 * c;
  a.bias = bias;
  a.residual = residual;
  a.ld_res = ld_res;
  a.act = act;
  a.out_fp32 = 0;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  a.force_mode = 0;
  a.force_block_n = 0;
  a.force_ctas = -1;
  a.conv_n = n;
  a.conv_h = h;
  a.conv_w = w;
  a.conv_c = c;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// GEMM whose epilogue dispatches the output head-sharded to peers (see GemmScatter): D is not written locally.
// peers: `world` device pointers to every rank's receive buffer [global rows, N / (heads * 128), heads_per_rank, 128].
int swb_gemm_bf16_scatter(const void* A, int lda, const void* W, int ldw, int T, int N, int K, const void* bias,
                          int act, void* const* peers, int world, int heads, int row_split, int row_off0,
                          int row_off1, void* stream) {
  if (world < 1 || world > 8 || heads % world != 0 || N % (heads * 128) != 0) return -3;
  swb::GemmScatter sc{};
  for (int r = 0; r < world; ++r) sc.peer[r] = reinterpret_cast<__nv_bfloat16*>(peers[r]);
  sc.enabled = 1;
  sc.hd_total = heads * 128;
  sc.heads_per_rank = heads / world;
  sc.ld = (N / sc.hd_total) * sc.heads_per_rank * 128;
  sc.row_split = row_split;
  sc.row_off0 = row_off0;
  sc.row_off1 = row_off1;
  swb::GemmArgs a{};
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = nullptr;
  a.ldd = 16;
  a.T = T;
  a.N = N;
  a.K = K;
  a.bias = bias;
  a.act = act;
  a.force_mode = 0;
  a.scatter = &sc;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// Row-parallel GEMM whose epilogue performs the scatter half of a reduce-scatter: this rank's partial sums for token
// row t go to rank t / rows_per_rank, slot `rank` of its [world, rows_per_rank, N] buffer (peers[r]).
int swb_gemm_bf16_scatter_rows(const void* A, int lda, const void* W, int ldw, int T, int N, int K, void* const* peers,
                               int world, int rank, int rows_per_rank, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_rank <= 0 ||
      (long long)rows_per_rank * world < T)
    return -3;
  swb::GemmScatter sc{};
  for (int r = 0; r < world; ++r) sc.peer[r] = reinterpret_cast<__nv_bfloat16*>(peers[r]);
  sc.enabled = 2;
  sc.ld = N;
  sc.rows_per_rank = rows_per_rank;
  sc.src_rank = rank;
  swb::GemmArgs a{};
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = nullptr;
  a.ldd = 16;
  a.T = T;
  a.N = N;
  a.K = K;
  a.force_mode = 0;
  a.scatter = &sc;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// Grouped GEMM for mixture-of-experts layers: rows [128 * i, 128 * i + 128) of A multiply weight group
// group_of_mtile[i] of the stacked W [groups * N, K]; tiles whose entry is negative are skipped (their output rows
// are left untouched). T must be a multiple of 128; the table lives in device memory, so routing never touches the host.
int swb_gemm_bf16_grouped(const void* A, int lda, const void* W, int ldw, int groups, const int* group_of_mtile, void* D,
                          int ldd, int T, int N, int K, int act, void* stream) {
  if (groups <= 0 || !group_of_mtile || T % 128 != 0) return -3;
  swb::GemmArgs a{};
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = D;
  a.ldd = ldd;
  a.T = T;
  a.N = N;
  a.K = K;
  a.act = act;
  a.force_mode = 0;
  a.force_ctas = -1;
  a.group_of_mtile = group_of_mtile;
  a.groups = groups;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// Decode GEMM inside a folded-RMSNorm chain (T <= 64, cluster kernel): ssq_in (nullable) = per-token sums of squares
// accumulated by the producer of A, the accumulators are scaled by rsqrt(sum / norm_dim + eps) per token; ssq_out
// (nullable) accumulates this launch's sums of the rows it stores (after the residual add) and must be zero at
// launch; ssq_zero (nullable) is zeroed by this launch (the chain's other accumulator). Buffers: 64 x u64, 2^-24
// fixed point. Returns -3 when the shape is not served by the cluster kernel.
int swb_gemm_bf16_normed(const void* A, int lda, const void* W, int ldw, void* D, int ldd, int T, int N, int K,
                         const void* bias, const void* residual, int ld_res, int act, const void* ssq_in,
                         void* ssq_out, void* ssq_zero, int norm_dim, float norm_eps, void* stream) {
  swb::GemmArgs a{};
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = D;
  a.ldd = ldd;
  a.T = T;
  a.N = N;
  a.K = K;
  a.bias = bias;
  a.residual = residual;
  a.ld_res = ld_res;
  a.act = act;
  a.force_mode = -1;
  a.ssq_in = ssq_in;
  a.ssq_out = ssq_out;
  a.ssq_zero = ssq_zero;
  a.norm_dim = norm_dim;
  a.norm_eps = norm_eps;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

// Row-parallel decode GEMM (T <= 64) whose epilogue sums the partial products over the tensor-parallel ranks through
// peer memory (see GemmPeerReduce): D = sum_ranks(A_r W_r^T) + residual on every rank; ssq_out / ssq_zero as in
// swb_gemm_bf16_normed. slots / results: `world` device pointers each to line buffers of [world][cap][slot_ld / 8][2]
// and [cap][slot_ld / 8][2] 16-byte lines (zero at start); epochs: local [swb_gemm_peer_max_ctas()] words, zero at
// start.
int swb_gemm_bf16_peer_reduce(const void* A, int lda, const void* W, int ldw, void* D, int ldd, int T, int N, int K,
                              const void* residual, int ld_res, void* ssq_out, void* ssq_zero, void* const* slots,
                              void* const* results, void* epochs, int cap, int slot_ld, int mode, int world, int rank,
                              int force_cluster, void* stream) {
  if (world < 2 || world > 8 || !slots || !epochs || (mode == 2 && !results)) return -3;
  swb::GemmPeerReduce q{};
  for (int r = 0; r < world; ++r) {
    q.slots[r] = reinterpret_cast<uint4*>(slots[r]);
    q.result[r] = results ? reinterpret_cast<uint4*>(results[r]) : nullptr;
  }
  q.epochs = reinterpret_cast<uint32_t*>(epochs);
  q.cap = cap;
  q.ld = slot_ld;
  q.mode = mode;
  q.world = world;
  q.rank = rank;
  swb::GemmArgs a{};
  a.A = A;
  a.lda = lda;
  a.W = W;
  a.ldw = ldw;
  a.D = D;
  a.ldd = ldd;
  a.T = T;
  a.N = N;
  a.K = K;
  a.residual = residual;
  a.ld_res = ld_res;
  a.force_mode = 2;
  a.force_ctas = force_cluster;
  a.ssq_out = ssq_out;
  a.ssq_zero = ssq_zero;
  a.peer = &q;
  return swb::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}

int swb_gemm_peer_max_ctas(void) { return swb::SWB_PEER_MAX_CTAS; }

int swb_gemm_gated_supported(int T, int N, int K) { return swb::gemm_bf16_gated_supported(T, N, K); }

size_t swb_gemm_workspace_min(void) { return swb::SWB_GEMM_COUNTER_BYTES + (size_t)(8u << 20); }

int swb_sm_count(void) { return swb::device_sm_count(); }

}  // extern "C"
