// Parameter blocks for the tcgen05 bf16 GEMM (kernel in gemm_tcgen05.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace swb {

// 3 / 4: gated pairs. Output features come in (gate, up) row pairs of the weight: out[t, f] = silu|gelu(acc[2f]) * acc[2f+1],
// so the output is half as wide as the weight has rows (SwiGLU / GeGLU fused into the gate-up projection).
enum GemmAct : int { SWB_ACT_NONE = 0, SWB_ACT_SILU = 1, SWB_ACT_GELU_TANH = 2, SWB_ACT_SWIGLU_PAIRS = 3,
                     SWB_ACT_GEGLU_PAIRS = 4 };

// The first SWB_GEMM_COUNTER_BYTES of a GEMM workspace hold per-tile arrival counters (zero between
// launches: the caller zeroes them once, the kernel restores zero); fp32 split-K partials follow.
constexpr size_t SWB_GEMM_COUNTER_BYTES = 64 * 1024;

// Dispatch of the output to peers from the epilogue (tokens-as-M kernel, 16-byte stores only).
// enabled == 1, head-sharded (sequence-parallel attention): output columns are laid out [which (q/k/v...)][head][128];
//   head h belongs to rank h / heads_per_rank, whose buffer is [global rows, which, heads_per_rank, 128] with row
//   stride `ld`. Local row r lands at global row (r < row_split ? row_off0 : row_off1) + r.
// enabled == 2, row-sharded (reduce-scatter of a row-parallel GEMM): row t belongs to rank t / rows_per_rank, whose
//   buffer is [source rank, rows_per_rank, ld]; this rank's partial sums go to slot `src_rank`.
struct GemmScatter {
  __nv_bfloat16* peer[8];
  int enabled;
  int hd_total;        // heads * 128: width of one `which` block
  int heads_per_rank;
  int ld;
  int row_split, row_off0, row_off1;
  int rows_per_rank, src_rank;
};

// Sum of a row-parallel decode GEMM over the tensor-parallel ranks, performed inside the cluster kernel's epilogue
// over peer memory (plain 16-byte peer stores; no collective library call, no multicast, no fence, no barrier).
// Rows travel as flag-in-data lines: 16 bytes = {2 bf16, epoch, 2 bf16, epoch}; a reader spins (bounded) on the
// lines it needs until both epochs match, so a row costs one NVLink hop and the wire carries 2x the row bytes.
// CTA b of every rank owns the same slice of the output, so the exchange is per CTA and per 16-byte group.
// mode 1 (one shot): each CTA stores its bf16 partial slice into slot `rank` of every PEER's slot buffer
//   [world][cap tokens][ld / 8][2 lines], keeps its own slice in registers, then sums the `world` contributions in
//   rank order (bit-identical on every rank), adds the local residual and stores the rows.
// mode 2 (two shot): the slice of weight tile t belongs to rank t % world. Every rank sends its partial only to the
//   owner; the owner sums, adds its residual, stores its own rows and sends the finished bf16 slice to every peer's
//   result buffer [cap][ld / 8][2 lines], from which the peers copy it into their output. About 2 / world of the
//   one-shot traffic at the price of a second hop.
// epochs: local [SWB_PEER_MAX_CTAS] launch counters advanced by the kernel (graph-replay safe); a line's epoch is
// (counter << 9 | CTA index). Two slot / result buffer pairs must alternate between consecutive reductions of a
// stream: a rank enters reduction k + 2 only after reduction k + 1 delivered every peer's lines to it, which those
// peers sent after they had finished reading reduction k.
constexpr int SWB_PEER_MAX_CTAS = 512;
struct GemmPeerReduce {
  uint4* slots[8];
  uint4* result[8];
  uint32_t* epochs;
  int cap;                 // token rows of a slot
  int ld;                  // row width in elements (multiple of 8)
  int mode, world, rank;
};

// Kernel-level problem: D[M, N] = A[M, K] * B[N, K]^T, possibly stored transposed.
struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, kblocks_total;
  int stream_k;       // 1: contiguous (tile, k-block) ranges per CTA; 0: whole tiles, strided over CTAs
  int iters_per_cta;  // stream-K range length in k-block iterations
  int transposed;  // 1: rows of the tile are output features, columns are tokens
  int stream_a;    // 1: A is a weight read once (L2 evict-first)
  int vec_ok;      // 16-byte vector epilogue accesses are legal
  int ldd;
  void* out;
  int out_fp32;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ld_res;
  int act;
  float* workspace;
  int* counters;
  int* status;
  unsigned long long* trace;  // optional [grid][8] globaltimer stamps of kernel phases (profiling aid)
  GemmScatter scatter;
  int staged_epilogue;   // tokens-as-M, bf16 output: stage rows in shared memory and store 256-byte runs
  // grouped (mixture-of-experts) mode: row tile tm multiplies weight group group_of_mtile[tm] (rows
  // [g * group_rows, g * group_rows + N) of the stacked weight); a negative entry skips the tile
  const int* group_of_mtile;
  int group_rows;
  // RMSNorm folded into a chain of decode GEMMs (cluster kernel only). A producer (o / down projection with the
  // residual add in its epilogue) adds, per token, the sum of squares of the rows it stored to ssq_out[token] in
  // 2^-24 fixed point (64 x u64; integer adds commute, so the result does not depend on CTA order). The consumer
  // (qkv / gate-up projection on the un-normalised residual stream, norm weight pre-multiplied into its weights)
  // scales its accumulators by rsqrt(sum / norm_dim + eps) per token. An accumulator must be zero when its producer
  // starts: each producer zeroes the chain's OTHER accumulator (ssq_zero), whose consumer has finished by then.
  unsigned long long* ssq_out;
  const unsigned long long* ssq_in;
  unsigned long long* ssq_zero;
  int norm_dim;
  float norm_eps;
  GemmPeerReduce peer;   // decode cluster kernel only
  // 3x3 convolution as an implicit GEMM (conv_c > 0): A is an NHWC activation [n, conv_h, conv_w, conv_c] behind a 4-D
  // tensor map with a box of 64 channels x (tile of 128 pixels); reduction block kb is tap kb / (conv_c / 64) (row
  // major over the 3 x 3 window) and channel slab kb % (conv_c / 64), loaded at the tile's pixel origin shifted by the
  // tap, zero filled outside the image (= the convolution's padding). Weights are [out, (ky, kx, in)].
  int conv_h, conv_w, conv_c;
};

// User-level problem: D[T, N] = act(A[T, K] * W[N, K]^T + bias[N]) + residual[T, N].
struct GemmArgs {
  const void* A;
  int lda;
  const void* W;
  int ldw;
  void* D;
  int ldd;
  int T, N, K;
  const void* bias;
  const void* residual;
  int ld_res;
  int act;
  int out_fp32;
  void* workspace;
  size_t workspace_bytes;
  int force_mode;     // -1 auto, 0 tokens-as-M, 1 swapped (weights-as-M), 2 cluster split-K (T <= 64; force_ctas = cluster size)
  int force_block_n;  // 0 auto
  int force_ctas;     // 0 auto; > 0 stream-K over that many CTAs; < 0 whole tiles only
  const GemmScatter* scatter = nullptr;
  const int* group_of_mtile = nullptr;   // device [ceil(T / 128)]: weight group per 128-row tile, < 0 = skip
  int groups = 0;                        // W is [groups * N, K] when group_of_mtile is set
  void* ssq_out = nullptr;               // see GemmParams (decode cluster kernel only): 64 x u64
  const void* ssq_in = nullptr;
  void* ssq_zero = nullptr;
  int norm_dim = 0;
  float norm_eps = 0.f;
  const GemmPeerReduce* peer = nullptr;  // see GemmPeerReduce (decode cluster kernel only)
  int conv_n = 0, conv_h = 0, conv_w = 0, conv_c = 0;   // see GemmParams: A = NHWC activation, T = n h w, K = 9 c
};

int gemm_bf16_launch(const GemmArgs& a, cudaStream_t stream);
int gemm_bf16_gated_supported(int T, int N, int K);
int gemm_decode_cluster_supported(int T);
int gemm_decode_cluster_launch(const GemmArgs& a, int force_cluster, cudaStream_t stream);
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);
int make_tmap_bf16_nhwc(CUtensorMap* out, const void* ptr, int n, int h, int w, int c, int box_w, int box_h);
int make_tmap_u32_3d(CUtensorMap* out, const void* ptr, const unsigned long long dims[3], const unsigned long long strides[2],
                     const unsigned box[3]);
int make_tmap_u16_2d(CUtensorMap* out, const void* ptr, long long cols, long long rows, long long row_pitch_bytes,
                     int box_cols, int box_rows, int swizzle128);
int device_sm_count();
unsigned long long* gemm_trace_buffer();

}  // namespace swb
