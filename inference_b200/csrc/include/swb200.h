/* C ABI of the sm_100a kernel library (libswb200_kernels.so).
 *
 * Every function takes raw device pointers and the CUDA stream to launch on, returns 0 on success and a
 * negative value on a launch/argument error. No function allocates device memory: scratch buffers are
 * passed in by the caller. All tensors are row-major; "ld" arguments are row strides in elements.
 */
#ifndef SWB200_H_
#define SWB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* swb_stream_t; /* cudaStream_t */

/* ---- status / health -------------------------------------------------------------------------- */
int swb_status_read(int* out8);
int swb_status_clear(void);
int swb_set_wait_limit_ns(unsigned long long ns);
int swb_sm_count(void);

/* ---- dense bf16 GEMM on tcgen05 ---------------------------------------------------------------
 * D[T, N] = act(A[T, K] * W[N, K]^T + bias[N]) + residual[T, N]; A, W, bias, residual bf16;
 * D bf16 or fp32 (out_fp32). act: 0 none, 1 SiLU, 2 tanh-GELU.
 * workspace: >= swb_gemm_workspace_min() bytes, zero-filled once by the caller; it lets small problems
 * split K across CTAs. Calls that share a workspace must be ordered on one stream.
 * force_mode: -1 auto, 0 tokens-as-M, 1 weights-as-M (T <= 256). force_block_n: 0 auto. force_ctas: 0 auto, > 0 stream-K over that many CTAs, < 0 whole tiles only. */
int swb_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* D, int ldd, int T, int N, int K,
                  const void* bias, const void* residual, int ld_res, int act, int out_fp32, void* workspace,
                  size_t workspace_bytes, int force_mode, int force_block_n, int force_ctas,
                  swb_stream_t stream);
size_t swb_gemm_workspace_min(void);

/* Grouped GEMM (mixture of experts): rows [128 i, 128 i + 128) of A [T, K] multiply group group_of_mtile[i] of the
 * stacked weight W [groups * N, K]; negative entries skip the tile. T is a multiple of 128; the table is device memory. */
int swb_gemm_bf16_grouped(const void* A, int lda, const void* W, int ldw, int groups, const int* group_of_mtile, void* D,
                          int ldd, int T, int N, int K, int act, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SWB200_H_ */
