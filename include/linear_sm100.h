/*
 * linear_sm100.h: C ABI of the B200 (sm_100a) Linear kernels that sit either side of the attention
 * layer in gpt.c (the QKV projection before it, c_proj after it).  Same library as attn_sm100.h
 * (libattn_sm100.so), same conventions: device pointers on the current device, 16-byte aligned,
 * row-major fp32, work only enqueued on `stream`, return ATTN_OK / negative ATTN_ERR_* /
 * positive cudaError_t, never exit, never synchronise.
 *
 * Reference interfaces these entry points replace (paths relative to the gpt.c project root):
 *
 *   linear_sm100_forward    linear_forward_cuda_kernel   kernels/src/cuda/Linear.cu:37-60
 *                           (declared kernels/src/cuda/Linear.h:9-12): sgemm_cuda (cuBLAS, TF32
 *                           tensor-op math, kernels/src/cuda/Tensor.cu:147-176) + add_bias kernel (:7-18)
 *   linear_sm100_backward   linear_backward_cuda_kernel  kernels/src/cuda/Linear.cu:62-92
 *                           (declared Linear.h:14-18): two SGEMMs + bias_backward (:20-32)
 *   CPU counterparts (the oracle's source): kernels/src/cpu/Linear.c:4-31 and :33-88
 *
 * Arithmetic: TF32 inputs (the fp32 operands are read as they are, the tensor cores use the upper
 * 19 bits), fp32 accumulation: the same precision class as the reference's CUDA path.
 */
#ifndef LINEAR_SM100_H
#define LINEAR_SM100_H

#include "attn_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * y[M, N] = x[M, K] . w[N, K]^T + bias[N]        (M = B*T rows, K = in_features, N = out_features)
 *   bias    may be NULL (no bias, like the reference's `b == NULL`).
 *   planes  may be NULL.  Otherwise it receives y a second time as two bf16 planes (hi = bf16(y),
 *           lo = bf16(y - hi)), laid out exactly like the `saved` buffer of attn_sm100_forward
 *           (attn_sm100_saved_bytes(B, T, H, D) bytes with 3*H*D = N): the attention layer can then be
 *           called with ATTN_FLAG_CORE_ONLY and skip its own split pass.  No counterpart in the reference.
 * Requirements: K % 4 == 0 (N % 8 == 0 with planes); else ATTN_ERR_UNSUPPORTED.  When N is not a multiple
 * of 4 (gpt.c's vocabulary projection, N = 50257) the rows of y are not 16-byte aligned: the result is
 * then written with plain coalesced stores instead of the copy engine, and y and bias need no alignment.
 */
int linear_sm100_forward(const float *x, const float *w, const float *bias, float *y, void *planes, int M, int N, int K,
                         void *stream);

/*
 * Bytes of device scratch linear_sm100_backward needs: 0 when N is a multiple of 32, else room for a copy of
 * dy whose rows are padded to the next multiple of 32 columns (the vocabulary projection, N = 50257: its rows
 * start on 4-byte boundaries only, which the copy engine cannot tile).
 */
size_t linear_sm100_backward_scratch_bytes(int M, int N, int K);

/*
 * dx[M, K]  = dy[M, N] . w[N, K]           (overwritten, like the reference's beta = 0)
 * dw[N, K] += dy[M, N]^T . x[M, K]         (accumulated, like the reference's beta = 1)
 * db[N]    += column sums of dy            (accumulated; db may be NULL)
 * dx or dw may be NULL (not both): that product is skipped, e.g. dx for a layer whose input needs no
 * gradient.  scratch: linear_sm100_backward_scratch_bytes(M, N, K) bytes, 16-byte aligned (NULL when 0).
 * Requirements: K % 32 == 0; else ATTN_ERR_UNSUPPORTED.  dy, x, w, dx, dw and scratch start on 16-byte
 * boundaries (dy too when N is not a multiple of 4: only its later rows are unaligned then); else
 * ATTN_ERR_ALIGN.
 * dw and db are built from fp32 additions whose order is not fixed (split over M): results can differ
 * in the last bits between runs.
 */
int linear_sm100_backward(const float *dy, const float *x, const float *w, float *dx, float *dw, float *db, void *scratch,
                          int M, int N, int K, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* LINEAR_SM100_H */
