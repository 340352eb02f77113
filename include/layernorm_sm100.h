/*
 * layernorm_sm100.h: C ABI of the B200 (sm_100a) LayerNorm kernels (the normalisation in front of the
 * attention layer and of the MLP in every gpt.c block).  Same library and conventions as
 * attn_sm100.h: device pointers on the current device, 16-byte aligned rows, row-major fp32, work
 * only enqueued on `stream`, ATTN_OK / negative ATTN_ERR_* / positive cudaError_t, never exit.
 *
 * Reference interfaces these entry points replace (paths relative to the gpt.c project root):
 *
 *   layernorm_sm100_forward    layer_norm_forward_cuda_kernel    kernels/src/cuda/LayerNorm.cu:115-136
 *                              (declared kernels/src/cuda/LayerNorm.h:9-16) and its kernel :7-60
 *   layernorm_sm100_backward   layer_norm_backward_cuda_kernel   kernels/src/cuda/LayerNorm.cu:138-165
 *                              (declared LayerNorm.h:18-25) and its kernel :62-110
 *   CPU counterparts (the oracle's source): kernels/src/cpu/LayerNorm.c:5-59 and :61-123
 */
#ifndef LAYERNORM_SM100_H
#define LAYERNORM_SM100_H

#include "attn_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * y[r, :] = (x[r, :] - mean[r]) * rstd[r] * w + b,  mean and rstd (= 1 / sqrt(var + eps)) written per row.
 *   rows = B*T, C = features; b may be NULL.  Requirements: C % 4 == 0 and C <= 2048, else
 *   ATTN_ERR_UNSUPPORTED.
 */
int layernorm_sm100_forward(const float *x, const float *w, const float *b, float eps, float *mean, float *rstd, float *y,
                            int rows, int C, void *stream);

/*
 * dw[C] += sum_r dy * xhat,  db[C] += sum_r dy (db may be NULL),  dx[r, :] += the input gradient:
 * all three ACCUMULATE into what the buffers hold, like the reference (whose layer hands in a
 * zero-filled dx).  dw and db are built with one fp32 atomic per column and thread block, so their
 * last bits can differ between runs.  Same shape requirements as the forward.
 */
int layernorm_sm100_backward(const float *dy, const float *x, const float *mean, const float *rstd, const float *w, float *dw,
                             float *db, float *dx, int rows, int C, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* LAYERNORM_SM100_H */
