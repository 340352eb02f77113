/*
 * xent_sm100.h: C ABI of the B200 (sm_100a) cross-entropy kernels (the loss over the vocabulary
 * projection at the end of gpt.c's transformer).  Same library and conventions as attn_sm100.h
 * (device pointers on the current device, row-major fp32, any 4-byte alignment, work only enqueued on
 * `stream`, ATTN_OK / negative ATTN_ERR_* / positive cudaError_t).
 *
 * Reference interfaces these entry points replace (paths relative to the gpt.c project root):
 *
 *   xent_sm100_forward    cross_entropy_forward_cuda_kernel    kernels/src/cuda/CrossEntropyLoss.cu:136-156 (kernel :8-79)
 *   xent_sm100_backward   cross_entropy_backward_cuda_kernel   kernels/src/cuda/CrossEntropyLoss.cu:158-178 (kernel :82-129)
 *   (declared kernels/src/cuda/CrossEntropyLoss.h:9-20); CPU counterparts: kernels/src/cpu/CrossEntropyLoss.c
 */
#ifndef XENT_SM100_H
#define XENT_SM100_H

#include "attn_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * logsm[r, :] = log_softmax(logits[r, :]);  *loss += sum_r -logsm[r, (int)targets[r]] / rows.
 * targets holds class indices as floats (the reference's convention); *loss must be initialised by the
 * caller (the reference's layer hands in zeros).  rows = B*T, C = classes.
 */
int xent_sm100_forward(const float *logits, const float *targets, float *logsm, float *loss, int rows, int C, void *stream);

/*
 * dout[r, target_r] = -g[r] / rows;  s = sum_j dout[r, j];  dout[r, j] -= exp(logsm[r, j]) * s.
 * Works on what dout holds (read-modify-write), like the reference, whose layer hands in zeros; g has one
 * value per row.
 */
int xent_sm100_backward(const float *g, const float *targets, const float *logsm, float *dout, int rows, int C, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* XENT_SM100_H */
