/*
 * adamw_sm100.h: C ABI of the B200 (sm_100a) AdamW step used by gpt.c's optimizer.  Same library and
 * conventions as attn_sm100.h (ATTN_OK / negative ATTN_ERR_* / positive cudaError_t, work only enqueued on
 * `stream`, never synchronises).
 *
 * Reference interface this entry point replaces (paths relative to the gpt.c project root):
 *
 *   adamw_sm100_step   step_adamW_cuda_kernel   kernels/src/cuda/AdamW.cu:64-148 (declared
 *                      kernels/src/cuda/AdamW.h:10-22) and its kernel :13-57; CPU counterpart
 *                      kernels/src/cpu/AdamW.c
 */
#ifndef ADAMW_SM100_H
#define ADAMW_SM100_H

#include "attn_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * One AdamW step (decoupled weight decay) over n tensors.  params/grads/m/v are HOST arrays of n device
 * pointers, lengths a host array of n element counts; `step` counts from 1.  Per element, in the reference's
 * order:  p -= lr*wd*p;  m = lerp(g, m, beta1);  v = lerp(g*g, v, beta2);
 *         p -= lr * (m / (1 - beta1^step)) / (sqrt(v / (1 - beta2^step)) + eps)
 * with lerp(a, b, w) = fma(w, b, fma(-w, a, a)).  The device copy of the tensor list is kept between calls
 * and re-uploaded only when the host arrays change (stream-ordered allocation on `stream` then).
 */
int adamw_sm100_step(float *const *params, float *const *grads, float *const *m, float *const *v, const int *lengths, int n,
                     float lr, float beta1, float beta2, float weight_decay, float eps, int step, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* ADAMW_SM100_H */
