/*
 * tensor_sm100.h: C ABI of the B200 (sm_100a) element-wise tensor helpers: the fills, copies and
 * residual adds around the attention layer in every gpt.c block.  Same library and conventions as
 * attn_sm100.h (device pointers on the current device, work only enqueued on `stream`, ATTN_OK /
 * negative ATTN_ERR_* / positive cudaError_t); any alignment is accepted, 16-byte aligned pointers
 * take the vectorised path.  n == 0 is a no-op.
 *
 * Reference interfaces these entry points replace (paths relative to the gpt.c project root):
 *
 *   tensor_sm100_fill     zeros/ones/fill_tensor_data_cuda   kernels/src/cuda/Tensor.cu:79-107 (kernel :8-13)
 *   tensor_sm100_arange   arange_tensor_data_cuda            kernels/src/cuda/Tensor.cu:109-117 (kernel :15-20)
 *   tensor_sm100_copy     copy_tensor_data_cuda              kernels/src/cuda/Tensor.cu:119-130 (kernel :22-27)
 *   tensor_sm100_axpy     saxpy_cuda with unit strides       kernels/src/cuda/Tensor.cu:132-141 (cublasSaxpy)
 *   tensor_sm100_gelu_forward / _backward   gelu_forward/backward_cuda_kernel   kernels/src/cuda/GeLU.cu:40-64 (kernels :5-38)
 */
#ifndef TENSOR_SM100_H
#define TENSOR_SM100_H

#include "attn_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/* p[i] = value for i < n. */
int tensor_sm100_fill(float *p, size_t n, float value, void *stream);
/* p[i] = (float)(start + step * i), the integer expression of the reference. */
int tensor_sm100_arange(float *p, size_t n, int start, int step, void *stream);
/* dst[i] = src[i]; the ranges must not overlap. */
int tensor_sm100_copy(float *dst, const float *src, size_t n, void *stream);
/* y[i] = alpha * x[i] + y[i], one fused multiply-add per element. */
int tensor_sm100_axpy(size_t n, float alpha, const float *x, float *y, void *stream);
/* y[i] = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))): the tanh approximation of GELU the reference uses. */
int tensor_sm100_gelu_forward(const float *x, float *y, size_t n, void *stream);
/* dx[i] = g[i] * d/dx of the above at x[i] (overwritten, like the reference). */
int tensor_sm100_gelu_backward(const float *g, const float *x, float *dx, size_t n, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* TENSOR_SM100_H */
