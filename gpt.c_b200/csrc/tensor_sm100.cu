// Element-wise tensor helpers for sm_100a: fill, copy, arange and y += alpha * x as vectorised
// grid-stride kernels (16 bytes per thread and trip, enough blocks to keep every SM's memory pipes
// busy).  They replace the one-element-per-thread kernels of gpt.c's kernels/src/cuda/Tensor.cu
// (:8-28, launched from zeros/ones/fill/arange/copy_tensor_data_cuda :79-130) and its cublasSaxpy
// wrapper (:132-141) for the contiguous case: the residual adds and copies of every block
// (src/block.c:69-86, 108-126) and the zero-fills in front of every accumulating backward kernel; and the
// tanh-approximated GELU of the MLP (kernels/src/cuda/GeLU.cu), forward and backward.
// All of them are pure HBM traffic; the bound is the copy bandwidth.
#include "attn_internal.h"
#include "tc05.cuh"

#include "../../include/tensor_sm100.h"

namespace tens {
namespace {

constexpr int kThreads = 256;

int grid_for(size_t work_items) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t need = (work_items + kThreads - 1) / kThreads;
    const size_t cap = (size_t)sms * 16;
    return (int)(need < cap ? (need ? need : 1) : cap);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__global__ void __launch_bounds__(kThreads) fill_kernel(float *__restrict__ p, size_t n, float v) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n4 = n / 4;
    const float4 v4 = make_float4(v, v, v, v);
    for (size_t i = tid; i < n4; i += stride) reinterpret_cast<float4 *>(p)[i] = v4;
    for (size_t i = n4 * 4 + tid; i < n; i += stride) p[i] = v;
}

__global__ void __launch_bounds__(kThreads) fill_scalar_kernel(float *__restrict__ p, size_t n, float v) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

__global__ void __launch_bounds__(kThreads) arange_kernel(float *__restrict__ p, size_t n, int start, int step) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        p[i] = (float)(start + step * (int)i);  // integer arithmetic first, like the reference
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) copy_kernel(float *__restrict__ dst, const float *__restrict__ src, size_t n) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (kVec) {
        const size_t n4 = n / 4;
        size_t i = tid;
        for (; i + stride < n4; i += 2 * stride) {  // two loads in flight
            const float4 a = __ldcs(reinterpret_cast<const float4 *>(src) + i);
            const float4 b = __ldcs(reinterpret_cast<const float4 *>(src) + i + stride);
            reinterpret_cast<float4 *>(dst)[i] = a;
            reinterpret_cast<float4 *>(dst)[i + stride] = b;
        }
        if (i < n4) reinterpret_cast<float4 *>(dst)[i] = __ldcs(reinterpret_cast<const float4 *>(src) + i);
        for (size_t j = n4 * 4 + tid; j < n; j += stride) dst[j] = src[j];
    } else {
        for (size_t i = tid; i < n; i += stride) dst[i] = src[i];
    }
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) axpy_kernel(size_t n, float alpha, const float *__restrict__ x, float *__restrict__ y) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (kVec) {
        const size_t n4 = n / 4;
        for (size_t i = tid; i < n4; i += stride) {
            const float4 a = __ldcs(reinterpret_cast<const float4 *>(x) + i);
            float4 b = reinterpret_cast<float4 *>(y)[i];
            b.x = fmaf(alpha, a.x, b.x), b.y = fmaf(alpha, a.y, b.y), b.z = fmaf(alpha, a.z, b.z), b.w = fmaf(alpha, a.w, b.w);
            reinterpret_cast<float4 *>(y)[i] = b;
        }
        for (size_t j = n4 * 4 + tid; j < n; j += stride) y[j] = fmaf(alpha, x[j], y[j]);
    } else {
        for (size_t i = tid; i < n; i += stride) y[i] = fmaf(alpha, x[i], y[i]);
    }
}

// tanh-approximated GELU, the reference's formulas (kernels/src/cuda/GeLU.cu:5-38) term for term
__device__ __forceinline__ float gelu_fwd(float x) {
    const float kBeta = 0.7978845608028654f;  // sqrt(2 / pi)
    const float cube = 0.044715f * x * x * x;
    return 0.5f * x * (1.0f + tanhf(kBeta * (x + cube)));
}
__device__ __forceinline__ float gelu_bwd(float g, float x) {
    const float kBeta = 0.7978845608028654f;
    const float x_sq = x * x, x_cube = x_sq * x;
    const float t = tanhf(kBeta * (x + 0.044715f * x_cube));
    const float left = 0.5f * x, right = 1.0f + t;
    const float right_derivative = left * (1.0f - t * t) * (kBeta * (1.0f + 3.0f * 0.044715f * x_sq));
    return g * (0.5f * right + right_derivative);
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) gelu_forward_kernel(const float *__restrict__ x, float *__restrict__ y, size_t n) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (kVec) {
        const size_t n4 = n / 4;
        for (size_t i = tid; i < n4; i += stride) {
            const float4 a = __ldcs(reinterpret_cast<const float4 *>(x) + i);
            reinterpret_cast<float4 *>(y)[i] = make_float4(gelu_fwd(a.x), gelu_fwd(a.y), gelu_fwd(a.z), gelu_fwd(a.w));
        }
        for (size_t j = n4 * 4 + tid; j < n; j += stride) y[j] = gelu_fwd(x[j]);
    } else {
        for (size_t i = tid; i < n; i += stride) y[i] = gelu_fwd(x[i]);
    }
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) gelu_backward_kernel(const float *__restrict__ g, const float *__restrict__ x,
                                                                 float *__restrict__ dx, size_t n) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (kVec) {
        const size_t n4 = n / 4;
        for (size_t i = tid; i < n4; i += stride) {
            const float4 a = __ldcs(reinterpret_cast<const float4 *>(x) + i);
            const float4 b = __ldcs(reinterpret_cast<const float4 *>(g) + i);
            reinterpret_cast<float4 *>(dx)[i] =
                make_float4(gelu_bwd(b.x, a.x), gelu_bwd(b.y, a.y), gelu_bwd(b.z, a.z), gelu_bwd(b.w, a.w));
        }
        for (size_t j = n4 * 4 + tid; j < n; j += stride) dx[j] = gelu_bwd(g[j], x[j]);
    } else {
        for (size_t i = tid; i < n; i += stride) dx[i] = gelu_bwd(g[i], x[i]);
    }
}

}  // namespace
}  // namespace tens

extern "C" {

int tensor_sm100_fill(float *p, size_t n, float value, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!p) return ATTN_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (value == 0.0f && !signbit(value)) return (int)cudaMemsetAsync(p, 0, n * sizeof(float), s);
    if (aligned16(p)) return (int)attn::launch_after_previous(fill_kernel, dim3(grid_for(n / 4 + 1)), dim3(kThreads), 0, s, p, n, value);
    return (int)attn::launch_after_previous(fill_scalar_kernel, dim3(grid_for(n)), dim3(kThreads), 0, s, p, n, value);
}

int tensor_sm100_arange(float *p, size_t n, int start, int step, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!p) return ATTN_ERR_NULL;
    return (int)attn::launch_after_previous(arange_kernel, dim3(grid_for(n)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p,
                                            n, start, step);
}

int tensor_sm100_copy(float *dst, const float *src, size_t n, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!dst || !src) return ATTN_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (aligned16(dst) && aligned16(src))
        return (int)attn::launch_after_previous(copy_kernel<true>, dim3(grid_for(n / 8 + 1)), dim3(kThreads), 0, s, dst, src, n);
    return (int)attn::launch_after_previous(copy_kernel<false>, dim3(grid_for(n)), dim3(kThreads), 0, s, dst, src, n);
}

int tensor_sm100_axpy(size_t n, float alpha, const float *x, float *y, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!x || !y) return ATTN_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (aligned16(x) && aligned16(y))
        return (int)attn::launch_after_previous(axpy_kernel<true>, dim3(grid_for(n / 4 + 1)), dim3(kThreads), 0, s, n, alpha, x, y);
    return (int)attn::launch_after_previous(axpy_kernel<false>, dim3(grid_for(n)), dim3(kThreads), 0, s, n, alpha, x, y);
}

int tensor_sm100_gelu_forward(const float *x, float *y, size_t n, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!x || !y) return ATTN_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (aligned16(x) && aligned16(y))
        return (int)attn::launch_after_previous(gelu_forward_kernel<true>, dim3(grid_for(n / 4 + 1)), dim3(kThreads), 0, s, x, y, n);
    return (int)attn::launch_after_previous(gelu_forward_kernel<false>, dim3(grid_for(n)), dim3(kThreads), 0, s, x, y, n);
}

int tensor_sm100_gelu_backward(const float *g, const float *x, float *dx, size_t n, void *stream) {
    using namespace tens;
    if (n == 0) return ATTN_OK;
    if (!g || !x || !dx) return ATTN_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (aligned16(g) && aligned16(x) && aligned16(dx))
        return (int)attn::launch_after_previous(gelu_backward_kernel<true>, dim3(grid_for(n / 4 + 1)), dim3(kThreads), 0, s, g, x, dx, n);
    return (int)attn::launch_after_previous(gelu_backward_kernel<false>, dim3(grid_for(n)), dim3(kThreads), 0, s, g, x, dx, n);
}

}  // extern "C"
