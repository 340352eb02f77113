// tensor_t adapter between gpt.c's kernel-level Linear symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/Linear.cu of gpt.c: exports linear_forward_cuda_kernel and
// linear_backward_cuda_kernel with the signatures of kernels/src/cuda/Linear.h:9-18, runs on the
// reference runtime's stream and prints and exits on error like every CUDA entry of the reference.
// Shapes the tensor-core kernels do not take (in_features not a multiple of 4 forward, of 32 backward) go
// through the reference runtime's own SGEMM wrapper (sgemm_cuda, kernels/src/cuda/Tensor.h:24-29) with two
// small bias kernels below.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/Alloc.h>
#include <cuda/Tensor.h>
#include <cuda/Linear.h>
#include "linear_sm100.h"
#include "attn_planes.h"

static void lin_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[LINEAR ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

// ---- the one-slot hand-off described in attn_planes.h ----
static const float *g_offer_y = NULL;
static void *g_offer_planes = NULL;
static size_t g_offer_bytes = 0;

extern "C" void overlay_planes_offer(const float *y, void *planes, size_t bytes) {
    if (g_offer_planes) free_cuda(g_offer_planes);  // stream ordered
    g_offer_y = y;
    g_offer_planes = planes;
    g_offer_bytes = bytes;
}

extern "C" void *overlay_planes_take(const float *y, size_t bytes) {
    if (!g_offer_planes || g_offer_y != y || g_offer_bytes != bytes) return NULL;
    void *p = g_offer_planes;
    g_offer_y = NULL;
    g_offer_planes = NULL;
    g_offer_bytes = 0;
    return p;
}

extern "C" void overlay_planes_forget(const void *y) {
    if (!g_offer_planes || (y != NULL && (const void *)g_offer_y != y)) return;
    void *p = g_offer_planes;
    g_offer_y = NULL;
    g_offer_planes = NULL;
    g_offer_bytes = 0;
    free_cuda(p);  // stream ordered; the slot is already empty, so the nested call finds nothing to forget
}

// ---- fallback pieces for shapes outside the tensor-core kernels ----
__global__ void overlay_add_bias_kernel(float *y, const float *bias, size_t rows, int cols) {
    const size_t n = rows * (size_t)cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] += bias[i % cols];
}
__global__ void overlay_bias_grad_kernel(const float *dy, float *db, int rows, int cols) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= cols) return;
    float acc = 0.f;
    for (int r = blockIdx.y; r < rows; r += gridDim.y) acc += dy[(size_t)r * cols + col];
    atomicAdd(db + col, acc);
}

static bool fast_forward_ok(int N, int K) { (void)N; return K % 4 == 0; }
static bool fast_backward_ok(int N, int K) { (void)N; return K % 32 == 0; }

extern "C" {

void linear_forward_cuda_kernel(const tensor_t *W, const tensor_t *b, const tensor_t *input, tensor_t *output) {
    const int K = W->shape[1], N = W->shape[0];
    const int M = input->shape[0] * input->shape[1];
    cudaStream_t stream = get_cuda_stream();
    if (fast_forward_ok(N, K)) {
        void *planes = NULL;
        size_t bytes = 0;
        if (N == 3 * K && K % 64 == 0) {  // the fused QKV projection in front of an attention layer
            bytes = attn_sm100_saved_bytes(input->shape[0], input->shape[1], K / 64, 64);
            if (bytes) planes = alloc_cuda(bytes);
        }
        lin_check(linear_sm100_forward(input->t, W->t, b ? b->t : NULL, output->t, planes, M, N, K, (void *)stream),
                  "linear_sm100_forward");
        if (planes) overlay_planes_offer(output->t, planes, bytes);
        return;
    }
    sgemm_cuda(0, 1, M, N, K, 1.0f, input, 0, K, W, 0, K, 0.0f, output, 0, N);
    if (b != NULL) {
        overlay_add_bias_kernel<<<1184, 256, 0, stream>>>(output->t, b->t, (size_t)M, N);
        cudaCheck(cudaGetLastError());
    }
}

void linear_backward_cuda_kernel(const tensor_t *global_grad, const tensor_t *cache, const tensor_t *W, tensor_t *dW,
                                 tensor_t *db, tensor_t *dout) {
    const int K = W->shape[1], N = W->shape[0];
    const int M = global_grad->shape[0] * global_grad->shape[1];
    cudaStream_t stream = get_cuda_stream();
    if (fast_backward_ok(N, K)) {
        const size_t scratch_bytes = linear_sm100_backward_scratch_bytes(M, N, K);
        void *scratch = scratch_bytes ? alloc_cuda(scratch_bytes) : NULL;
        lin_check(linear_sm100_backward(global_grad->t, cache->t, W->t, dout->t, dW->t, db ? db->t : NULL, scratch, M, N, K,
                                        (void *)stream),
                  "linear_sm100_backward");
        free_cuda(scratch);  // stream ordered
        return;
    }
    sgemm_cuda(0, 0, M, K, N, 1.0f, global_grad, 0, N, W, 0, K, 0.0f, dout, 0, K);
    sgemm_cuda(1, 0, N, K, M, 1.0f, global_grad, 0, N, cache, 0, K, 1.0f, dW, 0, K);
    if (db != NULL) {
        dim3 grid((N + 255) / 256, 64);
        overlay_bias_grad_kernel<<<grid, 256, 0, stream>>>(global_grad->t, db->t, M, N);
        cudaCheck(cudaGetLastError());
    }
}

}  // extern "C"
