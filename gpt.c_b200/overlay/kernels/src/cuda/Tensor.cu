// Device tensor support for gpt.c on top of libattn_sm100.so: drop-in for kernels/src/cuda/Tensor.cu
// (declarations in kernels/src/cuda/Tensor.h).  Host<->device moves, creation and the cuBLAS wrappers
// keep the reference's behaviour (stream-ordered allocation, synchronise after a move, row-major
// operands handed to column-major cuBLAS by swapping them); fills, arange, copies and unit-stride
// saxpy go through the vectorised kernels of tensor_sm100.h.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cpu/Alloc.h>
#include <cuda/Alloc.h>
#include <cuda/Tensor.h>
#include <common/kutils.h>
#include "tensor_sm100.h"

static void tens_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[TENSOR ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

extern "C" {

void move_tensor_to_host_cuda(tensor_t *tensor) {
    CHECK_ERROR(tensor == NULL, "Expected *tensor to be a tensor_t pointer. Got NULL");
    CHECK_ERROR(tensor->t == NULL, "Expected *tensor->t to be a float pointer. Got NULL");
    if (tensor->device == CPU) return;
    float *dev = tensor->t;
    const size_t bytes = (size_t)tensor->length * sizeof(float);
    float *host = (float *)aligned_alloc_cpu(bytes, 64);
    cudaStream_t stream = get_cuda_stream();
    cudaCheck(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, stream));
    cudaCheck(cudaStreamSynchronize(stream));
    tensor->t = host;
    tensor->device = CPU;
    free_cuda(dev);
}

void move_tensor_to_device_cuda(tensor_t *tensor) {
    CHECK_ERROR(tensor == NULL, "Expected *tensor to be a tensor_t pointer. Got NULL");
    CHECK_ERROR(tensor->t == NULL, "Expected *tensor->t to be a float pointer. Got NULL");
    if (tensor->device == CUDA) {
        printf("Tensor already on CUDA. Returning.\n");
        return;
    }
    float *host = tensor->t;
    const size_t bytes = (size_t)tensor->length * sizeof(float);
    float *dev = (float *)alloc_cuda(bytes);
    cudaStream_t stream = get_cuda_stream();
    cudaCheck(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, stream));
    cudaCheck(cudaStreamSynchronize(stream));
    tensor->t = dev;
    tensor->device = CUDA;
    free_cpu(host);
}

void create_tensor_data_cuda(tensor_t *tensor) {
    CHECK_ERROR(tensor == NULL, "Expected *tensor to be a tensor_t pointer. Got NULL");
    CHECK_ERROR(tensor->t != NULL, "Expected *tensor->t to be NULL. Got a pointer to address %p.", tensor->t);
    tensor->t = (float *)alloc_cuda((size_t)tensor->length * sizeof(float));
}

void fill_tensor_data_cuda(tensor_t *tensor, const float value) {
    CHECK_ERROR(tensor == NULL, "Expected *tensor to be a tensor_t pointer. Got NULL");
    if (!tensor->t) create_tensor_data_cuda(tensor);
    tens_check(tensor_sm100_fill(tensor->t, (size_t)tensor->length, value, (void *)get_cuda_stream()), "tensor_sm100_fill");
}

void zeros_tensor_data_cuda(tensor_t *tensor) { fill_tensor_data_cuda(tensor, 0.0f); }

void ones_tensor_data_cuda(tensor_t *tensor) { fill_tensor_data_cuda(tensor, 1.0f); }

void arange_tensor_data_cuda(tensor_t *tensor, const int start, const int end, const int steps) {
    (void)end;  // the length of the tensor decides, like in the reference
    CHECK_ERROR(tensor == NULL, "Expected *tensor to be a tensor_t pointer. Got NULL");
    if (!tensor->t) create_tensor_data_cuda(tensor);
    tens_check(tensor_sm100_arange(tensor->t, (size_t)tensor->length, start, steps, (void *)get_cuda_stream()),
               "tensor_sm100_arange");
}

void copy_tensor_data_cuda(tensor_t *dst, const tensor_t *src) {
    CHECK_ERROR(dst == NULL, "Expected *dst to be a tensor_t pointer. Got NULL");
    CHECK_ERROR(src == NULL, "Expected *src to be a tensor_t pointer. Got NULL");
    CHECK_ERROR(dst->t == NULL, "Expected *dst->t to be a float pointer. Got NULL");
    CHECK_ERROR(src->t == NULL, "Expected *src->t to be a float pointer. Got NULL");
    CHECK_ERROR(src->length != dst->length, "Expected src and dst tensors to be of same length. Got %d != %d", src->length,
                dst->length);
    tens_check(tensor_sm100_copy(dst->t, src->t, (size_t)dst->length, (void *)get_cuda_stream()), "tensor_sm100_copy");
}

void saxpy_cuda(const int n, const float alpha, const tensor_t *x, const int offsetx, const int incx, tensor_t *y,
                const int offsety, const int incy) {
    const float *xp = x->t + offsetx;
    float *yp = y->t + offsety;
    if (incx == 1 && incy == 1) {
        tens_check(tensor_sm100_axpy((size_t)n, alpha, xp, yp, (void *)get_cuda_stream()), "tensor_sm100_axpy");
        return;
    }
    cublasCheck(cublasSaxpy(get_cublas_handle(), n, &alpha, xp, incx, yp, incy));
}

// Row-major C[M,N] = alpha * op(A) * op(B) + beta * C through column-major cuBLAS: the operands swap
// places and every matrix is read as its transpose.
void sgemm_cuda(const int TransA, const int TransB, const int M, const int N, const int K, const float alpha,
                const tensor_t *A, const int offsetA, const int lda, const tensor_t *B, const int offsetB, const int ldb,
                const float beta, tensor_t *C, const int offsetC, const int ldc) {
    const cublasOperation_t opa = TransA == 1 ? CUBLAS_OP_T : CUBLAS_OP_N;
    const cublasOperation_t opb = TransB == 1 ? CUBLAS_OP_T : CUBLAS_OP_N;
    cublasCheck(cublasSgemm(get_cublas_handle(), opb, opa, N, M, K, &alpha, B->t + offsetB, ldb, A->t + offsetA, lda, &beta,
                            C->t + offsetC, ldc));
}

void sgemm_strided_batched_cuda(const int TransA, const int TransB, const int M, const int N, const int K, const float alpha,
                                const tensor_t *A, const int lda, const int strideA, const tensor_t *B, const int ldb,
                                const int strideB, const float beta, tensor_t *C, const int ldc, const int strideC,
                                const int batch_count) {
    const cublasOperation_t opa = TransA == 1 ? CUBLAS_OP_T : CUBLAS_OP_N;
    const cublasOperation_t opb = TransB == 1 ? CUBLAS_OP_T : CUBLAS_OP_N;
    cublasCheck(cublasSgemmStridedBatched(get_cublas_handle(), opb, opa, N, M, K, &alpha, B->t, ldb, strideB, A->t, lda,
                                          strideA, &beta, C->t, ldc, strideC, batch_count));
}

}  // extern "C"
