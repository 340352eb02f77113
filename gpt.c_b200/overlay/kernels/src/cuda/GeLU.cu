// tensor_t adapter between gpt.c's kernel-level GELU symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/GeLU.cu of gpt.c: exports gelu_forward_cuda_kernel and
// gelu_backward_cuda_kernel with the signatures of kernels/src/cuda/GeLU.h:9-15 (cache = the layer input),
// runs on the reference runtime's stream and prints and exits on error like every CUDA entry of the reference.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/GeLU.h>
#include "tensor_sm100.h"

static void gelu_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[GELU ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

extern "C" {

void gelu_forward_cuda_kernel(const tensor_t *input, tensor_t *output) {
    gelu_check(tensor_sm100_gelu_forward(input->t, output->t, (size_t)input->length, (void *)get_cuda_stream()),
               "tensor_sm100_gelu_forward");
}

void gelu_backward_cuda_kernel(const tensor_t *global_grad, const tensor_t *cache, tensor_t *dout) {
    gelu_check(tensor_sm100_gelu_backward(global_grad->t, cache->t, dout->t, (size_t)global_grad->length,
                                          (void *)get_cuda_stream()),
               "tensor_sm100_gelu_backward");
}

}  // extern "C"
