// tensor_t adapter between gpt.c's kernel-level LayerNorm symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/LayerNorm.cu of gpt.c: exports layer_norm_forward_cuda_kernel and
// layer_norm_backward_cuda_kernel with the signatures of kernels/src/cuda/LayerNorm.h:9-25 (cache[0] =
// mean, cache[1] = rstd, cache[2] = the layer input), runs on the reference runtime's stream and
// prints and exits on error like every CUDA entry of the reference.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/LayerNorm.h>
#include "layernorm_sm100.h"

static void ln_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[LAYERNORM ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

extern "C" {

void layer_norm_forward_cuda_kernel(const tensor_t *W, const tensor_t *b, const tensor_t *input, const float eps,
                                    tensor_t **cache, tensor_t *output) {
    const int rows = input->shape[0] * input->shape[1], C = input->shape[2];
    ln_check(layernorm_sm100_forward(input->t, W->t, b ? b->t : NULL, eps, cache[0]->t, cache[1]->t, output->t, rows, C,
                                     (void *)get_cuda_stream()),
             "layernorm_sm100_forward");
}

void layer_norm_backward_cuda_kernel(const tensor_t *global_grad, const tensor_t **cache, const tensor_t *W, tensor_t *dW,
                                     tensor_t *db, tensor_t *dout) {
    const int rows = global_grad->shape[0] * global_grad->shape[1], C = global_grad->shape[2];
    ln_check(layernorm_sm100_backward(global_grad->t, cache[2]->t, cache[0]->t, cache[1]->t, W->t, dW->t,
                                      db ? db->t : NULL, dout->t, rows, C, (void *)get_cuda_stream()),
             "layernorm_sm100_backward");
}

}  // extern "C"
