// tensor_t adapter between gpt.c's kernel-level cross-entropy symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/CrossEntropyLoss.cu of gpt.c: exports cross_entropy_forward_cuda_kernel
// and cross_entropy_backward_cuda_kernel with the signatures of kernels/src/cuda/CrossEntropyLoss.h:9-20
// (cache[0] = log-softmax output [B, T, C], cache[1] = targets [B, T]), runs on the reference runtime's
// stream and prints and exits on error like every CUDA entry of the reference.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/CrossEntropyLoss.h>
#include "xent_sm100.h"

static void xent_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[CROSS ENTROPY ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

extern "C" {

void cross_entropy_forward_cuda_kernel(const tensor_t *logits, const tensor_t *targets, tensor_t **cache, tensor_t *output) {
    const int rows = logits->shape[0] * logits->shape[1], C = logits->shape[2];
    xent_check(xent_sm100_forward(logits->t, targets->t, cache[0]->t, output->t, rows, C, (void *)get_cuda_stream()),
               "xent_sm100_forward");
}

void cross_entropy_backward_cuda_kernel(const tensor_t *global_grad, const tensor_t **cache, tensor_t *dout) {
    const tensor_t *logsm = cache[0], *targets = cache[1];
    const int rows = logsm->shape[0] * logsm->shape[1], C = logsm->shape[2];
    xent_check(xent_sm100_backward(global_grad->t, targets->t, logsm->t, dout->t, rows, C, (void *)get_cuda_stream()),
               "xent_sm100_backward");
}

}  // extern "C"
