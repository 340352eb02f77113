// tensor_t adapter between gpt.c's kernel-level AdamW symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/AdamW.cu of gpt.c: exports step_adamW_cuda_kernel and
// zero_grad_adamW_cuda_kernel with the signatures of kernels/src/cuda/AdamW.h:10-24, runs on the
// reference runtime's stream and prints and exits on error like every CUDA entry of the reference.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/Tensor.h>
#include <cuda/AdamW.h>
#include "adamw_sm100.h"

extern "C" {

void step_adamW_cuda_kernel(tensor_t **parameters, tensor_t **gradients, tensor_t **m, tensor_t **v, const int n,
                            const float lr, const float beta1, const float beta2, const float weight_decay, const float eps,
                            const int step) {
    float **ptrs = (float **)malloc((size_t)n * 4 * sizeof(float *));
    int *lengths = (int *)malloc((size_t)n * sizeof(int));
    if (!ptrs || !lengths) {
        printf("[ADAMW ERROR] out of host memory\n");
        exit(EXIT_FAILURE);
    }
    for (int i = 0; i < n; i++) {
        ptrs[i] = parameters[i]->t;
        ptrs[n + i] = gradients[i]->t;
        ptrs[2 * n + i] = m[i]->t;
        ptrs[3 * n + i] = v[i]->t;
        lengths[i] = parameters[i]->length;
    }
    const int rc = adamw_sm100_step(ptrs, ptrs + n, ptrs + 2 * n, ptrs + 3 * n, lengths, n, lr, beta1, beta2, weight_decay,
                                    eps, step, (void *)get_cuda_stream());
    free(ptrs);
    free(lengths);
    if (rc != ATTN_OK) {
        printf("[ADAMW ERROR] adamw_sm100_step: %s (status %d)\n", attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

void zero_grad_adamW_cuda_kernel(tensor_t **gradients, const int n) {
    for (int i = 0; i < n; i++) zeros_tensor_data_cuda(gradients[i]);
}

}  // extern "C"
