// tensor_t adapter between gpt.c's kernel-level attention symbols and libattn_sm100.so.
//
// Drop-in for kernels/src/cuda/Attention.cu of gpt.c: exports attention_forward_cuda_kernel and
// attention_backward_cuda_kernel with the signatures of kernels/src/cuda/Attention.h:9-22, runs
// on the reference runtime's stream (get_cuda_stream, kernels/src/cuda/runtime.cu:39-43),
// allocates its scratch with the reference's stream-ordered allocator (kernels/src/cuda/Alloc.cu)
// and, like every CUDA entry of the reference, prints and exits on error
// (kernels/src/cuda/cuda_common.h:61-68).
//
// Cache convention (set up by the layer): cache[0] = bf16 hi/lo split of qkv, cache[1] = lse
// [B, H, T], cache[2] = private copy of the output [B, T, C], cache[3] = NULL.  The mask
// argument is unused: causality is implicit in the kernels.
#include <stdio.h>
#include <stdlib.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/Alloc.h>
#include <cuda/Attention.h>
#include "attn_sm100.h"
#include "attn_planes.h"

static void attn_check(int rc, const char *what) {
    if (rc != ATTN_OK) {
        printf("[ATTENTION ERROR] %s: %s (status %d)\n", what, attn_sm100_strerror(rc), rc);
        exit(EXIT_FAILURE);
    }
}

extern "C" {

void attention_forward_cuda_kernel(const tensor_t *input, const tensor_t *mask, const int n_heads, tensor_t **cache,
                                   tensor_t *output) {
    (void)mask;
    const int B = input->shape[0], T = input->shape[1], C = input->shape[2] / 3, D = C / n_heads;
    cudaStream_t stream = get_cuda_stream();
    int flags = 0;
    if (D == 64) {
        // When the Linear in front of this layer already wrote the bf16 planes of this very tensor, adopt
        // them as cache[0] (they come from the same allocator) and skip the split pass.
        void *planes = overlay_planes_take(input->t, attn_sm100_saved_bytes(B, T, n_heads, D));
        if (planes) {
            free_cuda(cache[0]->t);
            cache[0]->t = (float *)planes;
            flags = ATTN_FLAG_CORE_ONLY;
        }
    } else {
        overlay_planes_forget(NULL);  // planes are only made for head size 64: nobody will take a pending offer
    }
    attn_check(attn_sm100_forward(input->t, output->t, cache[2]->t, cache[1]->t, cache[0]->t, B, T, n_heads, D, flags,
                                  (void *)stream),
               "attn_sm100_forward");
}

void attention_backward_cuda_kernel(const tensor_t *global_grad, tensor_t **cache, const int n_heads, tensor_t *dout) {
    const int B = global_grad->shape[0], T = global_grad->shape[1], C = global_grad->shape[2], D = C / n_heads;
    cudaStream_t stream = get_cuda_stream();
    void *scratch = alloc_cuda(attn_sm100_backward_scratch_bytes(B, T, n_heads, D));
    attn_check(attn_sm100_backward(cache[0]->t, cache[2]->t, cache[1]->t, global_grad->t, dout->t, scratch, B, T,
                                   n_heads, D, 0, (void *)stream),
               "attn_sm100_backward");
    free_cuda(scratch);  // stream ordered: released after the kernels above have run
}

}  // extern "C"
