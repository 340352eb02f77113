/*
 * Device dispatch of the attention kernels; drop-in for kernels/src/core/Attention.c of gpt.c
 * (attention_forward_dispatch :6-44, attention_backward_dispatch :46-79).
 *
 * Same checks (every tensor on the same device), except that empty cache slots are allowed:
 * the CUDA path of this build keeps three tensors in the four slots.  CPU tensors go to the
 * reference's CPU kernel, CUDA tensors to the sm_100a library; nothing else is accepted.
 */
#include <core/Attention.h>
#include <cpu/Attention.h>
#include <cuda/Attention.h>
#include "utils.h"

static void check_cache_devices(tensor_t **cache, device_t device) {
    for (int i = 0; i < 4; i++) {
        CHECK_ERROR(cache[i] != NULL && cache[i]->device != device,
                    "Expected every attention cache tensor on the device of the input, but cache[%d] differs", i);
    }
}

void attention_forward_dispatch(const tensor_t *input, const tensor_t *mask, const int n_heads, tensor_t **cache,
                                tensor_t *output) {
    const device_t device = input->device;
    CHECK_ERROR(device != output->device, "Expected input and output tensors on the same device");
    check_cache_devices(cache, device);
    if (device == CPU) {
        CHECK_ERROR(mask->device != CPU, "Expected the attention mask on the CPU for a CPU input");
        attention_forward_cpu_kernel(input, mask, n_heads, cache, output);
    } else if (device == CUDA) {
        attention_forward_cuda_kernel(input, mask, n_heads, cache, output);
    } else {
        CHECK_ERROR(1, "Given device is not supported.");
    }
}

void attention_backward_dispatch(const tensor_t *global_grad, tensor_t **cache, const int n_heads, tensor_t *dout) {
    const device_t device = global_grad->device;
    CHECK_ERROR(device != dout->device, "Expected global_grad and dout tensors on the same device");
    check_cache_devices(cache, device);
    if (device == CPU)
        attention_backward_cpu_kernel(global_grad, cache, n_heads, dout);
    else if (device == CUDA)
        attention_backward_cuda_kernel(global_grad, cache, n_heads, dout);
    else
        CHECK_ERROR(1, "Given device is not supported.");
}
