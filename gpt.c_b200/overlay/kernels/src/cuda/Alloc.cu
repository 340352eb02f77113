// Stream-ordered device allocator for gpt.c: drop-in for kernels/src/cuda/Alloc.cu (alloc_cuda /
// free_cuda, declared in kernels/src/cuda/Alloc.h), same semantics (cudaMallocAsync / cudaFreeAsync
// on the runtime's stream, print and exit on error).
//
// One difference: on first use the device's default memory pool is told to keep what is freed
// (release threshold = unlimited).  With the default threshold of zero the pool hands every free
// block back to the driver at each stream synchronisation, and gpt.c synchronises at least twice per
// training step (loss read-back, AdamW pointer table, kernels/src/cuda/AdamW.cu:97-112), so each step
// re-acquired all of its hundreds of temporaries from the driver.  The setting lives in this process's
// pool object only; nothing on the GPU outlasts the process.
#include <stdint.h>
#include <cuda/cuda_common.h>
#include <cuda/runtime.cuh>
#include <cuda/Alloc.h>
#include "attn_planes.h"

static void keep_freed_memory_once(void) {
    static int done = 0;
    if (done) return;
    done = 1;
    int dev = 0;
    cudaMemPool_t pool;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
        uint64_t threshold = UINT64_MAX;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold);
    }
}

extern "C" {

void *alloc_cuda(const size_t size) {
    keep_freed_memory_once();
    void *ptr = NULL;
    cudaCheck(cudaMallocAsync(&ptr, size, get_cuda_stream()));
    return ptr;
}

void free_cuda(void *ptr) {
    if (ptr == NULL) return;
    overlay_planes_forget(ptr);  // bf16 planes offered for this tensor die with it (its address will be reused)
    cudaCheck(cudaFreeAsync(ptr, get_cuda_stream()));
}

}  // extern "C"
