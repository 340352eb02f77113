/*
 * Drives the Attention layer of gpt.c through its public API (include/attention.h:42-61):
 * construct, move to the device, forward, backward, free.  Linked against a libgpt.so that was
 * built from the gpt.c sources with this repository's overlay (the sm_100a attention), or against
 * an unmodified build of the reference, so the same program exercises both.
 *
 *   layer_driver <cpu|cuda> B T C n_heads x.bin dout.bin out.bin dx.bin [repeat [keep-pool]]
 *
 * x.bin holds B*T*3C floats, dout.bin B*T*C floats (raw fp32).  out.bin / dx.bin receive the layer
 * output and the gradient with respect to x.  With repeat > 1 the forward+backward pair is run
 * that many times and the mean wall time per pair (after one warm-up pair) is printed.
 *
 * gpt.c allocates every activation with cudaMallocAsync and frees it with cudaFreeAsync
 * (kernels/src/cuda/Alloc.cu:9-20); with the default pool settings each synchronisation hands the
 * freed memory back to the driver and the next pair pays for it again.  "keep-pool" (CUDA builds of
 * this driver only) raises the release threshold of the device's default memory pool before the
 * timed loop, so that the figure is the layer's kernels and not the allocator: the same library,
 * the same kernels, a process-wide pool attribute.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include "attention.h"
#include "runtime.h"
#include "tensor.h"
#include "utils.h"
#ifdef LAYER_DRIVER_CUDART
#include <cuda_runtime_api.h>
#include <stdint.h>
#endif

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static tensor_t *load(const char *path, const int *shape, int n) {
    FILE *fp = fopenCheck(path, "rb");
    tensor_t *t = tensor_load(fp, shape, n, CPU);
    fcloseCheck(fp);
    return t;
}

static void store(const char *path, tensor_t *t) {
    FILE *fp = fopenCheck(path, "wb");
    tensor_save(fp, t);
    fcloseCheck(fp);
}

int main(int argc, char **argv) {
    if (argc < 10) {
        fprintf(stderr, "usage: %s <cpu|cuda> B T C n_heads x.bin dout.bin out.bin dx.bin [repeat]\n", argv[0]);
        return 2;
    }
    const device_t device = strcmp(argv[1], "cuda") == 0 ? CUDA : CPU;
    const int B = atoi(argv[2]), T = atoi(argv[3]), C = atoi(argv[4]), H = atoi(argv[5]);
    const int repeat = argc > 10 ? atoi(argv[10]) : 1;
    const int keep_pool = argc > 11 && strcmp(argv[11], "keep-pool") == 0;
    const int xs[3] = {B, T, 3 * C}, gs[3] = {B, T, C};

    runtime_init(device);
    attention_t *attn = Attention(C, H, T);
    attn->to(attn, device);
    if (keep_pool) {
#ifdef LAYER_DRIVER_CUDART
        cudaMemPool_t pool;
        uint64_t keep = UINT64_MAX;
        if (device != CUDA || cudaDeviceGetDefaultMemPool(&pool, 0) != cudaSuccess ||
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) {
            fprintf(stderr, "layer_driver: keep-pool needs the cuda device\n");
            return 2;
        }
#else
        fprintf(stderr, "layer_driver: built without the CUDA runtime, keep-pool is not available\n");
        return 2;
#endif
    }

    double total = 0.0;
    for (int r = 0; r < repeat + (repeat > 1 ? 1 : 0); r++) {
        tensor_t *x = load(argv[6], xs, 3);
        tensor_t *g = load(argv[7], gs, 3);
        x->to(x, device);
        g->to(g, device);
        synchronize(device);
        const double t0 = now_s();
        tensor_t *out = attn->forward(attn, x); /* consumes x */
        tensor_t *out_keep = NULL;
        if (r == 0) { /* the next layer would own `out`; keep a host copy before it is freed */
            out_keep = create_tensor(gs, 3, device);
            tensor_copy(out_keep, out);
        }
        free_tensor(out);
        tensor_t *dx = attn->backward(attn, g); /* consumes g and the caches */
        synchronize(device);
        const double t1 = now_s();
        if (r > 0 || repeat == 1) total += t1 - t0;
        if (r == 0) {
            out_keep->to(out_keep, CPU);
            dx->to(dx, CPU);
            store(argv[8], out_keep);
            store(argv[9], dx);
            free_tensor(out_keep);
        }
        free_tensor(dx);
    }
    printf("layer_driver: device=%s B=%d T=%d C=%d H=%d pairs=%d keep_pool=%d mean_ms=%.4f\n", argv[1], B, T, C, H, repeat,
           keep_pool, 1e3 * total / (repeat > 0 ? repeat : 1));
    attn->free_layer(attn);
    runtime_destroy(device);
    return 0;
}
