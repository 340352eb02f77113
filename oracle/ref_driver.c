/*
 * Raw-pointer driver around the reference's own CPU attention kernel.  TEST INFRASTRUCTURE ONLY.
 *
 * Compiled together with the reference sources where they lie (kernels/src/cpu/Attention.c and
 * kernels/src/cpu/Alloc.c of gpt.c) into oracle/_ref/libref_attention.so by oracle/build.py; no
 * reference source is copied.  It wraps plain buffers in the reference's tensor_t
 * (include/tensor.h:44-51), builds the lower-triangular ones mask the layer constructor makes
 * (src/attention.c:28-35) and the four caches the layer allocates (src/attention.c:105-120),
 * then calls attention_forward_cpu_kernel / attention_backward_cpu_kernel unchanged.
 *
 * The backward kernel overwrites its incoming gradient with dq and the V cache with dk
 * (kernels/src/cpu/Attention.c:198-201), so the driver hands it a private copy of dout.
 */
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <cblas.h>
#include "tensor.h"
#include <cpu/Attention.h>

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static void wrap(tensor_t *t, float *data, int ndims, const int *shape) {
    memset(t, 0, sizeof(*t));
    t->t = data;
    t->ndims = ndims;
    t->length = 1;
    for (int i = 0; i < ndims; i++) { t->shape[i] = shape[i]; t->length *= shape[i]; }
    t->device = CPU;
}

static float *alloc64(size_t n) {
    size_t bytes = (n * sizeof(float) + 63) & ~(size_t)63;
    return (float *)aligned_alloc(64, bytes);
}

void ref_set_num_threads(int n) { openblas_set_num_threads(n); }
int ref_get_num_threads(void) { return openblas_get_num_threads(); }
const char *ref_blas_config(void) { return openblas_get_config(); }

/*
 * x [B,T,3C] -> out [B,T,C]; when dout is not NULL also dx [B,T,3C].  seconds[0], seconds[1]
 * receive the wall time of the forward and backward kernel calls (buffers already allocated).
 * Returns 0, -1 on a bad argument, -2 when out of memory.
 */
int ref_attention_run(const float *x, const float *dout, float *out, float *dx,
                      int B, int T, int H, int D, double *seconds) {
    if (!x || !out || B <= 0 || T <= 0 || H <= 0 || D <= 0) return -1;
    if (dout && !dx) return -1;
    const int C = H * D;
    const size_t nx = (size_t)B * T * 3 * C, no = (size_t)B * T * C;
    const size_t nh = (size_t)B * H * T * D, na = (size_t)B * H * T * T;
    float *xin = alloc64(nx), *mask = alloc64((size_t)T * T);
    float *q = alloc64(nh), *k = alloc64(nh), *v = alloc64(nh), *att = alloc64(na);
    float *o = alloc64(no), *g = dout ? alloc64(no) : NULL, *d = dout ? alloc64(nx) : NULL;
    int rc = 0;
    if (!xin || !mask || !q || !k || !v || !att || !o || (dout && (!g || !d))) { rc = -2; goto done; }

    memcpy(xin, x, nx * sizeof(float));
    for (int i = 0; i < T; i++)
        for (int j = 0; j < T; j++) mask[(size_t)i * T + j] = j <= i ? 1.0f : 0.0f;

    {
        tensor_t tx, tmask, tq, tk, tv, tatt, tout, tg, td;
        const int sx[3] = {B, T, 3 * C}, sm[2] = {T, T}, sh[4] = {B, H, T, D};
        const int sa[4] = {B, H, T, T}, so[3] = {B, T, C};
        wrap(&tx, xin, 3, sx); wrap(&tmask, mask, 2, sm);
        wrap(&tq, q, 4, sh); wrap(&tk, k, 4, sh); wrap(&tv, v, 4, sh);
        wrap(&tatt, att, 4, sa); wrap(&tout, o, 3, so);
        tensor_t *cache[4] = {&tq, &tk, &tv, &tatt};

        double t0 = now_s();
        attention_forward_cpu_kernel(&tx, &tmask, H, cache, &tout);
        double t1 = now_s();
        if (seconds) seconds[0] = t1 - t0;
        memcpy(out, o, no * sizeof(float));

        if (dout) {
            memcpy(g, dout, no * sizeof(float));
            memset(d, 0, nx * sizeof(float));
            wrap(&tg, g, 3, so); wrap(&td, d, 3, sx);
            t0 = now_s();
            attention_backward_cpu_kernel(&tg, cache, H, &td);
            t1 = now_s();
            if (seconds) seconds[1] = t1 - t0;
            memcpy(dx, d, nx * sizeof(float));
        }
    }
done:
    free(xin); free(mask); free(q); free(k); free(v); free(att); free(o); free(g); free(d);
    return rc;
}
