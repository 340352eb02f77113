/*
 * Raw-pointer drivers around the reference's own CPU kernels either side of the attention layer.
 * TEST INFRASTRUCTURE ONLY.
 *
 * Compiled together with the reference sources where they lie (kernels/src/cpu/{Linear,LayerNorm,
 * CrossEntropyLoss,AdamW,GeLU}.c of gpt.c) into oracle/_ref/libref_ops.so by oracle/build.py; no
 * reference source is copied.  Every entry wraps plain buffers in the reference's tensor_t
 * (include/tensor.h:44-51) and calls the kernel unchanged.  The kernels assume 64-byte aligned data
 * (__builtin_assume_aligned), so every buffer goes through an aligned copy.
 * Return value: 0, or -2 when out of memory.
 */
#include <stdlib.h>
#include <string.h>
#include "tensor.h"
#include <cpu/Linear.h>
#include <cpu/LayerNorm.h>
#include <cpu/CrossEntropyLoss.h>
#include <cpu/AdamW.h>
#include <cpu/GeLU.h>

static void wrap(tensor_t *t, float *data, int ndims, const int *shape) {
    memset(t, 0, sizeof(*t));
    t->t = data;
    t->ndims = ndims;
    t->length = 1;
    for (int i = 0; i < ndims; i++) { t->shape[i] = shape[i]; t->length *= shape[i]; }
    t->device = CPU;
}

/* aligned private copy of n floats (zero-filled when src is NULL) */
static float *dup64(const float *src, size_t n) {
    size_t bytes = (n * sizeof(float) + 63) & ~(size_t)63;
    float *p = (float *)aligned_alloc(64, bytes ? bytes : 64);
    if (!p) return NULL;
    if (src) memcpy(p, src, n * sizeof(float)); else memset(p, 0, bytes ? bytes : 64);
    return p;
}

/* y[M,N] = x[M,K] w[N,K]^T (+ b) */
int ref_linear_forward(const float *x, const float *w, const float *b, float *y, int M, int N, int K) {
    float *ax = dup64(x, (size_t)M * K), *aw = dup64(w, (size_t)N * K), *ab = b ? dup64(b, N) : NULL, *ay = dup64(NULL, (size_t)M * N);
    if (!ax || !aw || !ay || (b && !ab)) return -2;
    tensor_t tx, tw, tb, ty;
    const int sx[3] = {1, M, K}, sw[2] = {N, K}, sb[1] = {N}, sy[3] = {1, M, N};
    wrap(&tx, ax, 3, sx); wrap(&tw, aw, 2, sw); wrap(&ty, ay, 3, sy);
    if (b) wrap(&tb, ab, 1, sb);
    linear_forward_cpu_kernel(&tw, b ? &tb : NULL, &tx, &ty);
    memcpy(y, ay, (size_t)M * N * sizeof(float));
    free(ax); free(aw); free(ab); free(ay);
    return 0;
}

/* dx = dy w (overwritten); dw += dy^T x; db += colsum(dy) (db may be NULL): dw and db are in/out */
int ref_linear_backward(const float *dy, const float *x, const float *w, float *dx, float *dw, float *db, int M, int N, int K) {
    float *ag = dup64(dy, (size_t)M * N), *ax = dup64(x, (size_t)M * K), *aw = dup64(w, (size_t)N * K);
    float *adx = dup64(NULL, (size_t)M * K), *adw = dup64(dw, (size_t)N * K), *adb = db ? dup64(db, N) : NULL;
    if (!ag || !ax || !aw || !adx || !adw || (db && !adb)) return -2;
    tensor_t tg, tx, tw, tdx, tdw, tdb;
    const int sg[3] = {1, M, N}, sx[3] = {1, M, K}, sw[2] = {N, K}, sb[1] = {N};
    wrap(&tg, ag, 3, sg); wrap(&tx, ax, 3, sx); wrap(&tw, aw, 2, sw); wrap(&tdx, adx, 3, sx); wrap(&tdw, adw, 2, sw);
    if (db) wrap(&tdb, adb, 1, sb);
    linear_backward_cpu_kernel(&tg, &tx, &tw, &tdw, db ? &tdb : NULL, &tdx);
    memcpy(dx, adx, (size_t)M * K * sizeof(float));
    memcpy(dw, adw, (size_t)N * K * sizeof(float));
    if (db) memcpy(db, adb, (size_t)N * sizeof(float));
    free(ag); free(ax); free(aw); free(adx); free(adw); free(adb);
    return 0;
}

int ref_layernorm_forward(const float *x, const float *w, const float *b, float eps, float *y, float *mean, float *rstd,
                          int rows, int C) {
    float *ax = dup64(x, (size_t)rows * C), *aw = dup64(w, C), *ab = b ? dup64(b, C) : NULL;
    float *ay = dup64(NULL, (size_t)rows * C), *am = dup64(NULL, rows), *ar = dup64(NULL, rows);
    if (!ax || !aw || !ay || !am || !ar || (b && !ab)) return -2;
    tensor_t tx, tw, tb, ty, tm, tr;
    const int sx[3] = {1, rows, C}, sc[1] = {C}, sr[2] = {1, rows};
    wrap(&tx, ax, 3, sx); wrap(&tw, aw, 1, sc); wrap(&ty, ay, 3, sx); wrap(&tm, am, 2, sr); wrap(&tr, ar, 2, sr);
    if (b) wrap(&tb, ab, 1, sc);
    tensor_t *cache[3] = {&tm, &tr, &tx};
    layer_norm_forward_cpu_kernel(&tw, b ? &tb : NULL, &tx, eps, cache, &ty);
    memcpy(y, ay, (size_t)rows * C * sizeof(float));
    memcpy(mean, am, rows * sizeof(float));
    memcpy(rstd, ar, rows * sizeof(float));
    free(ax); free(aw); free(ab); free(ay); free(am); free(ar);
    return 0;
}

/* dw, db (may be NULL), dx are in/out: the kernel accumulates on top of their contents */
int ref_layernorm_backward(const float *dy, const float *x, const float *mean, const float *rstd, const float *w, float *dw,
                           float *db, float *dx, int rows, int C) {
    float *ag = dup64(dy, (size_t)rows * C), *ax = dup64(x, (size_t)rows * C), *am = dup64(mean, rows), *ar = dup64(rstd, rows);
    float *aw = dup64(w, C), *adw = dup64(dw, C), *adb = db ? dup64(db, C) : NULL, *adx = dup64(dx, (size_t)rows * C);
    if (!ag || !ax || !am || !ar || !aw || !adw || !adx || (db && !adb)) return -2;
    tensor_t tg, tx, tm, tr, tw, tdw, tdb, tdx;
    const int sx[3] = {1, rows, C}, sc[1] = {C}, sr[2] = {1, rows};
    wrap(&tg, ag, 3, sx); wrap(&tx, ax, 3, sx); wrap(&tm, am, 2, sr); wrap(&tr, ar, 2, sr); wrap(&tw, aw, 1, sc);
    wrap(&tdw, adw, 1, sc); wrap(&tdx, adx, 3, sx);
    if (db) wrap(&tdb, adb, 1, sc);
    const tensor_t *cache[3] = {&tm, &tr, &tx};
    layer_norm_backward_cpu_kernel(&tg, cache, &tw, &tdw, db ? &tdb : NULL, &tdx);
    memcpy(dw, adw, C * sizeof(float));
    if (db) memcpy(db, adb, C * sizeof(float));
    memcpy(dx, adx, (size_t)rows * C * sizeof(float));
    free(ag); free(ax); free(am); free(ar); free(aw); free(adw); free(adb); free(adx);
    return 0;
}

/* logsm [rows,C] and loss[0] are written (the CPU kernel assigns the loss) */
int ref_xent_forward(const float *logits, const float *targets, float *logsm, float *loss, int rows, int C) {
    float *al = dup64(logits, (size_t)rows * C), *at = dup64(targets, rows), *as = dup64(NULL, (size_t)rows * C), *ao = dup64(NULL, 1);
    if (!al || !at || !as || !ao) return -2;
    tensor_t tl, tt, ts, to;
    const int sl[3] = {1, rows, C}, st[2] = {1, rows}, so[1] = {1};
    wrap(&tl, al, 3, sl); wrap(&tt, at, 2, st); wrap(&ts, as, 3, sl); wrap(&to, ao, 1, so);
    tensor_t *cache[2] = {&ts, &tt};
    cross_entropy_forward_cpu_kernel(&tl, &tt, cache, &to);
    memcpy(logsm, as, (size_t)rows * C * sizeof(float));
    loss[0] = ao[0];
    free(al); free(at); free(as); free(ao);
    return 0;
}

/* dout [rows,C] is in/out: the kernel works on what it holds */
int ref_xent_backward(const float *g, const float *targets, const float *logsm, float *dout, int rows, int C) {
    float *ag = dup64(g, rows), *at = dup64(targets, rows), *as = dup64(logsm, (size_t)rows * C), *ad = dup64(dout, (size_t)rows * C);
    if (!ag || !at || !as || !ad) return -2;
    tensor_t tg, tt, ts, td;
    const int sl[3] = {1, rows, C}, st[2] = {1, rows};
    wrap(&tg, ag, 2, st); wrap(&tt, at, 2, st); wrap(&ts, as, 3, sl); wrap(&td, ad, 3, sl);
    const tensor_t *cache[2] = {&ts, &tt};
    cross_entropy_backward_cpu_kernel(&tg, cache, &td);
    memcpy(dout, ad, (size_t)rows * C * sizeof(float));
    free(ag); free(at); free(as); free(ad);
    return 0;
}

/* one tensor of n elements: p, m, v are in/out */
int ref_adamw_step(float *p, const float *g, float *m, float *v, int n, float lr, float b1, float b2, float wd, float eps, int step) {
    float *ap = dup64(p, n), *ag = dup64(g, n), *am = dup64(m, n), *av = dup64(v, n);
    if (!ap || !ag || !am || !av) return -2;
    tensor_t tp, tg, tm, tv;
    const int s[1] = {n};
    wrap(&tp, ap, 1, s); wrap(&tg, ag, 1, s); wrap(&tm, am, 1, s); wrap(&tv, av, 1, s);
    tensor_t *pp[1] = {&tp}, *gg[1] = {&tg}, *mm[1] = {&tm}, *vv[1] = {&tv};
    step_adamW_cpu_kernel(pp, gg, mm, vv, 1, lr, b1, b2, wd, eps, step);
    memcpy(p, ap, n * sizeof(float)); memcpy(m, am, n * sizeof(float)); memcpy(v, av, n * sizeof(float));
    free(ap); free(ag); free(am); free(av);
    return 0;
}

int ref_gelu_forward(const float *x, float *y, int n) {
    float *ax = dup64(x, n), *ay = dup64(NULL, n);
    if (!ax || !ay) return -2;
    tensor_t tx, ty;
    const int s[1] = {n};
    wrap(&tx, ax, 1, s); wrap(&ty, ay, 1, s);
    gelu_forward_cpu_kernel(&tx, &ty);
    memcpy(y, ay, n * sizeof(float));
    free(ax); free(ay);
    return 0;
}

int ref_gelu_backward(const float *g, const float *x, float *dx, int n) {
    float *ag = dup64(g, n), *ax = dup64(x, n), *ad = dup64(NULL, n);
    if (!ag || !ax || !ad) return -2;
    tensor_t tg, tx, td;
    const int s[1] = {n};
    wrap(&tg, ag, 1, s); wrap(&tx, ax, 1, s); wrap(&td, ad, 1, s);
    gelu_backward_cpu_kernel(&tg, &tx, &td);
    memcpy(dx, ad, n * sizeof(float));
    free(ag); free(ax); free(ad);
    return 0;
}
