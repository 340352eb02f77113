/*
 * CPU oracle for the causal self-attention layer of gpt.c.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference CPU attention kernel.  It is
 * the checker the CUDA path is compared against; nothing in the product path may call it.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py) against
 *   - golden vectors produced by running the reference's own compiled CPU kernel
 *     (kernels/src/cpu/Attention.c) and its PyTorch twin (model.py) on fixed inputs,
 *     committed under tests/golden/ with the script that made them, and
 *   - the reference kernel itself whenever oracle/_ref/libref_attention.so is present.
 *
 * Reference functions restated here (paths are relative to the gpt.c project root):
 *   oracle_attention_forward   <- attention_forward_cpu_kernel   kernels/src/cpu/Attention.c:46-167
 *                                 _softmax_forward                kernels/src/cpu/Attention.c:8-29
 *   oracle_attention_backward  <- attention_backward_cpu_kernel  kernels/src/cpu/Attention.c:169-301
 *                                 _softmax_backward               kernels/src/cpu/Attention.c:31-44
 *
 * Layout (same as the reference): x is the fused QKV tensor [B, T, 3C] with C = H*D, where
 * q = x[..., 0:C], k = x[..., C:2C], v = x[..., 2C:3C] and head h owns columns h*D..h*D+D-1 of
 * each third.  out and dout are [B, T, C]; dx is [B, T, 3C] = [dq | dk | dv] per token.
 *
 * Differences from the reference that do not change results beyond fp32 rounding:
 *   - the reference fills the upper triangle with -inf and lets exp() produce exact zeros
 *     (Attention.c:135-144); here columns j > i are simply never visited, which is the same sum;
 *   - the reference runs six SGEMMs per (batch, head) through OpenBLAS; here the contractions
 *     are plain loops with double accumulators, so the result does not depend on a BLAS build;
 *   - (batch, head) pairs are independent and are spread over OpenMP threads.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* Number of worker threads the oracle will use (1 when built without OpenMP). */
int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static inline const float *row_ptr(const float *base, int b, int t, int T, int ld, int col) {
    return base + ((size_t)b * T + t) * (size_t)ld + col;
}

/* att[i][j] for j <= i of one (b, h): scale * q_i . k_j, then a numerically safe row softmax.
 * Follows Attention.c:125-144 (SGEMM with alpha = scale, mask, softmax). */
static void head_probabilities(const float *x, int b, int h, int T, int C, int D, float scale,
                               float *att /* [T*T], row-major, upper triangle left at 0 */) {
    const int C3 = 3 * C;
    for (int i = 0; i < T; i++) {
        const float *qi = row_ptr(x, b, i, T, C3, h * D);
        float *arow = att + (size_t)i * T;
        float m = -INFINITY;
        for (int j = 0; j <= i; j++) {
            const float *kj = row_ptr(x, b, j, T, C3, C + h * D);
            double acc = 0.0;
            for (int d = 0; d < D; d++) acc += (double)qi[d] * (double)kj[d];
            float s = (float)(acc * (double)scale);
            arow[j] = s;
            m = fmaxf(m, s);
        }
        double sum = 0.0;
        for (int j = 0; j <= i; j++) {
            float e = expf(arow[j] - m);
            arow[j] = e;
            sum += e;
        }
        float inv = (float)(1.0 / sum);
        for (int j = 0; j <= i; j++) arow[j] *= inv;
        for (int j = i + 1; j < T; j++) arow[j] = 0.0f;
    }
}

/*
 * Forward.  out[b, i, h*D + d] = sum_{j<=i} softmax_j(scale * q_i.k_j) * v_j[d]
 * (Attention.c:146-164: att @ v then the transpose back to [B, T, C]).
 * lse, when not NULL, receives log(sum_j exp(s_ij)) per (b, h, i) as [B, H, T]; the reference
 * does not produce it, it is here so the log-sum-exp saved by the CUDA forward can be checked.
 * Returns 0, or -1 on a bad argument.
 */
int oracle_attention_forward(const float *x, float *out, float *lse, int B, int T, int H, int D) {
    if (!x || !out || B <= 0 || T <= 0 || H <= 0 || D <= 0) return -1;
    const int C = H * D, C3 = 3 * C;
    const float scale = 1.0f / sqrtf((float)D);
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        float *srow = (float *)malloc((size_t)T * sizeof(float));
        double *acc = (double *)malloc((size_t)D * sizeof(double));
        if (!srow || !acc) { failed = 1; free(srow); free(acc); continue; }
        for (int i = 0; i < T; i++) {
            const float *qi = row_ptr(x, b, i, T, C3, h * D);
            float m = -INFINITY;
            for (int j = 0; j <= i; j++) {
                const float *kj = row_ptr(x, b, j, T, C3, C + h * D);
                double dot = 0.0;
                for (int d = 0; d < D; d++) dot += (double)qi[d] * (double)kj[d];
                srow[j] = (float)(dot * (double)scale);
                m = fmaxf(m, srow[j]);
            }
            double sum = 0.0;
            for (int j = 0; j <= i; j++) { srow[j] = expf(srow[j] - m); sum += srow[j]; }
            const float inv = (float)(1.0 / sum);
            for (int d = 0; d < D; d++) acc[d] = 0.0;
            for (int j = 0; j <= i; j++) {
                const float p = srow[j] * inv;
                const float *vj = row_ptr(x, b, j, T, C3, 2 * C + h * D);
                for (int d = 0; d < D; d++) acc[d] += (double)p * (double)vj[d];
            }
            float *oi = out + ((size_t)b * T + i) * C + h * D;
            for (int d = 0; d < D; d++) oi[d] = (float)acc[d];
            if (lse) lse[((size_t)b * H + h) * T + i] = m + (float)log(sum);
        }
        free(srow); free(acc);
    }
    return failed ? -2 : 0;
}

/*
 * Backward.  Given dout = dL/dout [B, T, C], writes dx = [dq | dk | dv] [B, T, 3C]
 * (every element assigned, as the reference CPU kernel does at Attention.c:277-297).
 *   datt = dout_h @ v^T ; dv = att^T @ dout_h                      (Attention.c:212-241)
 *   dpre[i][j] = (datt[i][j] - sum_k datt[i][k] att[i][k]) att[i][j]  (Attention.c:31-44, 243)
 *   dq = scale * dpre @ k ; dk = scale * dpre^T @ q                (Attention.c:245-275)
 * The reference reads att from the forward cache; it is recomputed here from x, which gives
 * the same numbers.  Returns 0, -1 on a bad argument, -2 when out of memory.
 */
int oracle_attention_backward(const float *x, const float *dout, float *dx, int B, int T, int H, int D) {
    if (!x || !dout || !dx || B <= 0 || T <= 0 || H <= 0 || D <= 0) return -1;
    const int C = H * D, C3 = 3 * C;
    const float scale = 1.0f / sqrtf((float)D);
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        float *att = (float *)malloc((size_t)T * T * sizeof(float));
        float *dpre = (float *)malloc((size_t)T * T * sizeof(float));
        double *acc = (double *)malloc((size_t)2 * D * sizeof(double));
        if (!att || !dpre || !acc) { failed = 1; free(att); free(dpre); free(acc); continue; }
        head_probabilities(x, b, h, T, C, D, scale, att);

        /* datt and the softmax backward, row by row */
        for (int i = 0; i < T; i++) {
            const float *doi = dout + ((size_t)b * T + i) * C + h * D;
            const float *arow = att + (size_t)i * T;
            float *drow = dpre + (size_t)i * T;
            double rs = 0.0;
            for (int j = 0; j <= i; j++) {
                const float *vj = row_ptr(x, b, j, T, C3, 2 * C + h * D);
                double dot = 0.0;
                for (int d = 0; d < D; d++) dot += (double)doi[d] * (double)vj[d];
                drow[j] = (float)dot;
                rs += dot * (double)arow[j];
            }
            const float rsf = (float)rs;
            for (int j = 0; j <= i; j++) drow[j] = (drow[j] - rsf) * arow[j];
            for (int j = i + 1; j < T; j++) drow[j] = 0.0f;
        }

        /* dq_i = scale * sum_{j<=i} dpre[i][j] k_j */
        for (int i = 0; i < T; i++) {
            const float *drow = dpre + (size_t)i * T;
            for (int d = 0; d < D; d++) acc[d] = 0.0;
            for (int j = 0; j <= i; j++) {
                const float *kj = row_ptr(x, b, j, T, C3, C + h * D);
                const double w = (double)drow[j];
                for (int d = 0; d < D; d++) acc[d] += w * (double)kj[d];
            }
            float *dq = dx + ((size_t)b * T + i) * C3 + h * D;
            for (int d = 0; d < D; d++) dq[d] = (float)(acc[d] * (double)scale);
        }

        /* dk_j = scale * sum_{i>=j} dpre[i][j] q_i ;  dv_j = sum_{i>=j} att[i][j] dout_i */
        for (int j = 0; j < T; j++) {
            double *ak = acc, *av = acc + D;
            for (int d = 0; d < D; d++) { ak[d] = 0.0; av[d] = 0.0; }
            for (int i = j; i < T; i++) {
                const float *qi = row_ptr(x, b, i, T, C3, h * D);
                const float *doi = dout + ((size_t)b * T + i) * C + h * D;
                const double wk = (double)dpre[(size_t)i * T + j];
                const double wv = (double)att[(size_t)i * T + j];
                for (int d = 0; d < D; d++) { ak[d] += wk * (double)qi[d]; av[d] += wv * (double)doi[d]; }
            }
            float *dk = dx + ((size_t)b * T + j) * C3 + C + h * D;
            float *dv = dx + ((size_t)b * T + j) * C3 + 2 * C + h * D;
            for (int d = 0; d < D; d++) { dk[d] = (float)(ak[d] * (double)scale); dv[d] = (float)av[d]; }
        }
        free(att); free(dpre); free(acc);
    }
    return failed ? -2 : 0;
}
