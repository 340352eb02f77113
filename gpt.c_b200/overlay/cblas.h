/*
 * The three CBLAS entry points gpt.c's CPU kernels call, for building gpt.c where no OpenBLAS
 * source tree is checked out (gpt.c takes <cblas.h> from a submodule, third_party/OpenBLAS):
 * cblas_sgemm (kernels/src/cpu/Attention.c:126, kernels/src/cpu/Linear.c:15, kernels/src/cpu/Tensor.c:98),
 * cblas_scopy and cblas_saxpy (kernels/src/cpu/Tensor.c:68,78).  Enum values are those of the CBLAS
 * interface standard.  With GPTC_BLAS_SCIPY the names map to the prefixed symbols of the OpenBLAS
 * that ships inside the SciPy wheel.
 */
#ifndef GPTC_OVERLAY_CBLAS_H
#define GPTC_OVERLAY_CBLAS_H

#ifdef __cplusplus
extern "C" {
#endif

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };

#ifdef GPTC_BLAS_SCIPY
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_scopy scipy_cblas_scopy
#define cblas_saxpy scipy_cblas_saxpy
#endif

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE trans_a, enum CBLAS_TRANSPOSE trans_b, int m, int n,
                 int k, float alpha, const float *a, int lda, const float *b, int ldb, float beta, float *c, int ldc);
void cblas_scopy(int n, const float *x, int incx, float *y, int incy);
void cblas_saxpy(int n, float alpha, const float *x, int incx, float *y, int incy);

#ifdef __cplusplus
}
#endif

#endif
