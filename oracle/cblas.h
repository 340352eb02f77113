/*
 * Minimal CBLAS declarations for building the reference CPU attention kernel out of tree.
 * TEST INFRASTRUCTURE ONLY (see attention_oracle.c).
 *
 * The reference takes <cblas.h> from an OpenBLAS submodule that is not vendored
 * (third_party/OpenBLAS is empty, version unpinned).  The only CBLAS entry point on the
 * attention path is cblas_sgemm (kernels/src/cpu/Attention.c:126,149,226,234,260,268); the rest
 * of the library also calls cblas_scopy and cblas_saxpy (kernels/src/cpu/Tensor.c:68,78), which
 * are declared for the whole-library build used by the layer tests.
 * The enum values are the ones fixed by the CBLAS interface standard.
 *
 * REF_BLAS_PREFIX selects the symbol prefix of the OpenBLAS build that is linked: the copy
 * bundled with SciPy exports scipy_cblas_sgemm, a stock build exports cblas_sgemm.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };

#ifdef REF_BLAS_SCIPY
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_scopy scipy_cblas_scopy
#define cblas_saxpy scipy_cblas_saxpy
#define openblas_set_num_threads scipy_openblas_set_num_threads
#define openblas_get_num_threads scipy_openblas_get_num_threads
#define openblas_get_config scipy_openblas_get_config
#endif

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                 int M, int N, int K, float alpha, const float *A, int lda,
                 const float *B, int ldb, float beta, float *C, int ldc);
void cblas_scopy(int n, const float *x, int incx, float *y, int incy);
void cblas_saxpy(int n, float alpha, const float *x, int incx, float *y, int incy);
void openblas_set_num_threads(int n);
int openblas_get_num_threads(void);
char *openblas_get_config(void);

#ifdef __cplusplus
}
#endif
