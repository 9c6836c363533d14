/* The three host BLAS routines the reference's RVQ source names in its TRAINING code
 * (cblas_sscal / cblas_sdot / cblas_saxpy), so that the file compiles without a BLAS package.
 * RVQ::search, the only part the checker's driver runs, calls none of them. TEST INFRASTRUCTURE ONLY. */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
void cblas_sscal(int n, float alpha, float* x, int incx);
float cblas_sdot(int n, const float* x, int incx, const float* y, int incy);
void cblas_saxpy(int n, float alpha, const float* x, int incx, float* y, int incy);
#ifdef __cplusplus
}
#endif
