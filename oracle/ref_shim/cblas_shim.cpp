// Plain-loop definitions of the routines declared in cblas.h beside this file. TEST INFRASTRUCTURE ONLY.
#include "cblas.h"

extern "C" void cblas_sscal(int n, float alpha, float* x, int incx) {
    for (int i = 0; i < n; ++i) x[i * incx] *= alpha;
}
extern "C" float cblas_sdot(int n, const float* x, int incx, const float* y, int incy) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += x[i * incx] * y[i * incy];
    return s;
}
extern "C" void cblas_saxpy(int n, float alpha, const float* x, int incx, float* y, int incy) {
    for (int i = 0; i < n; ++i) y[i * incy] += alpha * x[i * incx];
}
