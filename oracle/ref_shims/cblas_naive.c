/* Test infrastructure (oracle build only).
 * Plain-loop implementations of the four CBLAS routines the reference evaluator calls,
 * row-major only, with a fixed left-to-right summation order so that the oracle is
 * deterministic and independent of any vendor BLAS. */
#include "external/cblas-prototypes/cblas.h"
#include <stdlib.h>

void cblas_dgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb,
                 int m, int n, int k, double alpha, const double* a, int lda,
                 const double* b, int ldb, double beta, double* c, int ldc)
{
    if (layout != CblasRowMajor) abort();
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            double s = 0.0;
            for (int p = 0; p < k; ++p) {
                const double av = (ta == CblasNoTrans) ? a[i * lda + p] : a[p * lda + i];
                const double bv = (tb == CblasNoTrans) ? b[p * ldb + j] : b[j * ldb + p];
                s += av * bv;
            }
            c[i * ldc + j] = (beta == 0.0) ? alpha * s : alpha * s + beta * c[i * ldc + j];
        }
    }
}

void cblas_dgemv(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE trans, int m, int n, double alpha,
                 const double* a, int lda, const double* x, int incx, double beta,
                 double* y, int incy)
{
    if (layout != CblasRowMajor) abort();
    const int ny = (trans == CblasNoTrans) ? m : n;
    const int nx = (trans == CblasNoTrans) ? n : m;
    for (int i = 0; i < ny; ++i) {
        double s = 0.0;
        for (int p = 0; p < nx; ++p) {
            const double av = (trans == CblasNoTrans) ? a[i * lda + p] : a[p * lda + i];
            s += av * x[p * incx];
        }
        y[i * incy] = (beta == 0.0) ? alpha * s : alpha * s + beta * y[i * incy];
    }
}

void cblas_dcopy(int n, const double* x, int incx, double* y, int incy)
{
    for (int i = 0; i < n; ++i) y[i * incy] = x[i * incx];
}

double cblas_ddot(int n, const double* x, int incx, const double* y, int incy)
{
    double s = 0.0;
    for (int i = 0; i < n; ++i) s += x[i * incx] * y[i * incy];
    return s;
}
