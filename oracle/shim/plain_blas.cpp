// Plain-loop CBLAS subset backing the oracle build of the reference's serial
// evaluator (test infrastructure only).  Row-major and column-major, with and
// without transposition; no blocking, no threads.
#include "external/cblas-prototypes/cblas.h"
#include <vector>

namespace {
template <typename T>
void gemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
          T alpha, const T* a, int lda, const T* b, int ldb, T beta, T* c, int ldc)
{
    if (order == CblasColMajor) {  // C^T = B^T A^T in row-major terms
        gemm<T>(CblasRowMajor, tb, ta, n, m, k, alpha, b, ldb, a, lda, beta, c, ldc);
        return;
    }
    const bool at = ta != CblasNoTrans, bt = tb != CblasNoTrans;
    for (int i = 0; i < m; ++i) {
        T* ci = c + static_cast<long>(i) * ldc;
        if (beta == T(0)) for (int j = 0; j < n; ++j) ci[j] = T(0);
        else if (beta != T(1)) for (int j = 0; j < n; ++j) ci[j] *= beta;
        if (!bt) {
            for (int p = 0; p < k; ++p) {
                const T av = alpha * (at ? a[static_cast<long>(p) * lda + i] : a[static_cast<long>(i) * lda + p]);
                const T* bp = b + static_cast<long>(p) * ldb;
                for (int j = 0; j < n; ++j) ci[j] += av * bp[j];
            }
        } else {
            for (int j = 0; j < n; ++j) {
                const T* bj = b + static_cast<long>(j) * ldb;
                T s = T(0);
                if (!at) { const T* ai = a + static_cast<long>(i) * lda; for (int p = 0; p < k; ++p) s += ai[p] * bj[p]; }
                else for (int p = 0; p < k; ++p) s += a[static_cast<long>(p) * lda + i] * bj[p];
                ci[j] += alpha * s;
            }
        }
    }
}

template <typename T>
void gemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int m, int n, T alpha, const T* a, int lda,
          const T* x, int incx, T beta, T* y, int incy)
{
    bool trans = ta != CblasNoTrans;
    if (order == CblasColMajor) { trans = !trans; int t = m; m = n; n = t; }
    // now a is row-major m x n (after the swap for column-major input)
    const int ylen = trans ? n : m;
    for (int i = 0; i < ylen; ++i) {
        if (beta == T(0)) y[static_cast<long>(i) * incy] = T(0);
        else y[static_cast<long>(i) * incy] *= beta;
    }
    if (!trans) {
        for (int i = 0; i < m; ++i) {
            T s = T(0);
            const T* ai = a + static_cast<long>(i) * lda;
            for (int j = 0; j < n; ++j) s += ai[j] * x[static_cast<long>(j) * incx];
            y[static_cast<long>(i) * incy] += alpha * s;
        }
    } else {
        for (int i = 0; i < m; ++i) {
            const T xv = alpha * x[static_cast<long>(i) * incx];
            const T* ai = a + static_cast<long>(i) * lda;
            for (int j = 0; j < n; ++j) y[static_cast<long>(j) * incy] += xv * ai[j];
        }
    }
}
}  // namespace

extern "C" {
void cblas_sgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                 const float* a, int lda, const float* b, int ldb, float beta, float* c, int ldc)
{ gemm<float>(o, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); }
void cblas_dgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, double alpha,
                 const double* a, int lda, const double* b, int ldb, double beta, double* c, int ldc)
{ gemm<double>(o, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); }
void cblas_sgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, int m, int n, float alpha, const float* a, int lda,
                 const float* x, int incx, float beta, float* y, int incy)
{ gemv<float>(o, ta, m, n, alpha, a, lda, x, incx, beta, y, incy); }
void cblas_dgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, int m, int n, double alpha, const double* a, int lda,
                 const double* x, int incx, double beta, double* y, int incy)
{ gemv<double>(o, ta, m, n, alpha, a, lda, x, incx, beta, y, incy); }
float cblas_sdot(int n, const float* x, int incx, const float* y, int incy)
{ float s = 0; for (int i = 0; i < n; ++i) s += x[static_cast<long>(i) * incx] * y[static_cast<long>(i) * incy]; return s; }
double cblas_ddot(int n, const double* x, int incx, const double* y, int incy)
{ double s = 0; for (int i = 0; i < n; ++i) s += x[static_cast<long>(i) * incx] * y[static_cast<long>(i) * incy]; return s; }
void cblas_scopy(int n, const float* x, int incx, float* y, int incy)
{ for (int i = 0; i < n; ++i) y[static_cast<long>(i) * incy] = x[static_cast<long>(i) * incx]; }
void cblas_dcopy(int n, const double* x, int incx, double* y, int incy)
{ for (int i = 0; i < n; ++i) y[static_cast<long>(i) * incy] = x[static_cast<long>(i) * incx]; }
}
