/*
 * TEST INFRASTRUCTURE — straightforward CBLAS subset used only when no OpenBLAS is found
 * when building the reference CPU tile (see oracle/Makefile).  Own code; textbook loops.
 */
#include "cblas.h"
#include <math.h>

#define AT(A, ld, order, i, j) ((order) == CblasRowMajor ? (A)[(size_t)(i) * (ld) + (j)] : (A)[(size_t)(j) * (ld) + (i)])

#define DEFINE_BLAS(T, p, ip)                                                                      \
  void cblas_##p##gemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, \
                       T alpha, const T *A, int lda, const T *B, int ldb, T beta, T *C, int ldc) { \
    for (int i = 0; i < M; i++) {                                                                  \
      for (int j = 0; j < N; j++) {                                                                \
        T acc = 0;                                                                                 \
        for (int k = 0; k < K; k++) {                                                              \
          T a = ta == CblasNoTrans ? AT(A, lda, o, i, k) : AT(A, lda, o, k, i);                    \
          T b = tb == CblasNoTrans ? AT(B, ldb, o, k, j) : AT(B, ldb, o, j, k);                    \
          acc += a * b;                                                                            \
        }                                                                                          \
        T *c = o == CblasRowMajor ? &C[(size_t)i * ldc + j] : &C[(size_t)j * ldc + i];             \
        *c = alpha * acc + (beta == 0 ? 0 : beta * *c);                                            \
      }                                                                                            \
    }                                                                                              \
  }                                                                                                \
  void cblas_##p##gemv(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, int M, int N, T alpha, const T *A,       \
                       int lda, const T *X, int incX, T beta, T *Y, int incY) {                    \
    int rows = ta == CblasNoTrans ? M : N, cols = ta == CblasNoTrans ? N : M;                      \
    for (int i = 0; i < rows; i++) {                                                               \
      T acc = 0;                                                                                   \
      for (int j = 0; j < cols; j++) {                                                             \
        T a = ta == CblasNoTrans ? AT(A, lda, o, i, j) : AT(A, lda, o, j, i);                      \
        acc += a * X[(size_t)j * incX];                                                            \
      }                                                                                            \
      T *y = &Y[(size_t)i * incY];                                                                 \
      *y = alpha * acc + (beta == 0 ? 0 : beta * *y);                                              \
    }                                                                                              \
  }                                                                                                \
  void cblas_##p##ger(CBLAS_ORDER o, int M, int N, T alpha, const T *X, int incX, const T *Y,      \
                      int incY, T *A, int lda) {                                                   \
    for (int i = 0; i < M; i++) {                                                                  \
      for (int j = 0; j < N; j++) {                                                                \
        T *a = o == CblasRowMajor ? &A[(size_t)i * lda + j] : &A[(size_t)j * lda + i];             \
        *a += alpha * X[(size_t)i * incX] * Y[(size_t)j * incY];                                   \
      }                                                                                            \
    }                                                                                              \
  }                                                                                                \
  size_t cblas_i##p##amax(int N, const T *X, int incX) {                                           \
    size_t best = 0;                                                                               \
    T bv = -1;                                                                                     \
    for (int i = 0; i < N; i++) {                                                                  \
      T v = (T)fabs((double)X[(size_t)i * incX]);                                                  \
      if (v > bv) {                                                                                \
        bv = v;                                                                                    \
        best = (size_t)i;                                                                          \
      }                                                                                            \
    }                                                                                              \
    return best;                                                                                   \
  }                                                                                                \
  void cblas_##p##copy(int N, const T *X, int incX, T *Y, int incY) {                              \
    for (int i = 0; i < N; i++)                                                                    \
      Y[(size_t)i * incY] = X[(size_t)i * incX];                                                   \
  }                                                                                                \
  void cblas_##p##scal(int N, T alpha, T *X, int incX) {                                           \
    for (int i = 0; i < N; i++)                                                                    \
      X[(size_t)i * incX] *= alpha;                                                                \
  }                                                                                                \
  T cblas_##p##nrm2(int N, const T *X, int incX) {                                                 \
    double acc = 0;                                                                                \
    for (int i = 0; i < N; i++) {                                                                  \
      double v = (double)X[(size_t)i * incX];                                                      \
      acc += v * v;                                                                                \
    }                                                                                              \
    return (T)sqrt(acc);                                                                           \
  }

DEFINE_BLAS(float, s, s)
DEFINE_BLAS(double, d, d)
