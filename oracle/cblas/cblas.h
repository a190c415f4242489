/*
 * TEST INFRASTRUCTURE — minimal CBLAS declarations for building the reference CPU tile.
 *
 * The reference calls an external CBLAS (OpenBLAS or MKL; cmake/dependencies.cmake:49-79) for
 * level-1/2/3 routines (src/rpucuda/math_util.cpp:16-296).  No cblas.h is installed in this
 * image, so this header declares exactly the routines the reference uses, with the standard
 * CBLAS signatures.  They resolve either to a system OpenBLAS or to cblas_fallback.c.
 */
#ifndef ORACLE_CBLAS_H_
#define ORACLE_CBLAS_H_
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef CBLAS_ORDER CBLAS_LAYOUT;

void cblas_sgemm(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int M, int N, int K, float alpha,
                 const float *A, int lda, const float *B, int ldb, float beta, float *C, int ldc);
void cblas_dgemm(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int M, int N, int K, double alpha,
                 const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc);
void cblas_sgemv(CBLAS_ORDER, CBLAS_TRANSPOSE, int M, int N, float alpha, const float *A, int lda,
                 const float *X, int incX, float beta, float *Y, int incY);
void cblas_dgemv(CBLAS_ORDER, CBLAS_TRANSPOSE, int M, int N, double alpha, const double *A, int lda,
                 const double *X, int incX, double beta, double *Y, int incY);
void cblas_sger(CBLAS_ORDER, int M, int N, float alpha, const float *X, int incX, const float *Y,
                int incY, float *A, int lda);
void cblas_dger(CBLAS_ORDER, int M, int N, double alpha, const double *X, int incX, const double *Y,
                int incY, double *A, int lda);
size_t cblas_isamax(int N, const float *X, int incX);
size_t cblas_idamax(int N, const double *X, int incX);
void cblas_scopy(int N, const float *X, int incX, float *Y, int incY);
void cblas_dcopy(int N, const double *X, int incX, double *Y, int incY);
void cblas_sscal(int N, float alpha, float *X, int incX);
void cblas_dscal(int N, double alpha, double *X, int incX);
float cblas_snrm2(int N, const float *X, int incX);
double cblas_dnrm2(int N, const double *X, int incX);
#ifdef __cplusplus
}
#endif
#endif
