/* Internal interface of the FP32 GEMM core (k_gemm_f32.cu). */
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

/* geometry of an implicit-GEMM convolution: A row m = (image, oy, ox), column k = (ky, kx, c) */
struct drk_ConvGeom {
    int W, H, Cin, kw, kh, sx, sy, Wo, Ho, px, py, ldi;
};

/*
 * C[z][m*ldc + coff + n] = act(bias[n] + sum_k A[z](m,k) * B[z][k*ldb + n]),  z < batch.
 * geom == NULL: A is dense row-major with leading dimension lda; otherwise A is gathered
 * from an N-HWC tensor.  sA/sB/sC are the per-z strides in floats.
 */
int drk_gemm_f32_launch(cudaStream_t st, const float *A, const float *B, const float *bias, float *C, int M, int N, int K,
                        int lda, int ldb, int ldc, int coff, int act, int batch, size_t sA, size_t sB, size_t sC,
                        const drk_ConvGeom *geom);

/* 3x3 stride-1 convolution specialised for Cin <= 4 (k_conv_first.cu); returns 0 when it does not take the shape */
int drk_conv3x3_smallcin_launch(cudaStream_t st, const float *in, const float *wpack, const float *bias, float *out, int n, int W, int H,
                                int Cin, int Cout, int act, int ldi, int ldo, int coff, int *rc);

/* Winograd F(2x2,3x3) transforms (k_winograd.cu): V[k][t][c] with Ts tiles between transform positions, and back. */
int drk_wino_input_launch(cudaStream_t st, const float *in, float *V, int nimg, int W, int H, int C, int ldi, size_t T, size_t Ts);
int drk_wino_output_launch(cudaStream_t st, const float *Mt, const float *bias, float *out, int W, int H, int O, int ldo, int coff,
                           size_t T, size_t Ts, int act);

/* Winograd F(4x4,3x3) transforms (k_winograd.cu): V[k][t][c], k = 0..35; split = rows of 2C floats, TF32 high parts then remainders */
int drk_wino4_input_launch(cudaStream_t st, const float *in, float *V, int W, int H, int C, int ldi, size_t T, size_t Ts, int split);
int drk_wino4_output_launch(cudaStream_t st, const float *Mt, const float *bias, float *out, int W, int H, int O, int ldo, int coff,
                            size_t T, size_t Ts, int act, int pool);
