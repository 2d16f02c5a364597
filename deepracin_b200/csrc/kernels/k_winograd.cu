/*
 * Winograd F(2x2,3x3) convolution, exact FP32, over N-HWC activations.
 *
 * Three launches per image chunk:
 *   1. input transform  V_k[t][c] = (B^T d B)_k for every 4x4 input tile t (origin = output
 *      (2tx,2ty) - 1, zero padded) and channel c;  HBM-bound: reads the input once (with a
 *      2x halo overlap from cache), writes 16 floats per (tile, channel);
 *   2. sixteen dense GEMMs  M_k[t][o] = sum_c V_k[t][c] * U_k[c][o]  on the FFMA GEMM core
 *      (1/2.25 of the direct multiplications);
 *   3. output transform  Y = A^T M A, bias, activation, guarded 2x2 store;  HBM-bound.
 * B^T, A^T and the filter transform G are the reference's own matrices
 * (Kernels/dR_winograd2.cl:55-251, src/dR_nodes_conv2d.c:1173-1176); its B^T has the last
 * row negated with respect to the textbook form and A^T compensates the sign.
 * The reference fuses all three steps in one work-group (re-transforming the input per
 * work-group); here V and M live in a scratch buffer between the launches.
 */
#include "k_common.cuh"
#include "k_gemm_f32.cuh"

#define WINO_SCRATCH_CAP ((size_t)1 << 28)   /* floats (1 GiB): larger layers are processed in image chunks */

__global__ void k_wino_input(const float *__restrict__ in, float *__restrict__ V, int nimg, int W, int H, int C, int ldi,
                             int tx, int ty, size_t T)
{
    const size_t total = T * C;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const size_t t = i / C;
        const int tix = (int)(t % tx);
        const size_t q = t / tx;
        const int tiy = (int)(q % ty);
        const int b = (int)(q / ty);
        const int x0 = tix * 2 - 1, y0 = tiy * 2 - 1;
        float d[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int y = y0 + r;
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const int x = x0 + s;
                d[r][s] = (x >= 0 && x < W && y >= 0 && y < H) ? in[(((size_t)b * H + y) * W + x) * ldi + c] : 0.0f;
            }
        }
        float m[4][4];
#pragma unroll
        for (int s = 0; s < 4; s++) {       /* B^T d : rows */
            m[0][s] = d[0][s] - d[2][s];
            m[1][s] = d[1][s] + d[2][s];
            m[2][s] = -d[1][s] + d[2][s];
            m[3][s] = -d[1][s] + d[3][s];
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {       /* (.) B : columns */
            const float a0 = m[r][0], a1 = m[r][1], a2 = m[r][2], a3 = m[r][3];
            V[((size_t)(r * 4 + 0) * T + t) * C + c] = a0 - a2;
            V[((size_t)(r * 4 + 1) * T + t) * C + c] = a1 + a2;
            V[((size_t)(r * 4 + 2) * T + t) * C + c] = -a1 + a2;
            V[((size_t)(r * 4 + 3) * T + t) * C + c] = -a1 + a3;
        }
    }
}

__global__ void k_wino_output(const float *__restrict__ Mt, const float *__restrict__ bias, float *__restrict__ out, int W, int H, int O,
                              int ldo, int coff, int tx, int ty, size_t T, int act)
{
    const size_t total = T * O;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(i % O);
        const size_t t = i / O;
        const int tix = (int)(t % tx);
        const size_t q = t / tx;
        const int tiy = (int)(q % ty);
        const int b = (int)(q / ty);
        float m[16];
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = Mt[((size_t)k * T + t) * O + o];
        float s[8];
#pragma unroll
        for (int r = 0; r < 4; r++) {       /* (.) A */
            s[r * 2 + 0] = m[r * 4 + 0] + m[r * 4 + 1] + m[r * 4 + 2];
            s[r * 2 + 1] = m[r * 4 + 1] - m[r * 4 + 2] + m[r * 4 + 3];
        }
        float y00 = s[0] + s[2] + s[4], y01 = s[1] + s[3] + s[5];      /* A^T (.) */
        float y10 = s[2] - s[4] + s[6], y11 = s[3] - s[5] + s[7];
        const float bv = bias ? bias[o] : 0.0f;
        const int ox = tix * 2, oy = tiy * 2;
        float *dst = out + (((size_t)b * H + oy) * W + ox) * ldo + coff + o;
        dst[0] = drk_act(y00 + bv, act);
        if (ox + 1 < W) dst[ldo] = drk_act(y01 + bv, act);
        if (oy + 1 < H) {
            dst[(size_t)W * ldo] = drk_act(y10 + bv, act);
            if (ox + 1 < W) dst[(size_t)W * ldo + ldo] = drk_act(y11 + bv, act);
        }
    }
}

static size_t wino_tiles_per_image(int W, int H) { return (size_t)((W + 1) / 2) * ((H + 1) / 2); }

/* images per chunk such that 16*T*(Cin+Cout) floats stay under the cap (at least one image) */
static int wino_chunk(int n, int W, int H, int Cin, int Cout)
{
    const size_t per = 16 * wino_tiles_per_image(W, H) * (size_t)(Cin + Cout);
    size_t c = WINO_SCRATCH_CAP / per;
    if (c < 1) c = 1;
    if (c > (size_t)n) c = (size_t)n;
    return (int)c;
}

extern "C" size_t dRk_winograd_scratch_floats(int n, int W, int H, int Cin, int Cout)
{
    if (n <= 0 || W <= 0 || H <= 0 || Cin <= 0 || Cout <= 0) return 0;
    return 16 * wino_tiles_per_image(W, H) * (size_t)(Cin + Cout) * wino_chunk(n, W, H, Cin, Cout);
}

extern "C" int dRk_conv2d_winograd_f32(dRk_stream stream, const float *in, const float *U, const float *bias, float *out,
                                       float *scratch, int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff)
{
    if (n <= 0 || W <= 0 || H <= 0 || Cin <= 0 || Cout <= 0 || !scratch) return -1;
    if (ldi < Cin || ldo < coff + Cout) return -3;
    cudaStream_t st = drk_stream(stream);
    const int tx = (W + 1) / 2, ty = (H + 1) / 2;
    const int chunk = wino_chunk(n, W, H, Cin, Cout);
    for (int b0 = 0; b0 < n; b0 += chunk) {
        const int nb = n - b0 < chunk ? n - b0 : chunk;
        const size_t T = (size_t)nb * tx * ty;
        if (T > 0x7fffffffull) return -2;
        float *V = scratch, *Mt = scratch + 16 * T * Cin;
        const float *src = in + (size_t)b0 * H * W * ldi;
        float *dst = out + (size_t)b0 * H * W * ldo;
        k_wino_input<<<drk_blocks(T * Cin, 256, 148u * 32u), 256, 0, st>>>(src, V, nb, W, H, Cin, ldi, tx, ty, T);
        DRK_COUNT_LAUNCH();
        int rc = DRK_LAUNCH_RESULT();
        if (rc) return rc;
        rc = drk_gemm_f32_launch(st, V, U, NULL, Mt, (int)T, Cout, Cin, Cin, Cout, Cout, 0, 0, 16,
                                 T * Cin, (size_t)Cin * Cout, T * Cout, NULL);
        if (rc) return rc;
        k_wino_output<<<drk_blocks(T * Cout, 256, 148u * 32u), 256, 0, st>>>(Mt, bias, dst, W, H, Cout, ldo, coff, tx, ty, T, act);
        DRK_COUNT_LAUNCH();
        rc = DRK_LAUNCH_RESULT();
        if (rc) return rc;
    }
    return 0;
}
