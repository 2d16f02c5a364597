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

/* float or float4 of consecutive channels per thread */
template <int VEC> struct WVec;
template <> struct WVec<1> {
    typedef float T;
    static __device__ __forceinline__ T zero() { return 0.0f; }
    static __device__ __forceinline__ T add(T a, T b) { return a + b; }
    static __device__ __forceinline__ T sub(T a, T b) { return a - b; }
    static __device__ __forceinline__ T bias_act(T v, const float *bias, int o, int act) { return drk_act(v + (bias ? bias[o] : 0.0f), act); }
};
template <> struct WVec<4> {
    typedef float4 T;
    static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ T add(T a, T b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
    static __device__ __forceinline__ T sub(T a, T b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
    static __device__ __forceinline__ T bias_act(T v, const float *bias, int o, int act)
    {
        float4 b = bias ? *reinterpret_cast<const float4 *>(bias + o) : make_float4(0.f, 0.f, 0.f, 0.f);
        return make_float4(drk_act(v.x + b.x, act), drk_act(v.y + b.y, act), drk_act(v.z + b.z, act), drk_act(v.w + b.w, act));
    }
};

/* V[k][t][c], k = 0..15, rows of one k are Ts tiles apart (Ts >= T: the tensor-core path pads the tile count to whole GEMM tiles) */
template <int VEC>
__global__ void k_wino_input(const float *__restrict__ in, float *__restrict__ V, int nimg, int W, int H, int C, int ldi,
                             int tx, int ty, size_t T, size_t Ts)
{
    typedef WVec<VEC> X;
    typedef typename X::T vt;
    const int CV = C / VEC;
    const size_t total = T * CV;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % CV) * VEC;
        const size_t t = i / CV;
        const int tix = (int)(t % tx);
        const size_t q = t / tx;
        const int tiy = (int)(q % ty);
        const int b = (int)(q / ty);
        const int x0 = tix * 2 - 1, y0 = tiy * 2 - 1;
        vt d[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int y = y0 + r;
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const int x = x0 + s;
                d[r][s] = (x >= 0 && x < W && y >= 0 && y < H) ? *reinterpret_cast<const vt *>(in + (((size_t)b * H + y) * W + x) * ldi + c) : X::zero();
            }
        }
        vt m[4][4];
#pragma unroll
        for (int s = 0; s < 4; s++) {       /* B^T d : rows */
            m[0][s] = X::sub(d[0][s], d[2][s]);
            m[1][s] = X::add(d[1][s], d[2][s]);
            m[2][s] = X::sub(d[2][s], d[1][s]);
            m[3][s] = X::sub(d[3][s], d[1][s]);
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {       /* (.) B : columns */
            const vt a0 = m[r][0], a1 = m[r][1], a2 = m[r][2], a3 = m[r][3];
            *reinterpret_cast<vt *>(V + ((size_t)(r * 4 + 0) * Ts + t) * C + c) = X::sub(a0, a2);
            *reinterpret_cast<vt *>(V + ((size_t)(r * 4 + 1) * Ts + t) * C + c) = X::add(a1, a2);
            *reinterpret_cast<vt *>(V + ((size_t)(r * 4 + 2) * Ts + t) * C + c) = X::sub(a2, a1);
            *reinterpret_cast<vt *>(V + ((size_t)(r * 4 + 3) * Ts + t) * C + c) = X::sub(a3, a1);
        }
    }
}

template <int VEC>
__global__ void k_wino_output(const float *__restrict__ Mt, const float *__restrict__ bias, float *__restrict__ out, int W, int H, int O,
                              int ldo, int coff, int tx, int ty, size_t T, size_t Ts, int act)
{
    typedef WVec<VEC> X;
    typedef typename X::T vt;
    const int OV = O / VEC;
    const size_t total = T * OV;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(i % OV) * VEC;
        const size_t t = i / OV;
        const int tix = (int)(t % tx);
        const size_t q = t / tx;
        const int tiy = (int)(q % ty);
        const int b = (int)(q / ty);
        vt m[16];
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = *reinterpret_cast<const vt *>(Mt + ((size_t)k * Ts + t) * O + o);
        vt s[8];
#pragma unroll
        for (int r = 0; r < 4; r++) {       /* (.) A */
            s[r * 2 + 0] = X::add(X::add(m[r * 4 + 0], m[r * 4 + 1]), m[r * 4 + 2]);
            s[r * 2 + 1] = X::add(X::sub(m[r * 4 + 1], m[r * 4 + 2]), m[r * 4 + 3]);
        }
        const vt y00 = X::add(X::add(s[0], s[2]), s[4]), y01 = X::add(X::add(s[1], s[3]), s[5]);      /* A^T (.) */
        const vt y10 = X::add(X::sub(s[2], s[4]), s[6]), y11 = X::add(X::sub(s[3], s[5]), s[7]);
        const int ox = tix * 2, oy = tiy * 2;
        float *dst = out + (((size_t)b * H + oy) * W + ox) * ldo + coff + o;
        *reinterpret_cast<vt *>(dst) = X::bias_act(y00, bias, o, act);
        if (ox + 1 < W) *reinterpret_cast<vt *>(dst + ldo) = X::bias_act(y01, bias, o, act);
        if (oy + 1 < H) {
            *reinterpret_cast<vt *>(dst + (size_t)W * ldo) = X::bias_act(y10, bias, o, act);
            if (ox + 1 < W) *reinterpret_cast<vt *>(dst + (size_t)W * ldo + ldo) = X::bias_act(y11, bias, o, act);
        }
    }
}

static bool wino_aligned16(const void *p) { return ((uintptr_t)p % 16) == 0; }

/* Input / output transform launches shared by the FP32 path below and the tensor-core path (k_umma_conv.cu); Ts is the row
 * stride between the 16 transform positions (Ts >= T). */
int drk_wino_input_launch(cudaStream_t st, const float *in, float *V, int nimg, int W, int H, int C, int ldi, size_t T, size_t Ts)
{
    const int tx = (W + 1) / 2, ty = (H + 1) / 2;
    if (C % 4 == 0 && ldi % 4 == 0 && wino_aligned16(in) && wino_aligned16(V))
        k_wino_input<4><<<drk_blocks(T * (C / 4), 256, 148u * 32u), 256, 0, st>>>(in, V, nimg, W, H, C, ldi, tx, ty, T, Ts);
    else
        k_wino_input<1><<<drk_blocks(T * C, 256, 148u * 32u), 256, 0, st>>>(in, V, nimg, W, H, C, ldi, tx, ty, T, Ts);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

int drk_wino_output_launch(cudaStream_t st, const float *Mt, const float *bias, float *out, int W, int H, int O, int ldo, int coff,
                           size_t T, size_t Ts, int act)
{
    const int tx = (W + 1) / 2, ty = (H + 1) / 2;
    if (O % 4 == 0 && ldo % 4 == 0 && coff % 4 == 0 && wino_aligned16(out) && wino_aligned16(Mt) && (!bias || wino_aligned16(bias)))
        k_wino_output<4><<<drk_blocks(T * (O / 4), 256, 148u * 32u), 256, 0, st>>>(Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act);
    else
        k_wino_output<1><<<drk_blocks(T * O, 256, 148u * 32u), 256, 0, st>>>(Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
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
        int rc = drk_wino_input_launch(st, src, V, nb, W, H, Cin, ldi, T, T);
        if (rc) return rc;
        rc = drk_gemm_f32_launch(st, V, U, NULL, Mt, (int)T, Cout, Cin, Cin, Cout, Cout, 0, 0, 16,
                                 T * Cin, (size_t)Cin * Cout, T * Cout, NULL);
        if (rc) return rc;
        rc = drk_wino_output_launch(st, Mt, bias, dst, W, H, Cout, ldo, coff, T, T, act);
        if (rc) return rc;
    }
    return 0;
}
