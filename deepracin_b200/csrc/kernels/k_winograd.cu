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
    static __device__ __forceinline__ T fma(T a, float s, T b) { return fmaf(a, s, b); }      /* a * s + b */
    static __device__ __forceinline__ T max(T a, T b) { return fmaxf(a, b); }
    static __device__ __forceinline__ T hi(T a) { return __uint_as_float(__float_as_uint(a) & 0xffffe000u); }     /* the 19 bits a TF32 operand keeps */
    static __device__ __forceinline__ T bias_act(T v, const float *bias, int o, int act) { return drk_act(v + (bias ? bias[o] : 0.0f), act); }
};
template <> struct WVec<2> {
    typedef float2 T;
    static __device__ __forceinline__ T zero() { return make_float2(0.f, 0.f); }
    static __device__ __forceinline__ T add(T a, T b) { return make_float2(a.x + b.x, a.y + b.y); }
    static __device__ __forceinline__ T sub(T a, T b) { return make_float2(a.x - b.x, a.y - b.y); }
    static __device__ __forceinline__ T fma(T a, float s, T b) { return make_float2(fmaf(a.x, s, b.x), fmaf(a.y, s, b.y)); }
    static __device__ __forceinline__ T max(T a, T b) { return make_float2(fmaxf(a.x, b.x), fmaxf(a.y, b.y)); }
    static __device__ __forceinline__ T hi(T a) { return make_float2(WVec<1>::hi(a.x), WVec<1>::hi(a.y)); }
    static __device__ __forceinline__ T bias_act(T v, const float *bias, int o, int act)
    {
        float2 b = bias ? *reinterpret_cast<const float2 *>(bias + o) : make_float2(0.f, 0.f);
        return make_float2(drk_act(v.x + b.x, act), drk_act(v.y + b.y, act));
    }
};
template <> struct WVec<4> {
    typedef float4 T;
    static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ T add(T a, T b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
    static __device__ __forceinline__ T sub(T a, T b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
    static __device__ __forceinline__ T fma(T a, float s, T b) { return make_float4(fmaf(a.x, s, b.x), fmaf(a.y, s, b.y), fmaf(a.z, s, b.z), fmaf(a.w, s, b.w)); }
    static __device__ __forceinline__ T max(T a, T b) { return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w)); }
    static __device__ __forceinline__ T hi(T a) { return make_float4(WVec<1>::hi(a.x), WVec<1>::hi(a.y), WVec<1>::hi(a.z), WVec<1>::hi(a.w)); }
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
    const size_t chunks = ((size_t)n + c - 1) / c;          /* equal chunks rather than full ones and a short last one */
    c = ((size_t)n + chunks - 1) / chunks;
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


/* ------------------------------------------------------------------------------------------------------------------
 * Winograd F(4x4,3x3), FP32: the same three steps on 6x6 input tiles that produce 4x4 outputs, with the published
 * minimal-filtering matrices for the interpolation points 0, +-1, +-2, infinity (Lavin & Gray, "Fast Algorithms for
 * Convolutional Neural Networks", 2015):
 *   B^T = [4 0 -5 0 1 0; 0 -4 -4 1 1 0; 0 4 -4 -1 1 0; 0 -2 -1 2 1 0; 0 2 -1 -2 1 0; 0 4 0 -5 0 1]
 *   G   = [1/4 0 0; -1/6 -1/6 -1/6; -1/6 1/6 -1/6; 1/24 1/12 1/6; 1/24 -1/12 1/6; 0 0 1]
 *   A^T = [1 1 1 1 1 0; 0 1 -1 2 -2 0; 0 1 1 4 4 0; 0 1 -1 8 -8 1]
 * 36 products per 16 outputs: 4x fewer multiplications than the direct form (F(2x2,3x3): 2.25x) and 2.25 transform-domain
 * values per output pixel and channel instead of 4, so both the GEMM and the V / M traffic shrink.  The larger
 * coefficients cost accuracy: measured error against a float64 convolution is 0.4 - 1.5e-5 of max|ref| for 64 - 512 input
 * channels (F(2x2,3x3): below 1e-6), inside the FP32 class bound of 1e-4.
 * ------------------------------------------------------------------------------------------------------------------ */
#define WINO4_SCRATCH_CAP ((size_t)1 << 28)     /* floats */

/* one column / row of B^T (.) : six values in, six out, in place */
template <class X, class vt>
static __device__ __forceinline__ void wino4_bt(vt &d0, vt &d1, vt &d2, vt &d3, vt &d4, vt &d5)
{
    const vt e42 = X::fma(d2, -4.0f, d4);           /* d4 - 4 d2 */
    const vt e31 = X::fma(d1, -4.0f, d3);           /* d3 - 4 d1 */
    const vt f42 = X::sub(d4, d2);
    const vt f31 = X::sub(d3, d1);
    const vt t0 = X::fma(d2, -5.0f, X::fma(d0, 4.0f, d4));
    const vt t5 = X::fma(d3, -5.0f, X::fma(d1, 4.0f, d5));
    d0 = t0;
    d1 = X::add(e42, e31);
    d2 = X::sub(e42, e31);
    d3 = X::fma(f31, 2.0f, f42);
    d4 = X::fma(f31, -2.0f, f42);
    d5 = t5;
}

/* V[k][t][c], k = 0..35.  SPLIT: rows are 2C wide, the value's TF32 high part (upper 19 bits) at [c] and the remainder at [C + c]:
   the operand layout of the FP32-accurate three-pass tensor-core product */
template <int VEC, bool SPLIT>
__global__ void __launch_bounds__(256) k_wino4_input(const float *__restrict__ in, float *__restrict__ V, int W, int H, int C, int ldi,
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
        const int x0 = tix * 4 - 1, y0 = tiy * 4 - 1;
        vt d[6][6];
#pragma unroll
        for (int r = 0; r < 6; r++) {
            const int y = y0 + r;
#pragma unroll
            for (int s = 0; s < 6; s++) {
                const int x = x0 + s;
                d[r][s] = (x >= 0 && x < W && y >= 0 && y < H) ? *reinterpret_cast<const vt *>(in + (((size_t)b * H + y) * W + x) * ldi + c) : X::zero();
            }
        }
#pragma unroll
        for (int s = 0; s < 6; s++) wino4_bt<X, vt>(d[0][s], d[1][s], d[2][s], d[3][s], d[4][s], d[5][s]);      /* B^T d */
#pragma unroll
        for (int r = 0; r < 6; r++) {                                                                           /* (.) B */
            wino4_bt<X, vt>(d[r][0], d[r][1], d[r][2], d[r][3], d[r][4], d[r][5]);
#pragma unroll
            for (int s = 0; s < 6; s++) {
                if (SPLIT) {
                    float *row = V + ((size_t)(r * 6 + s) * Ts + t) * (2 * (size_t)C) + c;
                    const vt h = X::hi(d[r][s]);
                    *reinterpret_cast<vt *>(row) = h;
                    *reinterpret_cast<vt *>(row + C) = X::sub(d[r][s], h);
                } else {
                    *reinterpret_cast<vt *>(V + ((size_t)(r * 6 + s) * Ts + t) * C + c) = d[r][s];
                }
            }
        }
    }
}

/* POOL: the 4x4 outputs of a tile are reduced to their 2x2 block maxima after bias and activation, and stored into the
   pooled tensor [H/2][W/2] (the 2x2/2 max pooling that follows the layer, evaluated here; W and H even) */
template <int VEC, bool POOL>
__global__ void __launch_bounds__(256) k_wino4_output(const float *__restrict__ Mt, const float *__restrict__ bias, float *__restrict__ out,
                                                      int W, int H, int O, int ldo, int coff, int tx, int ty, size_t T, size_t Ts, int act)
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
        vt s[6][4];                                                         /* M A : six rows of four */
#pragma unroll
        for (int r = 0; r < 6; r++) {
            vt m[6];
#pragma unroll
            for (int k = 0; k < 6; k++) m[k] = *reinterpret_cast<const vt *>(Mt + ((size_t)(r * 6 + k) * Ts + t) * O + o);
            const vt p12 = X::add(m[1], m[2]), q12 = X::sub(m[1], m[2]);
            const vt p34 = X::add(m[3], m[4]), q34 = X::sub(m[3], m[4]);
            s[r][0] = X::add(X::add(m[0], p12), p34);
            s[r][1] = X::fma(q34, 2.0f, q12);
            s[r][2] = X::fma(p34, 4.0f, p12);
            s[r][3] = X::add(X::fma(q34, 8.0f, q12), m[5]);
        }
        vt y[4][4];                                                         /* A^T (.) : y[row][column], bias and activation applied */
#pragma unroll
        for (int cx = 0; cx < 4; cx++) {
            const vt p12 = X::add(s[1][cx], s[2][cx]), q12 = X::sub(s[1][cx], s[2][cx]);
            const vt p34 = X::add(s[3][cx], s[4][cx]), q34 = X::sub(s[3][cx], s[4][cx]);
            y[0][cx] = X::bias_act(X::add(X::add(s[0][cx], p12), p34), bias, o, act);
            y[1][cx] = X::bias_act(X::fma(q34, 2.0f, q12), bias, o, act);
            y[2][cx] = X::bias_act(X::fma(p34, 4.0f, p12), bias, o, act);
            y[3][cx] = X::bias_act(X::add(X::fma(q34, 8.0f, q12), s[5][cx]), bias, o, act);
        }
        if (POOL) {
            const int Wp = W >> 1, Hp = H >> 1, px = tix * 2, py = tiy * 2;
            float *dst = out + (((size_t)b * Hp + py) * Wp + px) * ldo + coff + o;
#pragma unroll
            for (int cy = 0; cy < 2; cy++)
#pragma unroll
                for (int cx = 0; cx < 2; cx++)
                    if (px + cx < Wp && py + cy < Hp)
                        *reinterpret_cast<vt *>(dst + ((size_t)cy * Wp + cx) * ldo) =
                            X::max(X::max(y[2 * cy][2 * cx], y[2 * cy][2 * cx + 1]), X::max(y[2 * cy + 1][2 * cx], y[2 * cy + 1][2 * cx + 1]));
        } else {
            const int ox = tix * 4, oy = tiy * 4;
            float *dst = out + (((size_t)b * H + oy) * W + ox) * ldo + coff + o;
#pragma unroll
            for (int cy = 0; cy < 4; cy++)
#pragma unroll
                for (int cx = 0; cx < 4; cx++)
                    if (ox + cx < W && oy + cy < H) *reinterpret_cast<vt *>(dst + ((size_t)cy * W + cx) * ldo) = y[cy][cx];
        }
    }
}

static size_t wino4_tiles_per_image(int W, int H) { return (size_t)((W + 3) / 4) * ((H + 3) / 4); }

static int wino4_chunk(int n, int W, int H, int Cin, int Cout)
{
    const size_t per = 36 * wino4_tiles_per_image(W, H) * (size_t)(Cin + Cout);
    size_t c = WINO4_SCRATCH_CAP / per;
    if (c < 1) c = 1;
    if (c > (size_t)n) c = (size_t)n;
    const size_t chunks = ((size_t)n + c - 1) / c;          /* equal chunks rather than full ones and a short last one */
    c = ((size_t)n + chunks - 1) / chunks;
    return (int)c;
}

extern "C" size_t dRk_winograd4_scratch_floats(int n, int W, int H, int Cin, int Cout)
{
    if (n <= 0 || W <= 0 || H <= 0 || Cin <= 0 || Cout <= 0) return 0;
    return 36 * wino4_tiles_per_image(W, H) * (size_t)(Cin + Cout) * wino4_chunk(n, W, H, Cin, Cout);
}

/* U = G g G^T in double, stored [36][Cin][Cout] (each transform position one K x N matrix); w is the reference's [Cin][Cout][3][3] */
extern "C" int dRk_winograd4_pack_weights(const float *w, float *U, int Cin, int Cout)
{
    if (!w || !U || Cin <= 0 || Cout <= 0) return -1;
    static const double G[6][3] = {{1.0 / 4, 0, 0}, {-1.0 / 6, -1.0 / 6, -1.0 / 6}, {-1.0 / 6, 1.0 / 6, -1.0 / 6},
                                   {1.0 / 24, 1.0 / 12, 1.0 / 6}, {1.0 / 24, -1.0 / 12, 1.0 / 6}, {0, 0, 1}};
    for (int i = 0; i < Cin; i++)
        for (int o = 0; o < Cout; o++) {
            const float *g = w + ((size_t)i * Cout + o) * 9;
            double tmp[6][3];
            for (int r = 0; r < 6; r++)
                for (int s = 0; s < 3; s++) tmp[r][s] = G[r][0] * g[0 * 3 + s] + G[r][1] * g[1 * 3 + s] + G[r][2] * g[2 * 3 + s];
            for (int r = 0; r < 6; r++)
                for (int s = 0; s < 6; s++)
                    U[((size_t)(r * 6 + s) * Cin + i) * Cout + o] = (float)(tmp[r][0] * G[s][0] + tmp[r][1] * G[s][1] + tmp[r][2] * G[s][2]);
        }
    return 0;
}

template <int VEC>
static void wino4_launch_in(cudaStream_t st, const float *in, float *V, int W, int H, int C, int ldi, int tx, int ty, size_t T, size_t Ts, int split)
{
    const unsigned blocks = drk_blocks(T * (C / VEC), 256, 148u * 32u);
    if (split) k_wino4_input<VEC, true><<<blocks, 256, 0, st>>>(in, V, W, H, C, ldi, tx, ty, T, Ts);
    else k_wino4_input<VEC, false><<<blocks, 256, 0, st>>>(in, V, W, H, C, ldi, tx, ty, T, Ts);
}

template <int VEC>
static void wino4_launch_out(cudaStream_t st, const float *Mt, const float *bias, float *out, int W, int H, int O, int ldo, int coff,
                             int tx, int ty, size_t T, size_t Ts, int act, int pool)
{
    const unsigned blocks = drk_blocks(T * (O / VEC), 256, 148u * 32u);
    if (pool) k_wino4_output<VEC, true><<<blocks, 256, 0, st>>>(Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act);
    else k_wino4_output<VEC, false><<<blocks, 256, 0, st>>>(Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act);
}

/* F(4x4,3x3) transform launches shared with the tensor-core path (k_umma_conv.cu): Ts = row stride between the 36 transform
 * positions (Ts >= T), split = (high | low) operand rows for the three-pass product, pool = fused 2x2/2 max pooling */
int drk_wino4_input_launch(cudaStream_t st, const float *in, float *V, int W, int H, int C, int ldi, size_t T, size_t Ts, int split)
{
    const int tx = (W + 3) / 4, ty = (H + 3) / 4;
    if (C % 2 == 0 && ldi % 2 == 0 && ((uintptr_t)in % 8) == 0 && ((uintptr_t)V % 16) == 0) wino4_launch_in<2>(st, in, V, W, H, C, ldi, tx, ty, T, Ts, split);
    else wino4_launch_in<1>(st, in, V, W, H, C, ldi, tx, ty, T, Ts, split);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

int drk_wino4_output_launch(cudaStream_t st, const float *Mt, const float *bias, float *out, int W, int H, int O, int ldo, int coff,
                            size_t T, size_t Ts, int act, int pool)
{
    const int tx = (W + 3) / 4, ty = (H + 3) / 4;
    if (O % 2 == 0 && ldo % 2 == 0 && coff % 2 == 0 && ((uintptr_t)out % 8) == 0 && ((uintptr_t)Mt % 16) == 0 && (!bias || ((uintptr_t)bias % 8) == 0))
        wino4_launch_out<2>(st, Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act, pool);
    else wino4_launch_out<1>(st, Mt, bias, out, W, H, O, ldo, coff, tx, ty, T, Ts, act, pool);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

extern "C" int dRk_conv2d_winograd4_f32(dRk_stream stream, const float *in, const float *U, const float *bias, float *out,
                                        float *scratch, int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff, int pool)
{
    if (n <= 0 || W <= 0 || H <= 0 || Cin <= 0 || Cout <= 0 || !scratch) return -1;
    if (ldi < Cin || ldo < coff + Cout) return -3;
    if (pool && (pool != 1 || (W & 1) || (H & 1))) return -5;      /* only the 2x2/2 max pooling of an even plane is evaluated here */
    cudaStream_t st = drk_stream(stream);
    const int tx = (W + 3) / 4, ty = (H + 3) / 4;
    const int chunk = wino4_chunk(n, W, H, Cin, Cout);
    for (int b0 = 0; b0 < n; b0 += chunk) {
        const int nb = n - b0 < chunk ? n - b0 : chunk;
        const size_t T = (size_t)nb * tx * ty;
        if (T > 0x7fffffffull) return -2;
        float *V = scratch, *Mt = scratch + 36 * T * Cin;
        const float *src = in + (size_t)b0 * H * W * ldi;
        float *dst = out + (size_t)b0 * (pool ? (H / 2) * (W / 2) : H * W) * ldo;
        int rc = drk_wino4_input_launch(st, src, V, W, H, Cin, ldi, T, T, 0);
        if (rc) return rc;
        rc = drk_gemm_f32_launch(st, V, U, NULL, Mt, (int)T, Cout, Cin, Cin, Cout, Cout, 0, 0, 36,
                                 T * Cin, (size_t)Cin * Cout, T * Cout, NULL);
        if (rc) return rc;
        rc = drk_wino4_output_launch(st, Mt, bias, dst, W, H, Cout, ldo, coff, T, T, act, pool);
        if (rc) return rc;
    }
    return 0;
}
