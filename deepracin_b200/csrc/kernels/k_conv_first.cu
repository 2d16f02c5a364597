/*
 * 3x3 stride-1 convolution for very few input channels (Cin <= 4, e.g. the RGB first layer
 * of VGG / SqueezeNet), exact FP32.  With K = 9*Cin <= 36 the layer is bound by writing its
 * output (AI ~ 13 flop/B), so neither an implicit GEMM tile nor Winograd pays: here a thread
 * keeps a 3 x 6 x Cin input patch in registers, computes 4 neighbouring pixels x 8 output
 * channels, reads the packed filters [9*Cin][Cout] from shared memory as float4 (one shared
 * load per 16 FMAs) and stores 32-byte runs; the Cout/8 threads of a pixel quad write one
 * contiguous pixel.  Replaces the reference's Winograd launch for such layers
 * (src/dR_nodes_conv2d.c:36-53 sends every 3x3 stride-1 filter to Winograd).
 * Bound: HBM; algorithmic bytes = n*H*W*(Cin + Cout)*4.
 */
#include "k_common.cuh"

#define QUADS_PER_BLOCK 64
#define CPT 8                       /* output channels per thread */

template <int CIN>
__global__ void __launch_bounds__(256, 2) k_conv3x3_smallcin(const float *__restrict__ in, const float *__restrict__ wpack, const float *__restrict__ bias,
                                                          float *__restrict__ out, int n, int W, int H, int Cout, int act, int ldi, int ldo, int coff)
{
    extern __shared__ __align__(16) float ws[];            /* [9*CIN][Cout] */
    const int K = 9 * CIN;
    for (int i = threadIdx.x; i < K * Cout; i += blockDim.x) ws[i] = wpack[i];
    __syncthreads();
    const int groups = Cout / CPT;                          /* channel groups per pixel quad */
    const int quad_in_block = threadIdx.x / groups, cg = threadIdx.x - quad_in_block * groups;
    const int qx = (W + 3) / 4;
    const long long total = (long long)n * H * qx;
    /* persistent CTAs: the filters are staged once, then the CTA walks its share of the pixel quads */
    const int qpb = blockDim.x / groups;
    for (long long quad = (long long)blockIdx.x * qpb + quad_in_block; quad < total; quad += (long long)gridDim.x * qpb) {
    const int xq = (int)(quad % qx);
    const long long t = quad / qx;
    const int y = (int)(t % H), b = (int)(t / H);
    const int x0 = xq * 4;

    float patch[3][6][CIN];
#pragma unroll
    for (int r = 0; r < 3; r++) {
        const int iy = y + r - 1;
#pragma unroll
        for (int s = 0; s < 6; s++) {
            const int ix = x0 + s - 1;
            const bool ok = iy >= 0 && iy < H && ix >= 0 && ix < W;
            const float *p = in + (((size_t)b * H + (ok ? iy : 0)) * W + (ok ? ix : 0)) * ldi;
#pragma unroll
            for (int c = 0; c < CIN; c++) patch[r][s][c] = ok ? __ldg(p + c) : 0.0f;
        }
    }
    float acc[4][CPT];
#pragma unroll
    for (int j = 0; j < CPT; j++) {
        const float bv = bias ? __ldg(bias + cg * CPT + j) : 0.0f;
#pragma unroll
        for (int px = 0; px < 4; px++) acc[px][j] = bv;
    }
#pragma unroll
    for (int ky = 0; ky < 3; ky++)
#pragma unroll
        for (int kx = 0; kx < 3; kx++)
#pragma unroll
            for (int c = 0; c < CIN; c++) {
                const float *wrow = ws + ((ky * 3 + kx) * CIN + c) * Cout + cg * CPT;
                float wv[CPT];
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(wrow + j);
                    wv[j] = w4.x; wv[j + 1] = w4.y; wv[j + 2] = w4.z; wv[j + 3] = w4.w;
                }
#pragma unroll
                for (int px = 0; px < 4; px++) {
                    const float a = patch[ky][px + kx][c];
#pragma unroll
                    for (int j = 0; j < CPT; j++) acc[px][j] = fmaf(a, wv[j], acc[px][j]);
                }
            }
#pragma unroll
    for (int px = 0; px < 4; px++) {
        if (x0 + px >= W) break;
        float *dst = out + (((size_t)b * H + y) * W + x0 + px) * ldo + coff + cg * CPT;
#pragma unroll
        for (int j = 0; j < CPT; j += 4)
            *reinterpret_cast<float4 *>(dst + j) = make_float4(drk_act(acc[px][j], act), drk_act(acc[px][j + 1], act),
                                                               drk_act(acc[px][j + 2], act), drk_act(acc[px][j + 3], act));
    }
    }
}

/* 0 if the shape is not one this kernel takes (the caller then uses the implicit GEMM) */
int drk_conv3x3_smallcin_launch(cudaStream_t st, const float *in, const float *wpack, const float *bias, float *out, int n, int W, int H,
                                int Cin, int Cout, int act, int ldi, int ldo, int coff, int *rc)
{
    if (Cin < 1 || Cin > 4 || Cout % CPT != 0 || Cout > 128 || Cout < CPT || 256 % (Cout / CPT) != 0) return 0;
    if (ldo % 4 || coff % 4 || ((uintptr_t)out % 16)) return 0;
    const int groups = Cout / CPT;
    const int threads = 256;
    const int qpb = threads / groups;
    const long long quads = (long long)n * H * ((W + 3) / 4);
    long long blocks = (quads + qpb - 1) / qpb;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (blocks > (long long)sms * 2) blocks = (long long)sms * 2;
    const size_t smem = (size_t)9 * Cin * Cout * sizeof(float);
    const int nthreads = threads;
    switch (Cin) {
    case 1: k_conv3x3_smallcin<1><<<(unsigned)blocks, nthreads, smem, st>>>(in, wpack, bias, out, n, W, H, Cout, act, ldi, ldo, coff); break;
    case 2: k_conv3x3_smallcin<2><<<(unsigned)blocks, nthreads, smem, st>>>(in, wpack, bias, out, n, W, H, Cout, act, ldi, ldo, coff); break;
    case 3: k_conv3x3_smallcin<3><<<(unsigned)blocks, nthreads, smem, st>>>(in, wpack, bias, out, n, W, H, Cout, act, ldi, ldo, coff); break;
    default: k_conv3x3_smallcin<4><<<(unsigned)blocks, nthreads, smem, st>>>(in, wpack, bias, out, n, W, H, Cout, act, ldi, ldo, coff); break;
    }
    DRK_COUNT_LAUNCH();
    *rc = DRK_LAUNCH_RESULT();
    return 1;
}
