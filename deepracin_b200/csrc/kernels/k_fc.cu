/*
 * Fully connected layer, exact FP32.  The weight matrix [Nin][Nout] is the only large
 * operand (VGG fc6: 411 MB) and is read exactly once per batch:
 *   - batch <= 16: weight-streaming kernel; a warp owns 128 output columns and walks a
 *     K-slice with 128-bit loads, keeping batch x 4 accumulators per lane; the CTA's warps
 *     split the slice and combine through shared memory; K is split across CTAs so that a few
 *     hundred CTAs keep HBM busy.  HBM-bound: Nin*Nout*4 bytes per call.
 *   - larger batches: the FFMA GEMM core, batched over K-slices.
 * Both write per-slice partial sums to scratch; a second launch adds them, the bias and
 * applies the activation -- the same two-step shape as the reference's
 * matrixVectorMultFirst / matrixVectorMultSecond (Kernels/dR_fcl.cl:59-120).
 */
#include <stdio.h>
#include "k_common.cuh"
#include "k_gemm_f32.cuh"

#define FC_COLS 128        /* output columns per CTA (32 lanes x float4) */
#define FC_WARPS 8
#define FC_MAXB 16
#define FC_KSTAGE 256      /* input values staged in shared memory per step */

template <int NB>
__global__ void __launch_bounds__(FC_WARPS * 32) k_fc_stream(const float *__restrict__ in, const float *__restrict__ w, float *__restrict__ partial,
                                                            int nb, int Nin, int Nout, int kchunk)
{
    __shared__ float xs[NB][FC_KSTAGE];
    __shared__ float4 red[FC_WARPS][32];
    drk_dep_trigger();
    drk_dep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * FC_COLS + lane * 4;
    const int kbeg = blockIdx.y * kchunk;
    const int kend = min(Nin, kbeg + kchunk);
    const bool colok = col < Nout;      /* Nout % 4 == 0 is guaranteed by the launcher */
    float4 acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int k0 = kbeg; k0 < kend; k0 += FC_KSTAGE) {
        const int kn = min(FC_KSTAGE, kend - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < NB * FC_KSTAGE; i += blockDim.x) {
            const int b = i / FC_KSTAGE, k = i % FC_KSTAGE;
            xs[b][k] = (b < nb && k < kn) ? in[(size_t)b * Nin + k0 + k] : 0.f;
        }
        __syncthreads();
        if (colok) {
            /* warp `warp` takes rows warp, warp+8, ...; D rows in flight per lane.  With four or more batch rows the FMAs
               of a step take long enough to matter, so the D weight rows of the next step are requested before them. */
            int k = warp;
            if (NB <= 2) {
                for (; k + 3 * FC_WARPS < kn; k += 4 * FC_WARPS) {
                    float4 w0 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(k0 + k) * Nout + col));
                    float4 w1 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(k0 + k + FC_WARPS) * Nout + col));
                    float4 w2 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(k0 + k + 2 * FC_WARPS) * Nout + col));
                    float4 w3 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(k0 + k + 3 * FC_WARPS) * Nout + col));
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const float x0 = xs[b][k], x1 = xs[b][k + FC_WARPS], x2 = xs[b][k + 2 * FC_WARPS], x3 = xs[b][k + 3 * FC_WARPS];
                        acc[b].x = fmaf(x0, w0.x, acc[b].x); acc[b].y = fmaf(x0, w0.y, acc[b].y); acc[b].z = fmaf(x0, w0.z, acc[b].z); acc[b].w = fmaf(x0, w0.w, acc[b].w);
                        acc[b].x = fmaf(x1, w1.x, acc[b].x); acc[b].y = fmaf(x1, w1.y, acc[b].y); acc[b].z = fmaf(x1, w1.z, acc[b].z); acc[b].w = fmaf(x1, w1.w, acc[b].w);
                        acc[b].x = fmaf(x2, w2.x, acc[b].x); acc[b].y = fmaf(x2, w2.y, acc[b].y); acc[b].z = fmaf(x2, w2.z, acc[b].z); acc[b].w = fmaf(x2, w2.w, acc[b].w);
                        acc[b].x = fmaf(x3, w3.x, acc[b].x); acc[b].y = fmaf(x3, w3.y, acc[b].y); acc[b].z = fmaf(x3, w3.z, acc[b].z); acc[b].w = fmaf(x3, w3.w, acc[b].w);
                    }
                }
            } else {
                constexpr int D = NB <= 4 ? 8 : 4;
                float4 wv[D], nv[D];
                const float *wp = w + (size_t)(k0 + k) * Nout + col;
                const size_t rs = (size_t)FC_WARPS * Nout;
                bool have = k + (D - 1) * FC_WARPS < kn;
                if (have) {
#pragma unroll
                    for (int d = 0; d < D; d++) wv[d] = __ldg(reinterpret_cast<const float4 *>(wp + d * rs));
                }
                while (have) {
                    const int kc = k;
                    k += D * FC_WARPS;
                    wp += D * rs;
                    have = k + (D - 1) * FC_WARPS < kn;
                    if (have) {
#pragma unroll
                        for (int d = 0; d < D; d++) nv[d] = __ldg(reinterpret_cast<const float4 *>(wp + d * rs));
                    }
#pragma unroll
                    for (int b = 0; b < NB; b++) {
#pragma unroll
                        for (int d = 0; d < D; d++) {
                            const float x = xs[b][kc + d * FC_WARPS];
                            acc[b].x = fmaf(x, wv[d].x, acc[b].x); acc[b].y = fmaf(x, wv[d].y, acc[b].y);
                            acc[b].z = fmaf(x, wv[d].z, acc[b].z); acc[b].w = fmaf(x, wv[d].w, acc[b].w);
                        }
                    }
                    if (have) {
#pragma unroll
                        for (int d = 0; d < D; d++) wv[d] = nv[d];
                    }
                }
            }
            for (; k < kn; k += FC_WARPS) {
                float4 w0 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(k0 + k) * Nout + col));
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const float x0 = xs[b][k];
                    acc[b].x = fmaf(x0, w0.x, acc[b].x); acc[b].y = fmaf(x0, w0.y, acc[b].y); acc[b].z = fmaf(x0, w0.z, acc[b].z); acc[b].w = fmaf(x0, w0.w, acc[b].w);
                }
            }
        }
    }
    /* combine the CTA's warps, one batch row at a time */
#pragma unroll
    for (int b = 0; b < NB; b++) {
        __syncthreads();
        red[warp][lane] = acc[b];
        __syncthreads();
        if (warp == 0 && b < nb && colok) {
            float4 s = red[0][lane];
#pragma unroll
            for (int wv = 1; wv < FC_WARPS; wv++) {
                const float4 t = red[wv][lane];
                s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
            }
            *reinterpret_cast<float4 *>(partial + ((size_t)blockIdx.y * nb + b) * Nout + col) = s;
        }
    }
}

/* out[b][o] = clamp(act(bias[o] + sum_s partial[s][b][o])) -- step two of the reference (Kernels/dR_fcl.cl:99-120) */
__global__ void k_fc_reduce(const float *__restrict__ partial, const float *__restrict__ bias, float *__restrict__ out,
                            int total, int Nout, int splits, int act)
{
    drk_dep_trigger();
    drk_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float s = 0.f;
    for (int p = 0; p < splits; p++) s += partial[(size_t)p * total + i];
    if (bias) s += bias[i % Nout];
    out[i] = act ? fminf(fmaxf(s, 0.0f), FLT_MAX) : fminf(fmaxf(s, -FLT_MAX), FLT_MAX);
}

int drk_fc_reduce_launch(cudaStream_t st, const float *partial, const float *bias, float *out, int total, int Nout, int splits, int act)
{
    drk_launch_dep(k_fc_reduce, dim3((total + 255) / 256), dim3(256), 0, st, partial, bias, out, total, Nout, splits, act);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

static int fc_splits(int n, int Nin, int Nout)
{
    /* aim for roughly 4 CTAs per SM; keep slices a multiple of 64 rows and at least 256 long */
    const int colBlocks = n <= FC_MAXB && Nout % 4 == 0 ? (Nout + FC_COLS - 1) / FC_COLS
                                                        : ((Nout + 127) / 128) * ((n + 127) / 128);
    int splits = (4 * 148 + colBlocks - 1) / colBlocks;
    const int maxSplits = Nin / 256 > 0 ? Nin / 256 : 1;
    if (splits > maxSplits) splits = maxSplits;
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    return splits;
}

static int fc_kchunk(int Nin, int splits)
{
    int kc = (Nin + splits - 1) / splits;
    kc = (kc + 63) / 64 * 64;
    return kc;
}

extern "C" size_t dRk_fc_scratch_floats(int n, int Nin, int Nout)
{
    if (n <= 0 || Nin <= 0 || Nout <= 0) return 0;
    const int splits = fc_splits(n, Nin, Nout);
    return (size_t)splits * n * Nout;
}

extern "C" int dRk_fc_f32(dRk_stream stream, const float *in, const float *w, const float *bias, float *out, float *scratch,
                          int n, int Nin, int Nout, int act)
{
    if (n <= 0 || Nin <= 0 || Nout <= 0 || !scratch) return -1;
    cudaStream_t st = drk_stream(stream);
    int splits = fc_splits(n, Nin, Nout);
    const int kchunk = fc_kchunk(Nin, splits);
    splits = (Nin + kchunk - 1) / kchunk;       /* drop empty trailing slices */
    int rc;
    if (n <= FC_MAXB && Nout % 4 == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)scratch % 16) == 0) {
        dim3 grid((Nout + FC_COLS - 1) / FC_COLS, splits);
        if (n <= 1) drk_launch_dep(k_fc_stream<1>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        else if (n <= 2) drk_launch_dep(k_fc_stream<2>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        else if (n <= 4) drk_launch_dep(k_fc_stream<4>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        else if (n <= 8) drk_launch_dep(k_fc_stream<8>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        else drk_launch_dep(k_fc_stream<16>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        DRK_COUNT_LAUNCH();
        rc = DRK_LAUNCH_RESULT();
    } else {
        /* K-sliced GEMM: slice z multiplies A[:, z*kchunk : ...] by B[z*kchunk : ..., :]; the last slice may be shorter,
           so it is launched separately when Nin is not a multiple of kchunk */
        const int full = Nin / kchunk, tail = Nin - full * kchunk;
        rc = 0;
        if (full > 0)
            rc = drk_gemm_f32_launch(st, in, w, NULL, scratch, n, Nout, kchunk, Nin, Nout, Nout, 0, 0, full,
                                     (size_t)kchunk, (size_t)kchunk * Nout, (size_t)n * Nout, NULL);
        if (rc == 0 && tail > 0)
            rc = drk_gemm_f32_launch(st, in + (size_t)full * kchunk, w + (size_t)full * kchunk * Nout, NULL,
                                     scratch + (size_t)full * n * Nout, n, Nout, tail, Nin, Nout, Nout, 0, 0, 1, 0, 0, 0, NULL);
    }
    if (rc != 0) return rc;
    const int total = n * Nout;
    drk_launch_dep(k_fc_reduce, dim3((total + 255) / 256), dim3(256), 0, st, scratch, bias, out, total, Nout, splits, act);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

/*
 * Fully connected layer for callers that must not allocate.
 *
 * Some embedders of this library are not allowed to create device memory once they are running:
 * control loops with a memory budget that is frozen after start-up, and plug-in hosts that own
 * every device allocation themselves and only lend the library a stream plus input/output
 * pointers.  They cannot give dRk_fc_f32 the split-K scratch it needs, so this entry point brings
 * its own: a fixed array that is part of the library image (DRK_FC_STATIC_SCRATCH_FLOATS floats,
 * 8 MiB, resident on every GPU that loads the library until the process exits).
 *
 * The first call on each device looks the array's device address up (once, with that device
 * current) and remembers it; make that first call before starting any stream capture.  After that
 * a call only enqueues the same two kernels as dRk_fc_f32 -- no cudaMalloc, cudaFree or any other
 * allocating routine.  Shapes whose partial sums do not fit the array are refused with -4 and a
 * message naming the limit.  All calls on a device share the array: it keeps whatever the last
 * call left in it (every element a call reads was written by that same call first, so nothing has
 * to be cleared), and two calls that may overlap on the GPU (different streams) would race on it.
 * The device that is current at the call must be the stream's device (checked: -6 otherwise).
 */
#define DRK_FC_STATIC_SCRATCH_FLOATS (2u << 20)
static __device__ __align__(256) float g_fc_static_scratch[DRK_FC_STATIC_SCRATCH_FLOATS];
static float *g_fc_static_scratch_addr[64];     /* device address per device ordinal, filled on first use */

extern "C" int dRk_fc_f32_noalloc(dRk_stream stream, const float *in, const float *w, const float *bias, float *out,
                                  int n, int Nin, int Nout, int act)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return -1;
    {
        /* the array's address is looked up for the CURRENT device: the stream must belong to it */
        int sdev = dev;
        if (cudaStreamGetDevice(drk_stream(stream), &sdev) == cudaSuccess && sdev != dev) {
            fprintf(stderr, "dRk_fc_f32_noalloc: the stream belongs to device %d but device %d is current\n", sdev, dev);
            return -6;
        }
        (void)cudaGetLastError();
    }
    if (!__atomic_load_n(&g_fc_static_scratch_addr[dev], __ATOMIC_ACQUIRE)) {
        /* in host code the array's name is only a handle; the kernels need its device address */
        float *addr = NULL;
        e = cudaGetSymbolAddress((void **)&addr, g_fc_static_scratch);
        if (e != cudaSuccess || !addr) {
            fprintf(stderr, "dRk_fc_f32_noalloc: cannot resolve the built-in scratch array on device %d: %s\n", dev, cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : -1;
        }
        __atomic_store_n(&g_fc_static_scratch_addr[dev], addr, __ATOMIC_RELEASE);      /* threads racing here store the same value */
    }
    const size_t need = dRk_fc_scratch_floats(n, Nin, Nout);
    if (need == 0) return -1;
    if (need > DRK_FC_STATIC_SCRATCH_FLOATS) {
        fprintf(stderr, "dRk_fc_f32_noalloc: batch %d x %d -> %d needs %zu scratch floats, the built-in array holds %u; "
                        "use dRk_fc_f32 with caller-provided scratch\n", n, Nin, Nout, need, DRK_FC_STATIC_SCRATCH_FLOATS);
        return -4;
    }
    return dRk_fc_f32(stream, in, w, bias, out, g_fc_static_scratch_addr[dev], n, Nin, Nout, act);
}
