/*
 * Fully connected layer, exact FP32.  The weight matrix [Nin][Nout] is the only large
 * operand (VGG fc6: 411 MB) and is read exactly once per batch:
 *   - weight-streaming kernels: a warp owns 128 output columns and walks a K-slice with
 *     128-bit loads, keeping batch x 4 accumulators per lane; the CTA's warps split the slice
 *     and combine through shared memory; K is split across CTAs so that about two CTAs per SM
 *     keep HBM busy.  HBM-bound: Nin*Nout*4 bytes per pass.  Batch 1 loads weight rows into
 *     registers (k_fc_stream); 2..16 rows stage them through shared memory with cp.async
 *     (k_fc_stream_async: 0.90-0.97 of the measured HBM copy rate on 25088 -> 4096 up to batch
 *     8, FFMA-limited at 16); up to 32 rows -- 64 for matrices of 256 MB and more -- run in
 *     passes of 16, which re-read the weights per pass but still beat
 *   - the FFMA GEMM core, batched over K-slices (every other shape).
 * Both write per-slice partial sums to scratch; a second launch adds them, the bias and
 * applies the activation -- the same two-step shape as the reference's
 * matrixVectorMultFirst / matrixVectorMultSecond (Kernels/dR_fcl.cl:59-120).
 */
#include <stdio.h>
#include "k_common.cuh"
#include "k_gemm_f32.cuh"

#define FC_COLS 128        /* output columns per CTA (32 lanes x float4) */
#define FC_WARPS 8
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
#pragma unroll
        for (int b = 0; b < NB; b++)        /* rows past nb feed accumulators that are never stored */
            for (int k = threadIdx.x; k < kn; k += blockDim.x) xs[b][k] = b < nb ? in[(size_t)b * Nin + k0 + k] : 0.f;
        __syncthreads();
        if (colok) {
            /* warp `warp` takes rows warp, warp+8, ...; four rows in flight per lane */
            int k = warp;
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

/*
 * The same slice product for 2..16 batch rows with the weight rows staged through shared memory by cp.async, so that the
 * bytes in flight (what an HBM-bound kernel needs, about 1 us x 6.5 TB/s over the GPU) cost no registers: every lane owns a
 * private FIFO of FC_ASYNC_DEPTH steps x 4 rows x 16 bytes (64 KiB per CTA, two CTAs per SM) -- it reads back exactly the bytes it copied, so the weight path
 * needs no barrier at all, only cp.async.wait_group.  The input slice goes through two shared-memory buffers of 256 rows (next
 * stage fetched into registers while this one multiplies, stored just before the stage's only barrier).  Rows past the slice
 * end are copied as zeros (cp.async with source size 0), so there is no tail loop.
 */
#define FC_ASYNC_ROWS 4
#define FC_ASYNC_DEPTH 4        /* a power of two: the slot counter wraps with a mask */
#define FC_ASYNC_SMEM(NB) (FC_WARPS * FC_ASYNC_DEPTH * FC_ASYNC_ROWS * 32 * 16)

template <int NB>
__global__ void __launch_bounds__(FC_WARPS * 32) k_fc_stream_async(const float *__restrict__ in, const float *__restrict__ w, float *__restrict__ partial,
                                                                  int nb, int Nin, int Nout, int kchunk, int ntotal, int b0)
{
    constexpr int KS = FC_WARPS * 32;               /* rows per input stage = threads per CTA */
    constexpr int R = FC_ASYNC_ROWS, S = FC_ASYNC_DEPTH;
    constexpr int SPS = KS / (FC_WARPS * R);        /* steps per input stage (8) */
    extern __shared__ __align__(16) float4 ring[];  /* [warp][slot][row][lane] */
    __shared__ __align__(16) float xs[2][NB / 2][KS][2];     /* batch rows interleaved in pairs: (x[2p][k], x[2p+1][k]) */
    __shared__ float4 red[FC_WARPS][32];
    drk_dep_trigger();
    drk_dep_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = blockIdx.x * FC_COLS + lane * 4;
    const int kbeg = blockIdx.y * kchunk;
    const int kend = min(Nin, kbeg + kchunk);
    const bool colok = col < Nout;
    const int nsteps = (kend - kbeg + FC_WARPS * R - 1) / (FC_WARPS * R);
    const int nstages = (nsteps + SPS - 1) / SPS;
    const float4 *mine = ring + (size_t)warp * S * R * 32 + lane;
    const uint32_t mine_u = (uint32_t)__cvta_generic_to_shared(mine);

    /* producer state: the next step to copy -- its first row for this warp, that row's address, its FIFO slot */
    int p_row = kbeg + warp * R, p_slot = 0;
    const float *p_src = w + (colok ? col : 0) + (size_t)p_row * Nout;
    const size_t step_floats = (size_t)FC_WARPS * R * Nout;
    /* copy the four rows of the next step into its slot (zeros past the slice end or the last column) and close the group */
    auto issue = [&]() {
#pragma unroll
        for (int d = 0; d < R; d++) {
            const bool ok = colok && p_row + d < kend;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(mine_u + (uint32_t)((p_slot * R + d) * 32 * 16)),
                         "l"(ok ? p_src + (size_t)d * Nout : w), "r"(ok ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        p_row += FC_WARPS * R;
        p_src += step_floats;
        p_slot = (p_slot + 1) & (S - 1);
    };

    /* accumulators as pairs of batch rows per output column: one packed FFMA2 (fma.rn.f32x2: two IEEE round-to-nearest FMAs,
       the same results as two scalar ones) per pair, with the weight duplicated into both halves once per step */
    float2 acc[NB / 2][4];
#pragma unroll
    for (int p = 0; p < NB / 2; p++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[p][c] = make_float2(0.f, 0.f);
    float xr[NB];
#pragma unroll
    for (int g = 0; g < S; g++) issue();
#pragma unroll
    for (int b = 0; b < NB; b++) xs[0][b >> 1][tid][b & 1] = (b < nb && kbeg + tid < kend) ? __ldg(in + (size_t)b * Nin + kbeg + tid) : 0.f;
    __syncthreads();
    for (int s = 0; s < nstages; s++) {
        const int buf = s & 1;
        const bool more = s + 1 < nstages;
        if (more) {
            const int k = kbeg + (s + 1) * KS + tid;
#pragma unroll
            for (int b = 0; b < NB; b++) xr[b] = (b < nb && k < kend) ? __ldg(in + (size_t)b * Nin + k) : 0.f;
        }
        const int jn = min(SPS, nsteps - s * SPS);
#pragma unroll 1
        for (int j = 0; j < jn; j++) {
            asm volatile("cp.async.wait_group %0;" ::"n"(S - 1) : "memory");
            float2 wd[R][4];
#pragma unroll
            for (int d = 0; d < R; d++) {       /* the producer's next slot is the oldest one: the step to consume, refilled right after */
                const float4 t = mine[(p_slot * R + d) * 32];
                wd[d][0] = make_float2(t.x, t.x); wd[d][1] = make_float2(t.y, t.y); wd[d][2] = make_float2(t.z, t.z); wd[d][3] = make_float2(t.w, t.w);
            }
            issue();
#pragma unroll
            for (int p = 0; p < NB / 2; p++) {
                const float4 *xp = reinterpret_cast<const float4 *>(&xs[buf][p][(j * FC_WARPS + warp) * R][0]);
                const float4 x01 = xp[0], x23 = xp[1];          /* rows k, k+1 and k+2, k+3 of both batch rows */
                const float2 xk[R] = {make_float2(x01.x, x01.y), make_float2(x01.z, x01.w), make_float2(x23.x, x23.y), make_float2(x23.z, x23.w)};
#pragma unroll
                for (int d = 0; d < R; d++)
#pragma unroll
                    for (int c = 0; c < 4; c++) acc[p][c] = __ffma2_rn(xk[d], wd[d][c], acc[p][c]);
            }
        }
        if (more) {
#pragma unroll
            for (int b = 0; b < NB; b++) xs[buf ^ 1][b >> 1][tid][b & 1] = xr[b];
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int b = 0; b < NB; b++) {
        __syncthreads();
        red[warp][lane] = (b & 1) ? make_float4(acc[b >> 1][0].y, acc[b >> 1][1].y, acc[b >> 1][2].y, acc[b >> 1][3].y)
                                  : make_float4(acc[b >> 1][0].x, acc[b >> 1][1].x, acc[b >> 1][2].x, acc[b >> 1][3].x);
        __syncthreads();
        if (warp == 0 && b < nb && colok) {
            float4 s4 = red[0][lane];
#pragma unroll
            for (int wi = 1; wi < FC_WARPS; wi++) {
                const float4 t = red[wi][lane];
                s4.x += t.x; s4.y += t.y; s4.z += t.z; s4.w += t.w;
            }
            *reinterpret_cast<float4 *>(partial + ((size_t)blockIdx.y * ntotal + b0 + b) * Nout + col) = s4;
        }
    }
}

template <int NB>
static int fc_async_launch(cudaStream_t st, dim3 grid, const float *in, const float *w, float *scratch, int n, int Nin, int Nout, int kchunk,
                           int ntotal, int b0)
{
    static bool attr_done[64];                      /* the opt-in shared-memory size is a per-device function attribute */
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_fc_stream_async<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, FC_ASYNC_SMEM(NB));
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    drk_launch_dep(k_fc_stream_async<NB>, grid, dim3(FC_WARPS * 32), (size_t)FC_ASYNC_SMEM(NB), st, in, w, scratch, n, Nin, Nout, kchunk, ntotal, b0);
    return 0;
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

/* does the weight-streaming path take n rows of a Nin x Nout layer?  (measured against the K-sliced GEMM: 25088 x 4096 wins up to
   batch 64, 4096 x 4096 up to 32) */
static bool fc_streams(int n, int Nin, int Nout)
{
    if (Nout % 4 != 0) return false;
    return n <= 32 || (n <= 64 && (size_t)Nin * Nout >= ((size_t)64 << 20));
}

static int fc_splits(int n, int Nin, int Nout)
{
    /* aim for roughly 4 CTAs per SM; keep slices a multiple of 64 rows and at least 256 long */
    const int colBlocks = fc_streams(n, Nin, Nout) ? (Nout + FC_COLS - 1) / FC_COLS
                                                        : ((Nout + 127) / 128) * ((n + 127) / 128);
    int splits = 4 * 148 / colBlocks;           /* rounded down: a few CTAs past a whole wave would cost a wave */
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
    int kchunk = fc_kchunk(Nin, splits);
    if (!fc_streams(n, Nin, Nout)) {
        /* the GEMM path runs equal slices in one launch and a shorter last slice in a second one: prefer a slightly longer
           slice that divides Nin (never a shorter one: the scratch is sized for at most fc_splits() slices) */
        for (int kc = kchunk; kc <= kchunk + kchunk / 2; kc += 64)
            if (Nin % kc == 0) { kchunk = kc; break; }
    }
    splits = (Nin + kchunk - 1) / kchunk;       /* drop empty trailing slices */
    int rc;
    if (fc_streams(n, Nin, Nout) && ((uintptr_t)w % 16) == 0 && ((uintptr_t)scratch % 16) == 0) {
        dim3 grid((Nout + FC_COLS - 1) / FC_COLS, splits);
        if (n <= 1) {
            drk_launch_dep(k_fc_stream<1>, grid, dim3(FC_WARPS * 32), 0, st, in, w, scratch, n, Nin, Nout, kchunk);
        } else {
            /* 2..16 rows in one pass; more rows in passes of 16 (the weights are then read once per pass) */
            for (int b0 = 0; b0 < n; b0 += 16) {
                const int nb = n - b0 < 16 ? n - b0 : 16;
                const float *src = in + (size_t)b0 * Nin;
                int arc;
                if (nb <= 2) arc = fc_async_launch<2>(st, grid, src, w, scratch, nb, Nin, Nout, kchunk, n, b0);
                else if (nb <= 4) arc = fc_async_launch<4>(st, grid, src, w, scratch, nb, Nin, Nout, kchunk, n, b0);
                else if (nb <= 8) arc = fc_async_launch<8>(st, grid, src, w, scratch, nb, Nin, Nout, kchunk, n, b0);
                else arc = fc_async_launch<16>(st, grid, src, w, scratch, nb, Nin, Nout, kchunk, n, b0);
                if (arc) return arc;
                if (b0 + 16 < n) DRK_COUNT_LAUNCH();
            }
        }
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
 * a call only enqueues the same kernels as dRk_fc_f32 -- no cudaMalloc, cudaFree or any other
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
