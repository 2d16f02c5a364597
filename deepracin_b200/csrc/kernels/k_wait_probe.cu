/*
 * Test support for the failure path of the tensor-core kernels.  Those kernels bound every mbarrier wait
 * (mbar_wait / mbar_wait_warp in k_umma.cuh): when a wait runs out, the waiting role raises the CTA's abort flag,
 * writes a code to the graph's status word and every role leaves its loop.  In a healthy run no wait ever runs out, so
 * this probe makes one do so in the only harmless way: a single CTA waits, with a caller-given limit, on a barrier that
 * nothing ever arrives at.  It uses the same wait functions the kernels use, returns normally, and leaves the context
 * usable.  A second warp waits on a barrier that is arrived at, to show that the limit does not cut a good wait short.
 * The reference's counterpart is its return-code path (src/dR_clwrap.c:874-883, src/deepRACIN.c:230-234).
 */
#include "k_common.cuh"
#include "k_umma.cuh"

#define PROBE_CODE 9

__global__ void __launch_bounds__(64, 1) k_wait_probe(int *status, long long limit, int *result)
{
    __shared__ __align__(8) unsigned long long bar_mem[2];
    __shared__ int abort_flags[2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t never = smem_u32(&bar_mem[0]), arrived = smem_u32(&bar_mem[1]);
    if (threadIdx.x == 0) {
        mbar_init(never, 1);
        mbar_init(arrived, 1);
        abort_flags[0] = abort_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        const long long t0 = clock64();
        const bool ok = mbar_wait_warp(never, 0, &abort_flags[0], status, PROBE_CODE, limit);
        const long long waited = clock64() - t0;
        if (lane == 0) {
            result[0] = ok ? 1 : 0;
            result[2] = (int)min(waited >> 10, (long long)0x7fffffff);         /* units of 1024 clocks */
        }
    } else {
        if (lane == 0) mbar_arrive(arrived);
        const bool ok = mbar_wait_warp(arrived, 0, &abort_flags[1], NULL, PROBE_CODE + 1, limit);
        if (lane == 0) result[1] = ok ? 1 : 0;
    }
}

extern "C" int dRk_bounded_wait_probe(dRk_stream stream, int *status, long long limit_cycles, int *result)
{
    if (!status || !result || limit_cycles <= 0 || limit_cycles > 4000000000ll) return -1;
    k_wait_probe<<<1, 64, 0, drk_stream(stream)>>>(status, limit_cycles, result);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

/*
 * Measurement support: the rate at which this GPU retires FP32 fused multiply-adds from registers, as a yardstick for the
 * FFMA kernels (the nominal figure, SMs x 128 lanes x 2 x the maximum clock, is not reached even by a loop that touches no
 * memory).  Every thread runs an 8 x 8 register outer product -- the inner step of the FFMA GEMM, 32 packed FFMA2 or 64 scalar
 * FFMA per iteration, no loads -- for `iters` iterations; the launch fills every SM with `ctas_per_sm` CTAs of 256 threads.
 */
template <bool PACKED>
__global__ void __launch_bounds__(256) k_ffma_rate(float *sink, int iters, float seed)
{
    float2 acc[32], a[8], b[4];
#pragma unroll
    for (int i = 0; i < 32; i++) acc[i] = make_float2(threadIdx.x * 1e-3f + i, i * 0.5f);
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = make_float2(seed + i, seed - i);
#pragma unroll
    for (int i = 0; i < 4; i++) b[i] = make_float2(seed * i, seed + 2 * i);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float2 a2 = make_float2(a[i].x, a[i].x);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (PACKED) acc[i * 4 + j] = __ffma2_rn(a2, b[j], acc[i * 4 + j]);
                else {
                    acc[i * 4 + j].x = fmaf(a[i].x, b[j].x, acc[i * 4 + j].x);
                    acc[i * 4 + j].y = fmaf(a[i].x, b[j].y, acc[i * 4 + j].y);
                }
            }
        }
    }
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) r += acc[i].x + acc[i].y;
    sink[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = r;
}

extern "C" int dRk_ffma_rate_probe(dRk_stream stream, float *sink, size_t sink_floats, int packed, int iters, double *tflops)
{
    if (!sink || !tflops || iters <= 0 || iters > (1 << 22)) return -1;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    const int grid = sms * 4;
    if (sink_floats < (size_t)grid * 256) return -3;
    cudaStream_t st = drk_stream(stream);
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1;
    float best = 1e30f;
    for (int r = 0; r < 4; r++) {          /* the first run warms up */
        cudaEventRecord(e0, st);
        if (packed) k_ffma_rate<true><<<grid, 256, 0, st>>>(sink, r ? iters : 64, 1e-7f);
        else k_ffma_rate<false><<<grid, 256, 0, st>>>(sink, r ? iters : 64, 1e-7f);
        DRK_COUNT_LAUNCH();
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) { cudaEventDestroy(e0); cudaEventDestroy(e1); return (int)cudaGetLastError(); }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tflops = 2.0 * 64.0 * iters * 256.0 * grid / ((double)best * 1e-3) / 1e12;
    return DRK_LAUNCH_RESULT();
}
