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
