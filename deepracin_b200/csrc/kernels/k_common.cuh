/* Shared helpers of the kernel translation units: launch accounting and small device utilities. */
#pragma once
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include "dR_kernels.h"

extern thread_local long g_dRk_launches;
#define DRK_COUNT_LAUNCH() (++g_dRk_launches)
/* returns the launch error (if any) of the kernel just enqueued */
#define DRK_LAUNCH_RESULT() ((int)cudaPeekAtLastError())

static inline cudaStream_t drk_stream(dRk_stream s) { return (cudaStream_t)s; }
static inline unsigned drk_blocks(size_t work, unsigned per_block, unsigned cap = 0x7fffffffu)
{
    size_t b = (work + per_block - 1) / per_block;
    if (b < 1) b = 1;
    return (unsigned)(b > cap ? cap : b);
}

/* ReLU / linear as the reference kernels write them: clamp(v, 0, FLT_MAX) */
__device__ __forceinline__ float drk_act(float v, int act)
{
    if (act) v = fminf(fmaxf(v, 0.0f), FLT_MAX);
    return v;
}

/*
 * Programmatic dependent launch: a kernel launched through drk_launch_dep may start while its predecessor on
 * the stream is still running; it must call drk_dep_wait() before it touches memory the predecessor writes (or reads
 * and this kernel overwrites).  drk_dep_trigger() at a kernel's top lets its own successor be scheduled early; the
 * successor's wait still returns only when this grid has completed and its writes are visible.  What overlaps is the
 * launch latency and the successor's set-up (barrier initialisation, TMEM allocation, constant operands).
 * DRK_NO_DEP_LAUNCH=1 in the environment restores plain stream order (for A/B timing).
 */
__device__ __forceinline__ void drk_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void drk_dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int drk_dep_launch_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t drk_launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = drk_dep_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
