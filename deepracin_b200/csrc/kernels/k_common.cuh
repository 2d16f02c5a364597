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
