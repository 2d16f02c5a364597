/*
 * Microbenchmark of the tcgen05.mma (kind::tf32) issue rate on sm_100a, the measurement the tensor kernels' tile shapes
 * and issue loops rest on.  One CTA per SM; one thread issues MMAs on operands that sit (zeroed) in shared memory.
 *   part 1: back-to-back MMAs, nothing else, for several (M, N): clocks the tensor pipe needs per instruction;
 *   part 2: groups of four MMAs (one 128-byte K slab) fed through a ring of shared-memory stages that a producer thread
 *           fills with bulk copies from an L2-resident buffer, full/empty mbarriers as in the convolution kernels, with
 *           three versions of the issuer's loop: bounded wait as an out-of-line call, first probe inline, and probe of
 *           the next stage between MMA 2 and 3 with the commit deferred.
 * Every wait is bounded (k_umma.cuh); the program allocates ~33 MB and runs a few milliseconds.
 * Build: python deepracin_b200/build.py --microbench     Run: deepracin_b200/csrc/microbench/mma_rate
 */
#include <cstdio>
#include <cuda_runtime.h>
#include "../kernels/k_umma.cuh"

__device__ __host__ constexpr uint32_t idesc_mn(int bm, int bn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(bm >> 4) << 24);
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

#define NST 5                       /* ring stages of 32 KB */
#define SMEM_BYTES ((16 + NST * 32) * 1024 + 2048)

/* V = 0: part 1 (no ring); 1: out-of-line wait; 2: inline first probe; 3: look-ahead probe + deferred commit */
template <int V, int MM, int BN, int SBO = 1024>
__global__ void __launch_bounds__(192, 1) k_rate(int groups, const float *src, size_t src_floats, long long *out, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t a_base = base, b_base = base + 16 * 1024;
    const uint32_t bars = b_base + NST * 32 * 1024;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + 16 * 1024 + NST * 32 * 1024 + 128);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (NST + s); };
    const uint32_t donebar = bars + 8u * (2 * NST);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (16 + NST * 32) * 1024 / 4; i += blockDim.x) reinterpret_cast<float *>(gen)[i] = 0.0f;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(donebar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 0 && lane == 0 && V > 0) {
        int s = 0;
        uint32_t ph = 0;
        size_t off = (size_t)blockIdx.x * 8192;
        for (int g = 0; g < groups; g++) {
            if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, 1)) break;
            mbar_expect_tx(full(s), 32768u);
            bulk_load(b_base + s * 32 * 1024, src + off, 32768u, full(s));
            off += 8192;
            if (off + 8192 > src_floats) off = 0;
            if (++s == NST) { s = 0; ph ^= 1u; }
        }
        for (int i = 0; i < NST; i++) {         /* nothing may land after the CTA has gone */
            const long long t0 = clock64();
            while (!mbar_try(full(i), 0) && !mbar_try(full(i), 1) && clock64() - t0 < 1000000) { }
        }
    } else if (warp == 1 && lane == 0) {
        const uint64_t adesc = make_smem_desc(a_base);
        constexpr uint32_t idesc = idesc_mn(MM, BN);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        const long long t0 = clock64();
        if (V == 0) {
            const uint64_t bdesc = SBO == 1024 ? make_smem_desc(b_base) : make_smem_desc_sbo(b_base, SBO);
            for (int g = 0; g < groups; g++) {
#pragma unroll
                for (int j = 0; j < 4; j++) umma_tf32(tmem_base, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, 1u);
            }
        } else if (V <= 2) {
            for (int g = 0; g < groups && ok; g++) {
                ok = V == 1 ? mbar_wait_slow(full(s), ph, abort_flag, status, 3) : mbar_wait(full(s), ph, abort_flag, status, 3);
                if (!ok) break;
                const uint64_t bdesc = make_smem_desc(b_base + s * 32 * 1024);
#pragma unroll
                for (int j = 0; j < 4; j++) umma_tf32(tmem_base, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, 1u);
                umma_commit(empty(s));
                if (++s == NST) { s = 0; ph ^= 1u; }
            }
        } else {
            bool ready = mbar_try(full(0), 0) != 0;
            uint32_t pending = 0;
            for (int g = 0; g < groups && ok; g++) {
                if (!ready) ok = mbar_wait(full(s), ph, abort_flag, status, 3);
                if (!ok) break;
                const uint64_t bdesc = make_smem_desc(b_base + s * 32 * 1024);
                umma_tf32(tmem_base, adesc, bdesc, idesc, 1u);
                umma_tf32(tmem_base, adesc + 2, bdesc + 2, idesc, 1u);
                if (pending) umma_commit(pending);
                int ns = s + 1;
                uint32_t nph = ph;
                if (ns == NST) { ns = 0; nph ^= 1u; }
                ready = (g + 1 < groups) && mbar_try(full(ns), nph) != 0;
                umma_tf32(tmem_base, adesc + 4, bdesc + 4, idesc, 1u);
                umma_tf32(tmem_base, adesc + 6, bdesc + 6, idesc, 1u);
                pending = empty(s);
                s = ns; ph = nph;
            }
            if (pending) umma_commit(pending);
        }
        umma_commit(donebar);
        ok = mbar_wait(donebar, 0, abort_flag, status, 9) && ok;
        const long long t1 = clock64();
        if (blockIdx.x == 0) out[0] = ok ? (t1 - t0) : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <int V, int MM, int BN, int SBO = 1024>
static void run(const char *what, const float *src, size_t src_floats, long long *out, int *status)
{
    const int groups = 4096;
    cudaFuncSetAttribute(k_rate<V, MM, BN, SBO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaMemset(out, 0, 64);
    cudaMemset(status, 0, 4);
    for (int rep = 0; rep < 2; rep++) k_rate<V, MM, BN, SBO><<<148, 192, SMEM_BYTES, 0>>>(groups, src, src_floats, out, status);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h = 0;
    int st = 0;
    cudaMemcpy(&h, out, 8, cudaMemcpyDeviceToHost);
    cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    printf("%-78s M=%3d N=%3d  %s status=%d  clocks/MMA=%.1f\n", what, MM, BN, cudaGetErrorString(e), st, (double)h / (groups * 4.0));
}

int main()
{
    long long *out;
    int *status;
    float *src;
    const size_t src_floats = 8u << 20;         /* 32 MB: stays in L2 */
    if (cudaMalloc(&out, 64) || cudaMalloc(&status, 4) || cudaMalloc(&src, src_floats * 4)) { printf("no device memory\n"); return 1; }
    cudaMemset(src, 0, src_floats * 4);
    run<0, 128, 256>("back to back", src, src_floats, out, status);
    run<0, 128, 128>("back to back", src, src_floats, out, status);
    run<0, 128, 64>("back to back", src, src_floats, out, status);
    run<0, 128, 32>("back to back", src, src_floats, out, status);
    run<0, 128, 256, 1280>("back to back, B groups of 8 rows 1280 bytes apart", src, src_floats, out, status);
    run<0, 128, 224, 1280>("back to back, B groups of 8 rows 1280 bytes apart", src, src_floats, out, status);
    run<0, 128, 224>("back to back", src, src_floats, out, status);
    run<0, 64, 256>("back to back", src, src_floats, out, status);
    run<0, 64, 128>("back to back", src, src_floats, out, status);
    run<1, 128, 256>("ring of 32 KB bulk loads per 4 MMAs, bounded wait as an out-of-line call", src, src_floats, out, status);
    run<2, 128, 256>("ring, first probe of the wait inline", src, src_floats, out, status);
    run<3, 128, 256>("ring, next stage probed between MMA 2 and 3, commit deferred by 2 MMAs", src, src_floats, out, status);
    run<2, 128, 128>("ring, first probe inline", src, src_floats, out, status);
    return 0;
}
