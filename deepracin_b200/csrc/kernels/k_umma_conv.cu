/*
 * Tensor-core convolution for sm_100a: implicit GEMM on tcgen05.mma (kind::tf32, FP32
 * accumulators in TMEM) with TMA-staged operands.  Evaluates stride-1 1x1 and 3x3
 * convolutions over N-HWC activations with fused bias + ReLU/linear:
 *     D[pixel][o] = sum_{tap, c} X[pixel + tap][c] * Wt[o][tap*Cin + c]
 * i.e. M = output pixels (128 per CTA tile), N = Cout (BN = 64/128/256 per tile),
 * K = taps * Cin walked in slabs of 32 channels (one 128-byte swizzle row) per tap.
 * Replaces, in TF32 mode, the reference's conv2dwinograd2 / conv2d1x1 kernels
 * (Kernels/dR_winograd2.cl:23-254, Kernels/dR_conv2d1x1.cl:4-53).
 *
 * A operand: a 128-pixel tile is S spatial sub-boxes of TW x TH pixels (S*TW*TH = 128); each
 * sub-box of each tap is one 4-D TMA box {32 ch, TW, TH, 1 image} of the input at the tap's
 * shifted coordinates -- the zero padding of the convolution is TMA's out-of-bounds fill.
 * 1x1 convolutions use a flat 2-D map {C, pixels} instead.  B operand: 2-D box {32, BN} of
 * the K-major packed filters.  No multicast, no cluster: every CTA issues its own plain loads.
 *
 * Persistent CTAs (one per SM), 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer and
 * TMEM owner, warps 2-5 = epilogue (TMEM -> registers -> bias/activation -> global).  Two
 * TMEM accumulators so the epilogue of tile i overlaps the main loop of tile i+1; an
 * mbarrier ring of STAGES shared-memory stages between producer and MMA issuer.
 * Every mbarrier wait is bounded (about a second): on expiry the CTA raises an abort flag,
 * reports a code through `status`, drains its in-flight copies, frees its TMEM and returns.
 *
 * Bound: TF32 tensor pipe for K >= ~288 (all VGG layers but the first); algorithmic FLOPs
 * per launch = 2 * taps * Cin * Cout * n * H * W.
 */
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "k_common.cuh"

#define UMMA_THREADS 192
#include "k_umma.cuh"

template <int BN>
struct Cfg {
    static constexpr int B_STAGE_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int STG_PITCH = 36;                            /* floats per staged pixel row: 32 channels + 4 (bank spread, 16-byte aligned) */
    static constexpr int STG_BYTES = 4 * 32 * STG_PITCH * 4;        /* per epilogue warp 32 pixels x 32 channels, transposed for coalesced stores */
    static constexpr int STAGES_RAW = (SMEM_BUDGET - 2048 - STG_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + STG_BYTES;
};

template <int BN>
__global__ void __launch_bounds__(UMMA_THREADS, 1)
k_umma_conv(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const UmmaParams p)
{
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                       /* swizzled tiles need 1024-byte alignment */
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t bars = base + C::STAGES * C::STAGE_BYTES;            /* full[S], empty[S], tfull[2], tempty[2], drain */
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 5));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + 2 + a); };
    const uint32_t drain_bar = bars + 8u * (2 * C::STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles * p.ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        /* ------------------------------------------------ TMA producer (one lane) */
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapA) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapB) : "memory");
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            /* The filters are constants: the first stages' filter tiles are requested before this grid waits for the one
               before it (programmatic dependent launch), so that only the activation loads remain on the critical path.
               Only this thread reads memory the previous kernel writes, and every store of this kernel follows, through the
               barrier chain, from a load issued after the wait. */
            /* K slab -> x coordinate of the A and B maps (three-pass mode: the high halves of both, then A high x B low, then
               A low x B high; the low halves sit x3cat slabs to the right of the high ones) */
            auto a_slab = [&](int ks) { return p.x3cat ? (ks >= 2 * p.x3cat ? ks - p.x3cat : (ks >= p.x3cat ? ks - p.x3cat : ks)) : ks; };
            auto b_slab = [&](int ks) { return p.x3cat ? (ks >= 2 * p.x3cat ? ks - 2 * p.x3cat : ks) : ks; };
            int pre = 0;
            if ((int)blockIdx.x < total_tiles) {
                const int t = blockIdx.x;
                const int ksi = t % p.ksplit, tt = t / p.ksplit;
                const int nt = tt % p.n_tiles;
                const int brow = nt * BN + (p.bgroup_tiles ? ((tt / p.n_tiles) / p.bgroup_tiles) * p.bgroup_rows : 0);
                const int ks0 = ksi * p.kper, ks1 = min(p.kslabs, ks0 + p.kper);
                for (int tap = 0; tap < p.taps && pre < C::STAGES; tap++)
                    for (int ks = ks0; ks < ks1 && pre < C::STAGES; ks++, pre++) {
                        mbar_expect_tx(full_bar(pre), (uint32_t)p.stage_tx);
                        if (p.bpacked) tma_load_2d(base + pre * C::STAGE_BYTES + A_STAGE_BYTES, &mapB, 0, (nt * (p.x3cat ? 2 * p.x3cat : p.kslabs) + b_slab(ks)) * BN, full_bar(pre));
                        else tma_load_2d(base + pre * C::STAGE_BYTES + A_STAGE_BYTES, &mapB, tap * p.CinPad + b_slab(ks) * BK, brow, full_bar(pre));
                    }
            }
            drk_dep_wait();
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int ksi = t % p.ksplit, tt = t / p.ksplit;
                const int mt = tt / p.n_tiles, nt = tt - mt * p.n_tiles;
                const int brow = nt * BN + (p.bgroup_tiles ? (mt / p.bgroup_tiles) * p.bgroup_rows : 0);
                const int ks0 = ksi * p.kper, ks1 = min(p.kslabs, ks0 + p.kper);
                for (int tap = 0; tap < p.taps && ok; tap++) {
                    const int ky = tap / p.kw, kx = tap - ky * p.kw;
                    for (int ks = ks0; ks < ks1; ks++) {
                        const bool armed = issued < pre;            /* this stage's barrier is armed and its filter tile on the way */
                        if (!armed && !mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                        const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                        if (!armed) mbar_expect_tx(full_bar(stage), (uint32_t)p.stage_tx);
                        if (p.S == 0) {
                            tma_load_2d(sa, &mapA, a_slab(ks) * BK, mt * BM, full_bar(stage));
                        } else {
                            const int per = p.tiles_x * p.tiles_y;
                            const int sub_bytes = p.TW * p.TH * BK * 4;
                            for (int q = 0; q < p.S; q++) {
                                const long long sg = (long long)mt * p.S + q;
                                const int img = (int)(sg / per);
                                const int rem = (int)(sg - (long long)img * per);
                                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                                /* images past the end are entirely out of bounds: TMA fills zeros */
                                tma_load_4d(sa + q * sub_bytes, &mapA, ks * BK, txi * p.TW + kx - p.pad, tyi * p.TH + ky - p.pad, img, full_bar(stage));
                            }
                        }
                        if (!armed) {
                            if (p.bpacked) tma_load_2d(sb, &mapB, 0, (nt * (p.x3cat ? 2 * p.x3cat : p.kslabs) + b_slab(ks)) * BN, full_bar(stage));
                            else tma_load_2d(sb, &mapB, tap * p.CinPad + b_slab(ks) * BK, brow, full_bar(stage));
                        }
                        issued++;
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok) {
                /* drain: every armed stage still receives its bytes; wait (bounded) so no copy lands after exit */
                const long long pending = issued < C::STAGES ? issued : C::STAGES;
                int s = stage;
                uint32_t ph = phase;
                for (long long i = 0; i < pending; i++) {
                    if (--s < 0) { s = C::STAGES - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(full_bar(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        /* ------------------------------------------------ MMA issuer (one lane) */
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                const int ksi = t % p.ksplit;
                const int kiters = p.taps * (min(p.kslabs, (ksi + 1) * p.kper) - ksi * p.kper);
                for (int k = 0; k < kiters; k++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sb);
#pragma unroll
                    for (int j = 0; j < BK / 8; j++)    /* one MMA per 8 TF32 (32 bytes) of K inside the swizzle row */
                        umma_tf32(d_tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (k | j) ? 1u : 0u);
                    umma_commit(empty_bar(stage));       /* stage is free once these MMAs have read it */
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else {
        /* ------------------------------------------------ epilogue warps (TMEM lanes 32*(warp%4) ..) */
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;            /* row of the 128-pixel tile this thread owns */
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
            const int ksi = t % p.ksplit, tt = t / p.ksplit;
            const int mt = tt / p.n_tiles, nt = tt - mt * p.n_tiles;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            /* where does this thread's pixel live? */
            bool valid;
            size_t pix;
            if (p.S == 0) {
                const long long m = (long long)mt * BM + row;
                valid = m < p.total_sub;
                pix = (size_t)m;
            } else {
                const int sub = p.TW * p.TH;
                const int q = row / sub, rr = row - q * sub;
                const int dy = rr / p.TW, dx = rr - dy * p.TW;
                const long long sg = (long long)mt * p.S + q;
                const int per = p.tiles_x * p.tiles_y;
                const int img = (int)(sg / per);
                const int rem = (int)(sg - (long long)img * per);
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                const int y = tyi * p.TH + dy, x = txi * p.TW + dx;
                valid = q < p.S && img < p.n && y < p.H && x < p.W;
                if (p.pool) {
                    /* window (x&~1, y&~1): the lane with even x and even y stores; its three partners are lanes ^1, ^TW, ^(TW+1) */
                    valid = valid && !(dx & 1) && !(dy & 1);
                    pix = ((size_t)img * (p.H >> 1) + (y >> 1)) * (p.W >> 1) + (x >> 1);
                } else {
                    pix = ((size_t)img * p.H + y) * p.W + x;
                }
            }
            float *dst = p.out + (size_t)ksi * p.split_stride + pix * p.ldo + p.coff + nt * BN;
            /* Not pooled: a lane holds 32 channels of ONE pixel, so storing from there touches 32 cache lines per instruction.
               Each 32 x 32 chunk goes through a transposing stage in shared memory instead: afterwards lane l stores channels
               4*(l%8).. of pixels i*4 + l/8 (i = 0..7), i.e. an instruction writes four full 128-byte runs. */
            float *rowptr[8];
            uint32_t rowok = 0;
            if (!p.pool) {
                const uint32_t vm = __ballot_sync(0xffffffffu, valid);
                const unsigned long long d64 = (unsigned long long)(uintptr_t)dst;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int src = i * 4 + (lane >> 3);
                    const uint32_t lo32 = __shfl_sync(0xffffffffu, (uint32_t)d64, src), hi32 = __shfl_sync(0xffffffffu, (uint32_t)(d64 >> 32), src);
                    rowptr[i] = reinterpret_cast<float *>((uintptr_t)(((unsigned long long)hi32 << 32) | lo32));
                    rowok |= ((vm >> src) & 1u) << i;
                }
            }
            float *stg = reinterpret_cast<float *>(gen + C::STAGES * C::STAGE_BYTES + 256) + (warp - 2) * 32 * C::STG_PITCH;
            if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                const int col = nt * BN + c0;
                if (!p.pool) {
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4 *>(stg + lane * C::STG_PITCH + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    __syncwarp();
                    const int cl = (lane & 7) * 4;
                    if (col + cl < p.Cout) {
                        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (p.bias) b = __ldg(reinterpret_cast<const float4 *>(p.bias + col + cl));
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            float4 v = *reinterpret_cast<const float4 *>(stg + (i * 4 + (lane >> 3)) * C::STG_PITCH + cl);
                            v.x = drk_act(v.x + b.x, p.act); v.y = drk_act(v.y + b.y, p.act); v.z = drk_act(v.z + b.z, p.act); v.w = drk_act(v.w + b.w, p.act);
                            if ((rowok >> i) & 1u) *reinterpret_cast<float4 *>(rowptr[i] + c0 + cl) = v;
                        }
                    }
                    continue;
                }
                {
                    /* bias and activation are monotone, so max commutes with them: reduce the raw accumulators */
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float v = __uint_as_float(r[j]);
                        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
                        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, p.TW));
                        r[j] = __float_as_uint(v);
                    }
                }
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 v;
                        v.x = __uint_as_float(r[j + 0]); v.y = __uint_as_float(r[j + 1]);
                        v.z = __uint_as_float(r[j + 2]); v.w = __uint_as_float(r[j + 3]);
                        if (p.bias && col + j < p.Cout) {
                            const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + col + j));
                            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                        }
                        v.x = drk_act(v.x, p.act); v.y = drk_act(v.y, p.act); v.z = drk_act(v.z, p.act); v.w = drk_act(v.w, p.act);
                        if (col + j < p.Cout) *reinterpret_cast<float4 *>(dst + c0 + j) = v;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }

    /* teardown: every role leaves its loop (normally or on abort) and meets here */
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

/*
 * Halo variant for 3x3 layers whose image tiles exactly into 14 x 8 pixel blocks (224, 112, 56 ...).
 *
 * The plain kernel above re-stages the A tile for each of the nine taps, and the SM's shared-memory
 * port (TMA writes + MMA operand reads, 128 B/clk) is what bounds it.  Here the (14+2) x (8+2) haloed
 * input block of a 32-channel slab is staged ONCE (one TMA box, 160 rows of 128 B, pitch 16 pixels)
 * and all nine taps read it: output pixel (ty, tx) of the block is MMA row m = ty*16 + tx, and tap
 * (ky, kx) reads shared-memory rows m + ky*16 + kx -- a contiguous 128-row window of the same buffer,
 * addressed by moving the matrix descriptor's start address by (ky*16 + kx) rows.  Rows with
 * tx >= 14 are idle (12.5 % of the tensor pipe), A traffic into shared memory drops 7.2x.
 * B tiles stream through their own ring, nine per A slab.
 */
#define HALO_TW 14
#define HALO_TH 8
#define HALO_P 16
#define HALO_ROWS ((HALO_TH + 2) * HALO_P)             /* 160 rows loaded per slab */
#define HALO_A_BYTES (HALO_ROWS * BK * 4)              /* 20480 */
#define HALO_A_SLOT (21 * 1024)                        /* 168 rows: taps of the two idle tail rows read up to row 161 */

template <int BN>
struct HaloCfg {
    static constexpr int B_STAGE_BYTES = BN * BK * 4;
    /* transposing store stage as in Cfg<BN>; with BN = 256 the shared memory for it comes from the third activation slot
       (two suffice: a slot is consumed over nine taps = ~4600 clocks, far longer than a 20 KB load takes) */
    static constexpr int NA = BN <= 128 ? 3 : 2;
    static constexpr int STG_PITCH = 36;
    static constexpr int STG_BYTES = 4 * 32 * STG_PITCH * 4;
    static constexpr int NB_RAW = (SMEM_BUDGET - 2048 - NA * HALO_A_SLOT - STG_BYTES) / B_STAGE_BYTES;
    static constexpr int NB = NB_RAW > 10 ? 10 : NB_RAW;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int SMEM_BYTES = NA * HALO_A_SLOT + NB * B_STAGE_BYTES + 1024 + 512 + STG_BYTES;
};

template <int BN>
__global__ void __launch_bounds__(UMMA_THREADS, 1)
k_umma_conv_halo(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const UmmaParams p)
{
    using C = HaloCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t a_base = base, b_base = base + C::NA * HALO_A_SLOT;
    const uint32_t bars = b_base + C::NB * C::B_STAGE_BYTES;
    constexpr int NBARS = 2 * C::NA + 2 * C::NB + 5;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + C::NA * HALO_A_SLOT + C::NB * C::B_STAGE_BYTES + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto afull = [&](int s) { return bars + 8u * s; };
    auto aempty = [&](int s) { return bars + 8u * (C::NA + s); };
    auto bfull = [&](int s) { return bars + 8u * (2 * C::NA + s); };
    auto bempty = [&](int s) { return bars + 8u * (2 * C::NA + C::NB + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::NA + 2 * C::NB + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::NA + 2 * C::NB + 2 + a); };
    const uint32_t drain_bar = bars + 8u * (2 * C::NA + 2 * C::NB + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int per = p.tiles_x * p.tiles_y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NA; s++) { mbar_init(afull(s), 1); mbar_init(aempty(s), 1); }
        for (int s = 0; s < C::NB; s++) { mbar_init(bfull(s), 1); mbar_init(bempty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    drk_dep_wait();                 /* set-up above overlaps the previous kernel; its outputs are visible from here on */

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapA) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapB) : "memory");
            int as = 0, bs = 0;
            uint32_t aph = 0, bph = 0;
            long long a_issued = 0, b_issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int mt = t / p.n_tiles, nt = t - mt * p.n_tiles;
                const int img = mt / per, rem = mt - img * per;
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    if (!mbar_wait(aempty(as), aph ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
                    mbar_expect_tx(afull(as), HALO_A_BYTES);
                    tma_load_4d(a_base + as * HALO_A_SLOT, &mapA, ks * BK, txi * HALO_TW - 1, tyi * HALO_TH - 1, img, afull(as));
                    a_issued++;
                    if (++as == C::NA) { as = 0; aph ^= 1u; }
                    for (int tap = 0; tap < 9; tap++) {
                        if (!mbar_wait(bempty(bs), bph ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                        mbar_expect_tx(bfull(bs), C::B_STAGE_BYTES);
                        tma_load_2d(b_base + bs * C::B_STAGE_BYTES, &mapB, tap * p.CinPad + ks * BK, nt * BN, bfull(bs));
                        b_issued++;
                        if (++bs == C::NB) { bs = 0; bph ^= 1u; }
                    }
                }
            }
            if (!ok) {      /* drain what is still in flight (bounded) before the CTA's shared memory is released */
                long long pend = a_issued < C::NA ? a_issued : C::NA;
                int s = as; uint32_t ph = aph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = C::NA - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(afull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
                pend = b_issued < C::NB ? b_issued : C::NB;
                s = bs; ph = bph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = C::NB - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(bfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            int as = 0, bs = 0;
            uint32_t aph = 0, bph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    if (!mbar_wait(afull(as), aph, abort_flag, p.status, 6)) { ok = false; break; }
                    const uint32_t sa = a_base + as * HALO_A_SLOT;
                    for (int tap = 0; tap < 9; tap++) {
                        if (!mbar_wait(bfull(bs), bph, abort_flag, p.status, 3)) { ok = false; break; }
                        tc_fence_after();
                        const int ky = tap / 3, kx = tap - ky * 3;
                        const uint64_t adesc = make_smem_desc(sa + (uint32_t)((ky * HALO_P + kx) * BK * 4));
                        const uint64_t bdesc = make_smem_desc(b_base + bs * C::B_STAGE_BYTES);
#pragma unroll
                        for (int j = 0; j < BK / 8; j++)
                            umma_tf32(d_tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (ks | tap | j) ? 1u : 0u);
                        umma_commit(bempty(bs));
                        if (++bs == C::NB) { bs = 0; bph ^= 1u; }
                    }
                    if (ok) umma_commit(aempty(as));
                    if (++as == C::NA) { as = 0; aph ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int dy = row / HALO_P, dx = row - dy * HALO_P;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
            const int mt = t / p.n_tiles, nt = t - mt * p.n_tiles;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int img = mt / per, rem = mt - img * per;
            const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
            const int y = tyi * HALO_TH + dy, x = txi * HALO_TW + dx;
            bool valid = dx < HALO_TW && dy < HALO_TH && y < p.H && x < p.W;
            size_t pix;
            if (p.pool) {
                valid = valid && !(dx & 1) && !(dy & 1);
                pix = ((size_t)img * (p.H >> 1) + (y >> 1)) * (p.W >> 1) + (x >> 1);
            } else {
                pix = ((size_t)img * p.H + y) * p.W + x;
            }
            float *dst = p.out + pix * p.ldo + p.coff + nt * BN;
            /* not pooled, BN <= 128: stores go through the transposing stage (see k_umma_conv) */
            const bool staged = C::STG_BYTES > 0 && !p.pool;
            float *rowptr[8];
            uint32_t rowok = 0;
            if (staged) {
                const uint32_t vm = __ballot_sync(0xffffffffu, valid);
                const unsigned long long d64 = (unsigned long long)(uintptr_t)dst;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int src = i * 4 + (lane >> 3);
                    const uint32_t lo32 = __shfl_sync(0xffffffffu, (uint32_t)d64, src), hi32 = __shfl_sync(0xffffffffu, (uint32_t)(d64 >> 32), src);
                    rowptr[i] = reinterpret_cast<float *>((uintptr_t)(((unsigned long long)hi32 << 32) | lo32));
                    rowok |= ((vm >> src) & 1u) << i;
                }
            }
            float *stg = reinterpret_cast<float *>(gen + C::NA * HALO_A_SLOT + C::NB * C::B_STAGE_BYTES + 512) + (warp - 2) * 32 * C::STG_PITCH;
            if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                const int col = nt * BN + c0;
                if (staged) {
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4 *>(stg + lane * C::STG_PITCH + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    __syncwarp();
                    const int cl = (lane & 7) * 4;
                    if (col + cl < p.Cout) {
                        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (p.bias) b = __ldg(reinterpret_cast<const float4 *>(p.bias + col + cl));
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            float4 v = *reinterpret_cast<const float4 *>(stg + (i * 4 + (lane >> 3)) * C::STG_PITCH + cl);
                            v.x = drk_act(v.x + b.x, p.act); v.y = drk_act(v.y + b.y, p.act); v.z = drk_act(v.z + b.z, p.act); v.w = drk_act(v.w + b.w, p.act);
                            if ((rowok >> i) & 1u) *reinterpret_cast<float4 *>(rowptr[i] + c0 + cl) = v;
                        }
                    }
                    continue;
                }
                if (p.pool) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float v = __uint_as_float(r[j]);
                        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
                        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, HALO_P));
                        r[j] = __float_as_uint(v);
                    }
                }
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 v;
                        v.x = __uint_as_float(r[j + 0]); v.y = __uint_as_float(r[j + 1]);
                        v.z = __uint_as_float(r[j + 2]); v.w = __uint_as_float(r[j + 3]);
                        if (p.bias && col + j < p.Cout) {
                            const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + col + j));
                            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                        }
                        v.x = drk_act(v.x, p.act); v.y = drk_act(v.y, p.act); v.z = drk_act(v.z, p.act); v.w = drk_act(v.w, p.act);
                        if (col + j < p.Cout) *reinterpret_cast<float4 *>(dst + c0 + j) = v;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

/*
 * Transposed halo variant for layers with few output channels (Cout <= 128).
 *
 * A tcgen05.mma (kind::tf32, M = 128) occupies the tensor pipe for 128 clocks at N = 256, 64 at N = 128 and never
 * less than ~45 (N <= 64), and the single issuing thread has to get through its barrier probe, descriptors and
 * commit once per group of four instructions whatever N is: the fewer and wider the instructions, the closer the
 * kernel runs to the pipe's rate (before the issuer's barrier probe was inlined, issue cost alone made every
 * instruction take ~166 clocks for N = 64, 128 and 256 alike).  With pixels on M and output channels on N a 64-channel
 * layer issues four times the instructions of a 256-wide one for the same work.  This variant computes the
 * transposed product instead: M = output channels (the filter tile, rows past Cout are TMA zero fill),
 * N = 256 pixels -- a 14 x 16 pixel block read from its haloed (14+2) x (16+2) input block exactly
 * as in the halo kernel above, now through the B descriptor.  The accumulator is [channel][pixel]:
 * each epilogue lane owns one channel, a warp stores 32 consecutive channels of one pixel per
 * instruction, and the fused 2x2 max pooling is a maximum over four registers of the same lane.
 */
#define SWAP_N 256                                     /* most MMA columns per tile; a tile is TH block rows of P pixels, P * TH <= 256 */
#define SWAP_HALO_SLOT (38 * 1024)                     /* (TH + 2) * P <= 288 rows loaded; taps of idle columns read a few rows further */
#define SWAP_NH 2
#define SWAP_W_BYTES (BM * BK * 4)                     /* filter stage: 128 rows x 128 B */
#define SWAP_NW 9
#define SWAP_NW_X3 6                                   /* X3 mode: 2 blocks + the lo(x) buffer + 6 filter stages = 210 KB */
#define SWAP_EPI_WARPS 8
#define SWAP_SPLIT_WARPS 4                             /* X3 mode only */
#define SWAP_THREADS(X3) ((2 + SWAP_EPI_WARPS + ((X3) ? SWAP_SPLIT_WARPS : 0)) * 32)
#define SWAP_SMEM (SWAP_NH * SWAP_HALO_SLOT + SWAP_NW * SWAP_W_BYTES + 1024 + 512)

/*
 * X3 = true: FP32-accurate evaluation on the tensor cores ("3xTF32").  A kind::tf32 MMA reads only the upper 19 bits of
 * each FP32 operand (sign, exponent, 10 mantissa bits): x = hi(x) + lo(x) with hi(x) = x with its low 13 mantissa bits
 * cleared.  The product x*w is then evaluated as hi(x)*hi(w) + hi(x)*lo(w) + lo(x)*hi(w) in three passes over the nine
 * taps into the same FP32 accumulator; the dropped lo*lo term and the truncation of the lo parts are below 2^-21 of
 * the product, so a layer stays inside the exact-FP32 kernels' 1e-4 bound at three times the direct TF32 kernel's MMA count
 * instead of the FFMA rate.  The tensor maps are plain FLOAT32 here (no rounding by TMA): passes 0 and 1 read the haloed
 * block as loaded (the MMA ignores the low bits = hi(x)) against the filters W and a precomputed lo(W) tensor (mapWlo);
 * meanwhile four extra warps write lo(x) = x - hi(x) -- exact in FP32 -- into a buffer of its own, which pass 2 multiplies with W.
 */
template <bool X3>
__global__ void __launch_bounds__(SWAP_THREADS(X3), 1)
k_umma_conv_swap(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapWlo,
                 const UmmaParams p)
{
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    /* X3: one more block-sized buffer holds lo(x) of the slab in work, the filter ring is shorter to make room for it */
    constexpr int NW = X3 ? SWAP_NW_X3 : SWAP_NW;
    constexpr int XLO_BYTES = X3 ? SWAP_HALO_SLOT : 0;
    const uint32_t h_base = base, xlo_base = base + SWAP_NH * SWAP_HALO_SLOT, w_base = xlo_base + XLO_BYTES;
    const uint32_t bars = w_base + NW * SWAP_W_BYTES;
    constexpr int NBARS = 2 * SWAP_NH + 2 * NW + 7;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + SWAP_NH * SWAP_HALO_SLOT + XLO_BYTES + NW * SWAP_W_BYTES + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto hfull = [&](int s) { return bars + 8u * s; };
    auto hempty = [&](int s) { return bars + 8u * (SWAP_NH + s); };
    auto wfull = [&](int s) { return bars + 8u * (2 * SWAP_NH + s); };
    auto wempty = [&](int s) { return bars + 8u * (2 * SWAP_NH + NW + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * SWAP_NH + 2 * NW + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * SWAP_NH + 2 * NW + 2 + a); };
    const uint32_t drain_bar = bars + 8u * (2 * SWAP_NH + 2 * NW + 4);
    const uint32_t xlo_full = bars + 8u * (2 * SWAP_NH + 2 * NW + 5);          /* X3: the lo(x) buffer holds the current slab's low parts */
    const uint32_t xlo_free = bars + 8u * (2 * SWAP_NH + 2 * NW + 6);          /* X3: pass 2 of the previous slab has read it */
    constexpr int PASSES = X3 ? 3 : 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int per = p.tiles_x * p.tiles_y;
    constexpr int TMEM_COLS = 2 * SWAP_N;
    const uint32_t halo_bytes = (uint32_t)((p.TH + 2) * p.P * BK * 4);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SWAP_NH; s++) { mbar_init(hfull(s), 1); mbar_init(hempty(s), 1); }
        for (int s = 0; s < NW; s++) { mbar_init(wfull(s), 1); mbar_init(wempty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), SWAP_EPI_WARPS); }
        mbar_init(xlo_full, SWAP_SPLIT_WARPS);
        mbar_init(xlo_free, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    drk_dep_wait();                 /* set-up above overlaps the previous kernel; its outputs are visible from here on */

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapX) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapW) : "memory");
            if (X3) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapWlo) : "memory");
            int hs = 0, ws = 0;
            uint32_t hph = 0, wph = 0;
            long long h_issued = 0, w_issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int mt = t / p.n_tiles, nt = t - mt * p.n_tiles;
                const int img = mt / per, rem = mt - img * per;
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    if (!mbar_wait(hempty(hs), hph ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
                    mbar_expect_tx(hfull(hs), halo_bytes);
                    tma_load_4d(h_base + hs * SWAP_HALO_SLOT, &mapX, ks * BK, txi * p.TW - 1, tyi * p.TH - 1, img, hfull(hs));
                    h_issued++;
                    if (++hs == SWAP_NH) { hs = 0; hph ^= 1u; }
                    for (int pt = 0; pt < 9 * PASSES; pt++) {                   /* X3: filters, their low parts, filters again */
                        const int tap = pt % 9;
                        if (!mbar_wait(wempty(ws), wph ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                        mbar_expect_tx(wfull(ws), SWAP_W_BYTES);
                        tma_load_2d(w_base + ws * SWAP_W_BYTES, (X3 && pt / 9 == 1) ? &mapWlo : &mapW, tap * p.CinPad + ks * BK, nt * BM, wfull(ws));
                        w_issued++;
                        if (++ws == NW) { ws = 0; wph ^= 1u; }
                    }
                }
            }
            if (!ok) {
                long long pend = h_issued < SWAP_NH ? h_issued : SWAP_NH;
                int s = hs; uint32_t ph = hph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = SWAP_NH - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(hfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
                pend = w_issued < NW ? w_issued : NW;
                s = ws; ph = wph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = NW - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(wfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(p.ncols);
            int hs = 0, ws = 0;
            uint32_t hph = 0, wph = 0;
            int it = 0;
            uint32_t xph = 0;                        /* X3: parity of the lo(x) buffer's current use */
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * SWAP_N);
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    if (!mbar_wait(hfull(hs), hph, abort_flag, p.status, 6)) { ok = false; break; }
                    uint32_t sh = h_base + hs * SWAP_HALO_SLOT;
                    for (int pt = 0; pt < 9 * PASSES; pt++) {
                        const int tap = pt % 9;
                        if (X3 && pt == 18) {
                            /* passes 0 and 1 (block as loaded) are issued; pass 2 reads lo(x), which the splitter warps wrote to their
                               own buffer while those passes ran.  The block's slot is free once passes 0 and 1 have completed. */
                            if (!mbar_wait(xlo_full, xph, abort_flag, p.status, 12)) { ok = false; break; }
                            umma_commit(hempty(hs));
                            sh = xlo_base;
                        }
                        if (!mbar_wait(wfull(ws), wph, abort_flag, p.status, 3)) { ok = false; break; }
                        tc_fence_after();
                        const int ky = tap / 3, kx = tap - ky * 3;
                        const uint64_t adesc = make_smem_desc(w_base + ws * SWAP_W_BYTES);
                        const uint64_t bdesc = make_smem_desc(sh + (uint32_t)((ky * p.P + kx) * BK * 4));
#pragma unroll
                        for (int j = 0; j < BK / 8; j++)
                            umma_tf32(d_tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (ks | pt | j) ? 1u : 0u);
                        umma_commit(wempty(ws));
                        if (++ws == NW) { ws = 0; wph ^= 1u; }
                    }
                    if (X3) { if (ok) umma_commit(xlo_free); xph ^= 1u; }
                    else if (ok) umma_commit(hempty(hs));
                    if (++hs == SWAP_NH) { hs = 0; hph ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else if (warp < 2 + SWAP_EPI_WARPS) {
        /* eight epilogue warps: two per 32-lane quarter of TMEM, each taking half of the 256 pixel columns (with four, the
           224 scalar stores per lane and tile of a layer without pooling outlasted the 72 MMAs of a 64-channel-deep tile) */
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
            const int mt = t / p.n_tiles, nt = t - mt * p.n_tiles;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int img = mt / per, rem = mt - img * per;
            const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
            const int ch = nt * BM + quarter * 32 + lane;        /* the output channel this lane owns */
            const bool chok = ch < p.Cout;
            const float bv = (p.bias && chok) ? __ldg(p.bias + ch) : 0.0f;
            /* ReLU = clamp to [0, FLT_MAX]; linear = clamp to [-inf, +inf] (a no-op): same two instructions either way */
            const float lo = p.act ? 0.0f : -INFINITY, hi = p.act ? FLT_MAX : INFINITY;
            float *obase = p.out + p.coff + ch;
            if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * SWAP_N);
            if (p.P != 16) {
                /* 30- or 32-pixel pitch: a block row is one 32-column TMEM load starting at column row * P (the last P - TW columns
                   of it are idle, a load at pitch 30 also fetches two columns of the next row that are not used); the two warps of a
                   quarter take alternate rows, or row pairs when the 2x2 pool is fused.  The TMEM loads are warp-wide instructions:
                   every lane executes them, lanes past Cout only skip the stores. */
                const int x0 = txi * p.TW;
                if (p.pool) {
                    for (int u = half; u < (p.TH >> 1); u += 2) {
                        uint32_t r0[32], r1[32];
                        tmem_ld32(taddr + (uint32_t)(2 * u * p.P), r0);
                        tmem_ld32(taddr + (uint32_t)((2 * u + 1) * p.P), r1);
                        const int yo = ((tyi * p.TH) >> 1) + u;
                        if (yo >= (p.H >> 1)) break;
                        if (!chok) continue;
                        float *orow = obase + (((size_t)img * (p.H >> 1) + yo) * (size_t)(p.W >> 1) + (x0 >> 1)) * p.ldo;
                        const int nx = min(p.TW >> 1, (p.W >> 1) - (x0 >> 1));
#pragma unroll
                        for (int px = 0; px < 15; px++) {
                            const float v = fmaxf(fmaxf(__uint_as_float(r0[2 * px]), __uint_as_float(r0[2 * px + 1])),
                                                  fmaxf(__uint_as_float(r1[2 * px]), __uint_as_float(r1[2 * px + 1])));
                            if (px < nx) *orow = fminf(fmaxf(v + bv, lo), hi);
                            orow += p.ldo;
                        }
                    }
                } else {
                    for (int u = half; u < p.TH; u += 2) {
                        uint32_t r[32];
                        tmem_ld32(taddr + (uint32_t)(u * p.P), r);
                        const int y = tyi * p.TH + u;
                        if (y >= p.H) break;
                        if (!chok) continue;
                        float *optr = obase + (((size_t)img * p.H + y) * p.W + x0) * (size_t)p.ldo;
                        const int nx = min(p.TW, p.W - x0);
#pragma unroll
                        for (int dx = 0; dx < 30; dx++) {
                            if (dx < nx) *optr = fminf(fmaxf(__uint_as_float(r[dx]) + bv, lo), hi);
                            optr += p.ldo;
                        }
                    }
                }
            } else
            for (int c0 = half * 32; c0 < p.ncols; c0 += 64) {           /* the two warps of a quarter take alternate 32-column chunks */
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                if (!chok) continue;
                const int x0 = txi * p.TW;
                const int y0 = tyi * p.TH + (c0 >> 4);             /* 16-pixel pitch: this chunk holds block rows y0 and y0 + 1 */
                if (p.pool) {
                    const int yo = y0 >> 1;
                    if (yo < (p.H >> 1)) {
                        float *orow = obase + ((size_t)img * (p.H >> 1) + yo) * (size_t)(p.W >> 1) * p.ldo;
#pragma unroll
                        for (int px = 0; px < HALO_TW / 2; px++) {
                            const int xo = (x0 >> 1) + px;
                            float v = fmaxf(fmaxf(__uint_as_float(r[2 * px]), __uint_as_float(r[2 * px + 1])),
                                            fmaxf(__uint_as_float(r[16 + 2 * px]), __uint_as_float(r[16 + 2 * px + 1])));
                            if (xo < (p.W >> 1)) orow[(size_t)xo * p.ldo] = fminf(fmaxf(v + bv, lo), hi);
                        }
                    }
                } else {
#pragma unroll
                    for (int dy = 0; dy < 2; dy++) {
                        const int y = y0 + dy;
                        if (y >= p.H) break;
                        float *optr = obase + (((size_t)img * p.H + y) * p.W + x0) * (size_t)p.ldo;
                        const int nx = min(HALO_TW, p.W - x0);
#pragma unroll
                        for (int dx = 0; dx < HALO_TW; dx++) {
                            if (dx < nx) *optr = fminf(fmaxf(__uint_as_float(r[dy * 16 + dx]) + bv, lo), hi);
                            optr += p.ldo;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    } else if (X3) {
        /* splitter warps: lo(block) of every channel slab into the lo(x) buffer, while passes 0 and 1 of that slab run */
        const int sw = warp - (2 + SWAP_EPI_WARPS);
        int hs = 0;
        uint32_t hph = 0, xph = 0;
        bool ok = true;
        const int chunks = (int)(halo_bytes / 16);
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            for (int ks = 0; ks < p.kslabs; ks++) {
                /* the block was written by TMA: wait on its barrier (visibility); the buffer is free once pass 2 of the slab before
                   has read it (first use: the wait on the preceding phase returns at once) */
                if (!mbar_wait_warp(hfull(hs), hph, abort_flag, p.status, 10)) { ok = false; break; }
                if (!mbar_wait_warp(xlo_free, xph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                const uint4 *blk = reinterpret_cast<const uint4 *>(gen + hs * SWAP_HALO_SLOT);
                uint4 *lo = reinterpret_cast<uint4 *>(gen + SWAP_NH * SWAP_HALO_SLOT);
                for (int i = sw * 32 + lane; i < chunks; i += SWAP_SPLIT_WARPS * 32) {
                    uint4 v = blk[i];
                    v.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
                    v.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
                    v.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
                    v.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
                    lo[i] = v;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(xlo_full);
                xph ^= 1u;
                if (++hs == SWAP_NH) { hs = 0; hph ^= 1u; }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

/* ------------------------------------------------------------------------- host side */
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode()
{
    static PFN_encodeTiled fn = NULL;
    if (!fn) {
        void *p = NULL;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (PFN_encodeTiled)p;
    }
    return fn;
}

#define DRK_MAX_DEVICES 64
static int current_device()
{
    int dev = 0;
    cudaGetDevice(&dev);
    return dev >= 0 && dev < DRK_MAX_DEVICES ? dev : 0;
}

struct dRk_TensorConvPlan {
    CUtensorMap mapA, mapB;
    UmmaParams p;
    int BN;
    int grid;
    int halo;           /* 1: k_umma_conv_halo (one haloed A tile per channel slab, reused by all nine taps) */
    int swap;           /* 1: k_umma_conv_swap (channels on M, 256 pixels on N) for Cout <= 128 */
    int first;          /* 1: k_umma_conv_first (Cin <= 4: patches gathered by producer warps, no tensor maps) */
    int pair;           /* 1: k_umma_conv_pair (Cout <= 64: two output rows stacked on M); mapA = odd input rows, mapA2 = even */
    int x3;             /* 1: FP32-accurate three-pass evaluation: k_umma_conv_swap<true> (mapA2 = the filters' low parts) or, with pair,
                           k_umma_conv_pair<true> (mapB2 = the filters' low parts) */
    CUtensorMap mapA2, mapB2;
    const float *in, *wT;
    int sms;
    int ldi;            /* first-layer kernel: pixel stride of `in` and the optional affine channel map of its gather */
    int mapped, map_ch[4];
    float map_scale[4], map_shift[4];
};

double drk_umma_pair_fill(int W, int H);
double drk_umma_pair_geometry(int W, int H, int *P, int *TW, int *TJ);
int drk_umma_pair_launch(cudaStream_t st, const CUtensorMap *mapO, const CUtensorMap *mapE, const CUtensorMap *mapW, const CUtensorMap *mapWlo,
                         const UmmaParams *p, int grid, int x3);
int drk_umma_first_supported(int Cin, int Cout, int kw, int kh);
int drk_umma_first_can_pool(int W, int H, int Cin, int Cout);
int drk_umma_first_launch(cudaStream_t st, const float *in, const float *wT, const float *bias, float *out, int n, int W, int H, int Cin,
                          int Cout, int act, int ldi, int ldo, int coff, int pool, int *status, int sms, const int *map_ch, const float *map_scale,
                          const float *map_shift);

/*
 * Sub-box geometry of a CTA's pixel tile for a W x H image: S boxes of TW x TH pixels, TW*TH a multiple
 * of 8 (each box must start on a swizzle-atom boundary), S*TW*TH <= 128.  When the boxes do not fill
 * all 128 rows the remaining rows of the MMA tile are never loaded nor stored (idle tensor-pipe rows);
 * that is cheaper than covering a 28- or 14-pixel-wide image with many 4-pixel-wide boxes, whose short
 * contiguous runs make the TMA loads slow.
 */
static void pick_subtile(int W, int H, int pool, int *TW, int *TH, int *S)
{
    double best = 1e30;
    int widths[8] = {32, 16, 8, 4, 2, 1, 0, 0};
    int nw = 6;
    if (W <= 128 && W != 32 && W != 16 && W != 8 && W != 4) widths[nw++] = W;
    for (int wi = 0; wi < nw; wi++) {
        const int tw = widths[wi];
        /* fused 2x2 pooling exchanges partners by warp shuffles: box width a power of two <= 16, even height */
        if (pool && (tw > 16 || tw < 2 || (tw & (tw - 1)))) continue;
        for (int th = 1; th <= BM; th++) {
            if (pool && (th & 1)) continue;
            const int rows = tw * th;
            if (rows > BM) break;
            if (rows % 8) continue;
            if (pool && (32 % tw || ((32 / tw) & 1))) continue;
            for (int s = 1; s * rows <= BM && s <= (pool ? 1 : 8); s++) {
                const double cover = (double)((W + tw - 1) / tw * tw) * ((H + th - 1) / th * th) / ((double)W * H);
                const double idle = (double)BM / (s * rows);
                double cost = cover * idle * (1.0 + 0.3 * (s - 1));   /* every extra box is one more TMA instruction per stage: measured 27% slower with two */
                if (rows < 32) cost *= 2.0;                   /* tiny boxes: the fixed cost dominates */
                if (cost < best) { best = cost; *TW = tw; *TH = th; *S = s; }
            }
        }
    }
}

/* K pitch of one tap in the packed filters: whole 32-channel slabs, except for the few-channel first-layer kernel, which packs K densely */
extern "C" int dRk_tensor_conv_cin_pad(int Cin) { return Cin <= 4 ? Cin : (Cin + BK - 1) / BK * BK; }

extern "C" int dRk_tensor_conv_supported(int W, int H, int Cin, int Cout, int kw, int kh)
{
    if (W <= 0 || H <= 0) return 0;
    if (!((kw == 1 && kh == 1) || (kw == 3 && kh == 3))) return 0;
    if (drk_umma_first_supported(Cin, Cout, kw, kh)) return 1;
    /* channels past Cin inside the last 32-channel slab are TMA zero fill (activations) and zero padding (packed filters);
       TMA needs the pixel stride Cin*4 to be a multiple of 16 bytes */
    if (Cin % 4 != 0 || Cin < 8) return 0;
    if (Cout % 4 != 0 || Cout < 16) return 0;          /* rows past Cout are TMA zero fill; the epilogues mask them */
    return 1;
}

/* fraction of the halo kernel's MMA rows that produce output pixels for a W x H image (14 x 8 blocks, 16-pixel pitch) */
static double halo_fill(int W, int H)
{
    const double tx = (W + HALO_TW - 1) / HALO_TW, ty = (H + HALO_TH - 1) / HALO_TH;
    return (double)W * H / (tx * ty * BM);
}

/* Geometry of the transposed variant: block rows of P = 16 (14 valid), 30 (28 valid) or 32 (up to 30 valid) pixels, TH of
 * them per tile, N = P * TH <= 256 MMA columns (the operand is a window of consecutive shared-memory rows, so any pitch
 * works).  Picks the one with the largest share of columns that are output pixels; fused pooling needs an even TH.
 * Returns that share. */
static double swap_geometry(int W, int H, int pool, int *P, int *TW, int *TH)
{
    double best = -1.0;
    const int pitches[3] = {16, 30, 32};
    for (int pi = 0; pi < 3; pi++) {
        const int pitch = pitches[pi];
        const int tw = pitch == 16 ? HALO_TW : pitch == 30 ? 28 : (W < 30 ? (W & ~1) : 30);
        if (tw < 2) continue;
        for (int th = SWAP_N / pitch; th >= 4; th--) {
            const int ncols = pitch * th;
            if (ncols % 16) continue;                                    /* N of the MMA */
            if (pitch == 16 && ncols % 32) continue;                     /* 16-pixel pitch: whole 32-column epilogue chunks */
            if (pool && (th & 1)) continue;
            if (ncols + 2 * pitch + 2 > 304) continue;                   /* the taps of the last columns must stay inside the shared-memory slot */
            const double tx = (W + tw - 1) / tw, ty = (H + th - 1) / th;
            const double fill = (double)W * H / (tx * ty * ncols) - (ncols < 192 ? 0.15 : 0.0);   /* narrow instructions issue badly */
            if (fill > best + 1e-9) { best = fill; *P = pitch; *TW = tw; *TH = th; }
        }
    }
    return best;
}
static double swap_fill(int W, int H)
{
    int P, TW, TH;
    return swap_geometry(W, H, 1, &P, &TW, &TH);
}

/* the geometry and the tile count of a launch of n images */
static double swap_geometry_for(int n, int W, int H, int Cout, int pool, int sms, int *P, int *TW, int *TH, long long *tiles)
{
    (void)sms;
    const double fill = swap_geometry(W, H, pool, P, TW, TH);
    *tiles = fill > 0.0 ? (long long)n * ((W + *TW - 1) / *TW) * ((H + *TH - 1) / *TH) * ((Cout + BM - 1) / BM) : 0;
    return fill;
}

/* which kernel evaluates a layer shape; the packed-filter layout depends on it, so packing and planning both ask here.
 * The debug switches (dRk_debug_switches) exist for A/B comparisons of the variants when profiling. */
enum { VAR_NONE = 0, VAR_FLAT, VAR_PLAIN, VAR_HALO, VAR_SWAP, VAR_PAIR, VAR_FIRST };
static int pick_variant(int W, int H, int Cin, int Cout, int kw, int kh)
{
    if (!dRk_tensor_conv_supported(W, H, Cin, Cout, kw, kh)) return VAR_NONE;
    if (drk_umma_first_supported(Cin, Cout, kw, kh)) return VAR_FIRST;
    if (kw == 1) return VAR_FLAT;
    const drk_DebugSwitches *sw = dRk_debug_switches();
    const bool no_halo = sw->no_halo;
    if (Cout <= 64 && H >= 2 && drk_umma_pair_fill(W, H) >= 0.5 && !sw->no_pair && !no_halo) return VAR_PAIR;
    if (Cout <= BM && swap_fill(W, H) >= 0.8 && !sw->no_swap && !no_halo) return VAR_SWAP;
    /* halo or transposed kernel: which of the two is settled per plan, when the batch is known (use_swap_kernel) */
    if ((halo_fill(W, H) >= 0.55 || swap_fill(W, H) >= 0.55) && !no_halo) return VAR_HALO;
    return VAR_PLAIN;
}

/* pool_type: 0 none, 1 max 2x2/2, 2 average 2x2/2 */
extern "C" int dRk_tensor_conv_can_fuse_pool(int W, int H, int Cin, int Cout, int kw, int kh, int pool_type)
{
    if (pool_type == 0) return 1;
    const int v = pick_variant(W, H, Cin, Cout, kw, kh);
    if (v == VAR_NONE || v == VAR_FLAT || kw != 3 || (W & 1) || (H & 1)) return 0;
    if (v == VAR_FIRST) return (pool_type == 1 || pool_type == 2) && drk_umma_first_can_pool(W, H, Cin, Cout);
    return pool_type == 1;
}

extern "C" size_t dRk_tensor_conv_packed_floats(int W, int H, int Cin, int Cout, int kw, int kh)
{
    const int v = pick_variant(W, H, Cin, Cout, kw, kh);
    if (v == VAR_NONE) return 0;
    const size_t cp = (size_t)dRk_tensor_conv_cin_pad(Cin);
    if (v == VAR_PAIR) return (size_t)BM * 12 * cp;
    return (size_t)Cout * kw * kh * cp;
}

extern "C" int dRk_tensor_conv_pack_weights(const float *w, float *dst, int W, int H, int Cin, int Cout, int kw, int kh)
{
    const int v = pick_variant(W, H, Cin, Cout, kw, kh);
    if (v == VAR_NONE) return -1;
    const size_t cp = (size_t)dRk_tensor_conv_cin_pad(Cin);
    const int taps = kw * kh;
    memset(dst, 0, dRk_tensor_conv_packed_floats(W, H, Cin, Cout, kw, kh) * sizeof(float));
    if (v == VAR_PAIR) {
        /* [128 rows][(i*3 + kx)*CinPad + c]: row r < 64 = channel r with ky = i (upper output row), row 64 + o = channel o with
           ky = i - 1 (lower output row); i = 0..3 counts the four input rows a pair of output rows reads */
        for (int r = 0; r < BM; r++) {
            const int o = r & 63, lower = r >> 6;
            if (o >= Cout) continue;
            for (int i = 0; i < 4; i++) {
                const int ky = i - lower;
                if (ky < 0 || ky > 2) continue;
                for (int kx = 0; kx < 3; kx++)
                    for (int c = 0; c < Cin; c++)
                        dst[(size_t)r * 12 * cp + (size_t)(i * 3 + kx) * cp + c] = w[((size_t)c * Cout + o) * 9 + ky * 3 + kx];
            }
        }
        return 0;
    }
    /* [o][(ky*kw + kx)*CinPad + c], channels Cin..CinPad-1 stay zero */
    for (int c = 0; c < Cin; c++)
        for (int o = 0; o < Cout; o++)
            for (int t = 0; t < taps; t++)
                dst[(size_t)o * taps * cp + (size_t)t * cp + c] = w[((size_t)c * Cout + o) * taps + t];
    return 0;
}

/* Transposed or halo kernel for a 3x3 layer (their packed filters are the same, so this is decided per plan, with the batch
 * known).  With at least one tile per SM the transposed kernel is taken unless the halo kernel's 14 x 8 blocks leave fewer
 * MMA rows idle than its tiles leave columns (at equal fill it measured ~5 % faster; on 28- and 14-pixel images it fills
 * 0.875 against 0.766).  With fewer tiles than SMs (batch 1) latency counts, not idle columns, and the halo kernel's
 * smaller tiles spread further: then only layers of at most 128 channels whose image tiles well into 14 x 16 blocks go
 * to the transposed kernel. */
static int use_swap_kernel(int variant, int n, int W, int H, int Cout, int pool, int sms)
{
    int P, TW, TH;
    long long tiles;
    if (dRk_debug_switches()->no_swap) return 0;
    const double fill = swap_geometry_for(n, W, H, Cout, pool ? 1 : 0, sms, &P, &TW, &TH, &tiles);
    if (fill <= 0.0) return 0;
    if (tiles >= sms) return variant == VAR_SWAP || fill >= halo_fill(W, H) - 0.01;
    /* from about half a tile per SM the transposed kernel still wins (128 -> 128 @28x28 at batch 32, 128 tiles: 17 against 27 us;
       512 -> 512 @14x14 at batch 32: 48 against 54 us; at 64 tiles the two are level).  Halving the tile rows to double the tile
       count was measured and loses: an MMA of N = 128 columns issues at 104 clocks, barely faster than N = 224 (256 -> 256 @14x14
       at batch 64: 45 against 27 us). */
    if (2 * tiles >= sms) return 1;
    const double tx = (W + HALO_TW - 1) / HALO_TW, ty = (H + 15) / 16;
    return Cout <= BM && (double)W * H / (tx * ty * SWAP_N) >= 0.8;
}

static int pick_bn(int Cout, long long m_tiles, int sms)
{
    /* N tile: fewest waves of tiles over the SMs, weighting a tile by its width plus a fixed part (pipeline fill, epilogue tail);
       a tile wider than what is left of Cout wastes the difference */
    int best = 64;
    double best_cost = 1e30;
    const int cand[3] = {256, 128, 64};
    for (int i = 0; i < 3; i++) {
        const int bn = cand[i];
        const long long tiles = m_tiles * ((Cout + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        const double cost = (double)waves * (bn + 48.0);
        if (cost < best_cost * 0.97) { best_cost = cost; best = bn; }
    }
    return best;
}

template <int BN>
static int launch_umma_halo(cudaStream_t st, dRk_TensorConvPlan *pl)
{
    static bool attr_done[DRK_MAX_DEVICES];         /* the opt-in shared-memory size is a per-device function attribute */
    const int dev = current_device();
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_umma_conv_halo<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, HaloCfg<BN>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    drk_launch_dep(k_umma_conv_halo<BN>, dim3(pl->grid), dim3(UMMA_THREADS), HaloCfg<BN>::SMEM_BYTES, st, pl->mapA, pl->mapB, pl->p);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

template <int BN>
static int launch_umma(cudaStream_t st, dRk_TensorConvPlan *pl)
{
    static bool attr_done[DRK_MAX_DEVICES];
    const int dev = current_device();
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_umma_conv<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    drk_launch_dep(k_umma_conv<BN>, dim3(pl->grid), dim3(UMMA_THREADS), Cfg<BN>::SMEM_BYTES, st, pl->mapA, pl->mapB, pl->p);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

/* Which kernel and block geometry the planner takes for a layer, without touching a device (variant: 1 flat 1x1, 2 plain,
 * 3 halo, 4 transposed, 5 row pair, 6 few-channel first layer; 0 = not a tensor-path shape).  P / TW / TH are the pixel pitch,
 * valid pixels and rows (row pairs for variant 5) of a block, ncols the MMA's N; zero where the variant has no such notion. */
extern "C" int dRk_tensor_conv_describe(int n, int W, int H, int Cin, int Cout, int kw, int kh, int fuse_pool2, int sms,
                                        int *P, int *TW, int *TH, int *ncols)
{
    int v = pick_variant(W, H, Cin, Cout, kw, kh);
    *P = *TW = *TH = *ncols = 0;
    if (v == VAR_NONE || !dRk_tensor_conv_can_fuse_pool(W, H, Cin, Cout, kw, kh, fuse_pool2)) return 0;
    if (v == VAR_PAIR) {
        drk_umma_pair_geometry(W, H, P, TW, TH);
        *ncols = *P * *TH;
    } else if (v == VAR_SWAP || v == VAR_HALO) {
        if (use_swap_kernel(v, n, W, H, Cout, fuse_pool2, sms)) {
            v = VAR_SWAP;
            long long tiles;
            swap_geometry_for(n, W, H, Cout, fuse_pool2 ? 1 : 0, sms, P, TW, TH, &tiles);
            *ncols = *P * *TH;
        } else if (halo_fill(W, H) >= 0.55 && !dRk_debug_switches()->no_halo) {
            v = VAR_HALO;
            *P = HALO_P; *TW = HALO_TW; *TH = HALO_TH; *ncols = 0;
        } else {
            v = VAR_PLAIN;
        }
    }
    return v;
}

extern "C" dRk_TensorConvPlan *dRk_tensor_conv_plan(const float *in, const float *wT, const float *bias, float *out, int n, int W, int H,
                                                    int Cin, int Cout, int kw, int kh, int act, int ldo, int coff, int fuse_pool2, int *status)
{
    if (!dRk_tensor_conv_supported(W, H, Cin, Cout, kw, kh) || n <= 0) return NULL;
    if (!dRk_tensor_conv_can_fuse_pool(W, H, Cin, Cout, kw, kh, fuse_pool2)) return NULL;
    if (ldo % 4 || coff % 4 || ((uintptr_t)out % 16) || ((uintptr_t)in % 16) || ((uintptr_t)wT % 16) || (bias && ((uintptr_t)bias % 16))) return NULL;
    PFN_encodeTiled enc = get_encode();
    if (!enc) return NULL;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dRk_TensorConvPlan *pl = (dRk_TensorConvPlan *)calloc(1, sizeof(dRk_TensorConvPlan));
    if (!pl) return NULL;
    UmmaParams &p = pl->p;
    pl->in = in; pl->wT = wT; pl->sms = sms;
    const int variant = pick_variant(W, H, Cin, Cout, kw, kh);
    if (variant == VAR_FIRST) {
        pl->first = 1;
        pl->ldi = Cin;
        p.n = n; p.W = W; p.H = H; p.Cin = Cin; p.Cout = Cout; p.bias = bias; p.out = out; p.ldo = ldo; p.coff = coff; p.act = act; p.status = status;
        p.pool = fuse_pool2;
        return pl;
    }
    p.n = n; p.W = W; p.H = H; p.Cin = Cin; p.Cout = Cout;
    p.CinPad = (Cin + BK - 1) / BK * BK;
    p.taps = kw * kh; p.kw = kw; p.pad = kw / 2;
    p.kslabs = p.CinPad / BK;
    p.bias = bias; p.out = out; p.ldo = ldo; p.coff = coff; p.act = act; p.status = status; p.pool = fuse_pool2 ? 1 : 0;
    p.ksplit = 1; p.kper = p.kslabs; p.split_stride = 0;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    CUresult r;
    if (kw == 1) {
        p.S = 0; p.TW = BM; p.TH = 1; p.tiles_x = p.tiles_y = 1;
        p.total_sub = (long long)n * H * W;
        p.m_tiles = (int)((p.total_sub + BM - 1) / BM);
        const cuuint64_t dims[2] = {(cuuint64_t)Cin, (cuuint64_t)p.total_sub};
        const cuuint64_t strides[1] = {(cuuint64_t)Cin * 4};
        const cuuint32_t box[2] = {BK, BM};
        r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2, (void *)in, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (variant == VAR_PAIR) {
        pl->pair = 1;
        p.S = 1;
        drk_umma_pair_geometry(W, H, &p.P, &p.TW, &p.TH);          /* TH = row pairs per tile */
        p.ncols = p.P * p.TH;
        p.tiles_x = (W + p.TW - 1) / p.TW; p.tiles_y = (H + 2 * p.TH - 1) / (2 * p.TH);
        p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
        p.m_tiles = (int)p.total_sub;
        const cuuint32_t box[4] = {BK, (cuuint32_t)p.P, (cuuint32_t)(p.TH + 1), 1};
        /* input rows split by parity: the even plane starts at row 0, the odd plane at row 1, both step two rows */
        const cuuint64_t strides[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)2 * W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
        const cuuint64_t dimsE[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)((H + 1) / 2), (cuuint64_t)n};
        const cuuint64_t dimsO[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)(H / 2), (cuuint64_t)n};
        r = enc(&pl->mapA2, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)in, dimsE, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS)
            r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)(in + (size_t)W * Cin), dimsO, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if ((variant == VAR_SWAP || variant == VAR_HALO) && use_swap_kernel(variant, n, W, H, Cout, fuse_pool2, sms)) {
        pl->swap = 1;
        p.S = 1;
        long long geo_tiles;
        swap_geometry_for(n, W, H, Cout, fuse_pool2 ? 1 : 0, sms, &p.P, &p.TW, &p.TH, &geo_tiles);
        p.ncols = p.P * p.TH;
        p.tiles_x = (W + p.TW - 1) / p.TW; p.tiles_y = (H + p.TH - 1) / p.TH;
        p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
        p.m_tiles = (int)p.total_sub;
        const cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)n};
        const cuuint64_t strides[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
        const cuuint32_t box[4] = {BK, (cuuint32_t)p.P, (cuuint32_t)(p.TH + 2), 1};
        r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)in, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if ((variant == VAR_HALO || variant == VAR_SWAP) && halo_fill(W, H) >= 0.55 && !dRk_debug_switches()->no_halo) {
        pl->halo = 1;
        p.TW = HALO_TW; p.TH = HALO_TH; p.S = 1;
        p.tiles_x = (W + HALO_TW - 1) / HALO_TW; p.tiles_y = (H + HALO_TH - 1) / HALO_TH;
        p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
        p.m_tiles = (int)p.total_sub;
        const cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)n};
        const cuuint64_t strides[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
        const cuuint32_t box[4] = {BK, HALO_P, HALO_TH + 2, 1};
        r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)in, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        pick_subtile(W, H, fuse_pool2, &p.TW, &p.TH, &p.S);
        p.tiles_x = (W + p.TW - 1) / p.TW;
        p.tiles_y = (H + p.TH - 1) / p.TH;
        p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
        p.m_tiles = (int)((p.total_sub + p.S - 1) / p.S);
        const cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)n};
        const cuuint64_t strides[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
        const cuuint32_t box[4] = {BK, (cuuint32_t)p.TW, (cuuint32_t)p.TH, 1};
        r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)in, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) { fprintf(stderr, "tensor conv plan: activation tensor map rejected (%d)\n", (int)r); free(pl); return NULL; }
    pl->BN = (pl->swap || pl->pair) ? BM : pick_bn(Cout, p.m_tiles, sms);
    p.n_tiles = pl->pair ? 1 : pl->swap ? (Cout + BM - 1) / BM : (Cout + pl->BN - 1) / pl->BN;
    {
        const cuuint64_t K = (cuuint64_t)(pl->pair ? 12 : p.taps) * p.CinPad;
        const cuuint64_t dims[2] = {K, (cuuint64_t)(pl->pair ? BM : Cout)};
        const cuuint64_t strides[1] = {K * 4};
        const cuuint32_t box[2] = {BK, (cuuint32_t)pl->BN};
        r = enc(&pl->mapB, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2, (void *)wT, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) { fprintf(stderr, "tensor conv plan: filter tensor map rejected (%d)\n", (int)r); free(pl); return NULL; }
    p.stage_tx = (p.S == 0 ? A_STAGE_BYTES : p.S * p.TW * p.TH * BK * 4) + pl->BN * BK * 4;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    pl->grid = (int)(tiles < sms ? tiles : sms);
    return pl;
}

/*
 * FP32-accurate 3x3 convolution on the tensor cores (see k_umma_conv_swap<true>): stride 1, Cin % 4 == 0, Cin >= 8,
 * Cout % 4 == 0, Cout >= 16, any image size.  wT2 holds the filters [Cout][9*CinPad] (as dRk_tensor_conv_pack_weights writes
 * them for the transposed kernel) followed by their low parts in the same layout.
 */
extern "C" int dRk_tensor_conv_x3_supported(int W, int H, int Cin, int Cout)
{
    int P, TW, TH;
    /* Cin <= 768: the accumulator in TMEM rounds by truncation once per MMA, an error that grows with the MMA count per output
       (measured 4.7e-5 * max|ref| at Cin = 512); deeper layers would leave the FP32 class's 1e-4 bound and stay on FFMA */
    return dRk_tensor_conv_supported(W, H, Cin, Cout, 3, 3) && Cin >= 8 && Cin <= 768 && swap_geometry(W, H, 0, &P, &TW, &TH) > 0.0;
}

/* layers of at most 64 output channels whose image suits the row-pair blocks run k_umma_conv_pair<true>, all others k_umma_conv_swap<true> */
static bool x3_uses_pair(int W, int H, int Cout)
{
    const drk_DebugSwitches *sw = dRk_debug_switches();
    return Cout <= 64 && H >= 2 && drk_umma_pair_fill(W, H) >= 0.5 && !sw->no_pair && !sw->no_halo;
}

extern "C" size_t dRk_tensor_conv_x3_packed_floats(int W, int H, int Cin, int Cout)
{
    const size_t cp = (size_t)(Cin + BK - 1) / BK * BK;
    return x3_uses_pair(W, H, Cout) ? (size_t)2 * BM * 12 * cp : (size_t)2 * Cout * 9 * cp;
}

extern "C" int dRk_tensor_conv_x3_pack_weights(const float *w, float *dst, int W, int H, int Cin, int Cout)
{
    if (!w || !dst || Cin <= 0 || Cout <= 0) return -1;
    const size_t cp = (size_t)(Cin + BK - 1) / BK * BK;
    const bool pair = x3_uses_pair(W, H, Cout);
    const size_t half = pair ? (size_t)BM * 12 * cp : (size_t)Cout * 9 * cp;
    memset(dst, 0, 2 * half * sizeof(float));
    for (int c = 0; c < Cin; c++)
        for (int o = 0; o < Cout; o++)
            for (int t = 0; t < 9; t++) {
                const float v = w[((size_t)c * Cout + o) * 9 + t];
                uint32_t bits;
                memcpy(&bits, &v, 4);
                bits &= 0xffffe000u;                        /* what a kind::tf32 MMA reads of v */
                float hi;
                memcpy(&hi, &bits, 4);
                if (!pair) {
                    dst[(size_t)o * 9 * cp + (size_t)t * cp + c] = v;
                    dst[half + (size_t)o * 9 * cp + (size_t)t * cp + c] = v - hi;
                } else {
                    /* the row-pair layout of dRk_tensor_conv_pack_weights: row o holds tap (ky, kx) at i = ky, row 64 + o at i = ky + 1 */
                    const int ky = t / 3, kx = t - ky * 3;
                    for (int lower = 0; lower < 2; lower++) {
                        const size_t at = (size_t)(lower * 64 + o) * 12 * cp + (size_t)((ky + lower) * 3 + kx) * cp + c;
                        dst[at] = v;
                        dst[half + at] = v - hi;
                    }
                }
            }
    return 0;
}

extern "C" dRk_TensorConvPlan *dRk_tensor_conv_x3_plan(const float *in, const float *wT2, const float *bias, float *out, int n, int W, int H,
                                                       int Cin, int Cout, int act, int ldo, int coff, int fuse_pool2, int *status)
{
    if (n <= 0 || !dRk_tensor_conv_x3_supported(W, H, Cin, Cout)) return NULL;
    if (fuse_pool2 && (fuse_pool2 != 1 || (W & 1) || (H & 1))) return NULL;
    if (ldo % 4 || coff % 4 || ((uintptr_t)out % 16) || ((uintptr_t)in % 16) || ((uintptr_t)wT2 % 16) || (bias && ((uintptr_t)bias % 16))) return NULL;
    PFN_encodeTiled enc = get_encode();
    if (!enc) return NULL;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dRk_TensorConvPlan *pl = (dRk_TensorConvPlan *)calloc(1, sizeof(dRk_TensorConvPlan));
    if (!pl) return NULL;
    UmmaParams &p = pl->p;
    pl->in = in; pl->wT = wT2; pl->sms = sms; pl->x3 = 1; pl->BN = BM;
    p.n = n; p.W = W; p.H = H; p.Cin = Cin; p.Cout = Cout;
    p.CinPad = (Cin + BK - 1) / BK * BK;
    p.taps = 9; p.kw = 3; p.pad = 1; p.kslabs = p.CinPad / BK;
    p.bias = bias; p.out = out; p.ldo = ldo; p.coff = coff; p.act = act; p.status = status; p.pool = fuse_pool2 ? 1 : 0;
    p.ksplit = 1; p.kper = p.kslabs; p.S = 1;
    if (x3_uses_pair(W, H, Cout)) {
        /* the row-pair kernel in three-pass mode: planes and filters exactly as in dRk_tensor_conv_plan, FLOAT32 maps, one more map for the filters' low parts */
        pl->pair = 1;
        drk_umma_pair_geometry(W, H, &p.P, &p.TW, &p.TH);
        p.ncols = p.P * p.TH;
        p.tiles_x = (W + p.TW - 1) / p.TW; p.tiles_y = (H + 2 * p.TH - 1) / (2 * p.TH);
        p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
        p.m_tiles = (int)p.total_sub;
        p.n_tiles = 1;
        const cuuint32_t ones4[4] = {1, 1, 1, 1};
        const cuuint32_t pbox[4] = {BK, (cuuint32_t)p.P, (cuuint32_t)(p.TH + 1), 1};
        const cuuint64_t pstr[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)2 * W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
        const cuuint64_t dimsE[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)((H + 1) / 2), (cuuint64_t)n};
        const cuuint64_t dimsO[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)(H / 2), (cuuint64_t)n};
        CUresult rp = enc(&pl->mapA2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)in, dimsE, pstr, pbox, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rp == CUDA_SUCCESS)
            rp = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)(in + (size_t)W * Cin), dimsO, pstr, pbox, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        const cuuint64_t Kp = (cuuint64_t)12 * p.CinPad;
        const cuuint64_t fdims[2] = {Kp, (cuuint64_t)BM}, fstr[1] = {Kp * 4};
        const cuuint32_t fbox[2] = {BK, BM};
        if (rp == CUDA_SUCCESS)
            rp = enc(&pl->mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)wT2, fdims, fstr, fbox, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rp == CUDA_SUCCESS)
            rp = enc(&pl->mapB2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)(wT2 + (size_t)BM * Kp), fdims, fstr, fbox, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rp != CUDA_SUCCESS) { fprintf(stderr, "tensor conv x3 plan: tensor map rejected (%d)\n", (int)rp); free(pl); return NULL; }
        p.stage_tx = p.TW * p.TH * BK * 4 + BM * BK * 4;
        pl->grid = (int)(p.m_tiles < sms ? p.m_tiles : sms);
        return pl;
    }
    pl->swap = 1;
    long long geo_tiles;
    swap_geometry_for(n, W, H, Cout, fuse_pool2 ? 1 : 0, sms, &p.P, &p.TW, &p.TH, &geo_tiles);
    p.ncols = p.P * p.TH;
    p.tiles_x = (W + p.TW - 1) / p.TW; p.tiles_y = (H + p.TH - 1) / p.TH;
    p.total_sub = (long long)n * p.tiles_x * p.tiles_y;
    p.m_tiles = (int)p.total_sub;
    p.n_tiles = (Cout + BM - 1) / BM;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    const cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)n};
    const cuuint64_t strides[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
    const cuuint32_t box[4] = {BK, (cuuint32_t)p.P, (cuuint32_t)(p.TH + 2), 1};
    /* FLOAT32 maps: TMA must deliver the bits unchanged, the split into high and low parts happens in the kernel */
    CUresult r = enc(&pl->mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)in, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    const cuuint64_t K = (cuuint64_t)9 * p.CinPad;
    const cuuint64_t wdims[2] = {K, (cuuint64_t)Cout}, wstr[1] = {K * 4};
    const cuuint32_t wbox[2] = {BK, BM};
    if (r == CUDA_SUCCESS)
        r = enc(&pl->mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)wT2, wdims, wstr, wbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS)
        r = enc(&pl->mapA2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)(wT2 + (size_t)Cout * K), wdims, wstr, wbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "tensor conv x3 plan: tensor map rejected (%d)\n", (int)r); free(pl); return NULL; }
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    pl->grid = (int)(tiles < sms ? tiles : sms);
    return pl;
}

/* The kernel and block geometry of a built plan, in the numbering of dRk_tensor_conv_describe. */
extern "C" int dRk_tensor_conv_plan_describe(const dRk_TensorConvPlan *pl, int *P, int *TW, int *TH, int *ncols)
{
    *P = *TW = *TH = *ncols = 0;
    if (!pl) return VAR_NONE;
    if (pl->first) return VAR_FIRST;
    if (pl->p.S == 0) return VAR_FLAT;
    *TW = pl->p.TW; *TH = pl->p.TH;
    if (pl->pair || pl->swap) { *P = pl->p.P; *ncols = pl->p.ncols; return pl->pair ? VAR_PAIR : VAR_SWAP; }
    if (pl->halo) { *P = HALO_P; return VAR_HALO; }
    return VAR_PLAIN;
}

extern "C" int dRk_tensor_conv_set_input_map(dRk_TensorConvPlan *pl, int ldi, const int *ch, const float *scale, const float *shift)
{
    if (!pl || !pl->first || !ch || !scale || !shift || ldi < pl->p.Cin) return -1;
    unsigned seen = 0;
    for (int c = 0; c < pl->p.Cin; c++) {
        if (ch[c] < 0 || ch[c] >= pl->p.Cin || (seen >> ch[c]) & 1u) return -1;      /* a permutation of the first Cin source channels */
        seen |= 1u << ch[c];
        pl->map_ch[c] = ch[c]; pl->map_scale[c] = scale[c]; pl->map_shift[c] = shift[c];
    }
    pl->ldi = ldi;
    pl->mapped = 1;
    return 0;
}

extern "C" int dRk_tensor_conv_run(dRk_stream stream, dRk_TensorConvPlan *pl)
{
    if (!pl) return -1;
    cudaStream_t st = drk_stream(stream);
    if (pl->first)
        return drk_umma_first_launch(st, pl->in, pl->wT, pl->p.bias, pl->p.out, pl->p.n, pl->p.W, pl->p.H, pl->p.Cin, pl->p.Cout, pl->p.act,
                                     pl->ldi, pl->p.ldo, pl->p.coff, pl->p.pool, pl->p.status, pl->sms, pl->mapped ? pl->map_ch : NULL,
                                     pl->map_scale, pl->map_shift);
    if (pl->pair) return drk_umma_pair_launch(st, &pl->mapA, &pl->mapA2, &pl->mapB, pl->x3 ? &pl->mapB2 : &pl->mapB, &pl->p, pl->grid, pl->x3);
    if (pl->swap) {
        static bool attr_done[DRK_MAX_DEVICES];
        const int dev = current_device();
        if (!attr_done[dev]) {
            cudaError_t e = cudaFuncSetAttribute(k_umma_conv_swap<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SWAP_SMEM);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(k_umma_conv_swap<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SWAP_SMEM);
            if (e != cudaSuccess) return (int)e;
            attr_done[dev] = true;
        }
        if (pl->x3) drk_launch_dep(k_umma_conv_swap<true>, dim3(pl->grid), dim3(SWAP_THREADS(1)), SWAP_SMEM, st, pl->mapA, pl->mapB, pl->mapA2, pl->p);
        else drk_launch_dep(k_umma_conv_swap<false>, dim3(pl->grid), dim3(SWAP_THREADS(0)), SWAP_SMEM, st, pl->mapA, pl->mapB, pl->mapB, pl->p);
        DRK_COUNT_LAUNCH();
        return DRK_LAUNCH_RESULT();
    }
    if (pl->halo) {
        switch (pl->BN) {
        case 256: return launch_umma_halo<256>(st, pl);
        case 128: return launch_umma_halo<128>(st, pl);
        case 64: return launch_umma_halo<64>(st, pl);
        }
        return -1;
    }
    switch (pl->BN) {
    case 256: return launch_umma<256>(st, pl);
    case 128: return launch_umma<128>(st, pl);
    case 64: return launch_umma<64>(st, pl);
    }
    return -1;
}

extern "C" void dRk_tensor_conv_free(dRk_TensorConvPlan *pl) { free(pl); }

/*
 * Fully connected layer on the tensor cores (TF32 mode, larger batches): the activations [n][Nin] are the
 * A operand of a flat GEMM (rows past the batch are TMA zero fill), the weights the B operand with N = 256 per tile,
 * stored block by block (256 output columns x 32 inputs = one TMA request = one contiguous 32 KiB run); K is split over enough CTAs to occupy every SM, the partial products
 * land in `scratch` ([ksplit][n][Nout]) and the reduce kernel of the FP32 path adds bias and activation.
 * Bound: HBM (weights read once).  Replaces matrixVectorMultFirst/Second (Kernels/dR_fcl.cl:59-120).
 */
int drk_fc_reduce_launch(cudaStream_t st, const float *partial, const float *bias, float *out, int total, int Nout, int splits, int act);

struct dRk_TensorFcPlan {
    dRk_TensorConvPlan conv;
    const float *bias, *in;
    float *out, *scratch;       /* split-K partial sums */
    float *in2;                 /* three-pass mode: the activations as (high | low) rows [n][2*Nin], rewritten by every run */
    int n, Nin, Nout, act;
};

extern "C" int dRk_tensor_fc_supported(int n, int Nin, int Nout)
{
    /* output columns past Nout inside the last 256-wide tile are TMA zero fill (weights) and masked stores */
    return n >= 16 && n <= BM && Nin % BK == 0 && Nout % 4 == 0 && Nout >= 64 && Nin >= 8 * BK;
}

extern "C" size_t dRk_tensor_fc_scratch_floats(int n, int Nin, int Nout)
{
    if (!dRk_tensor_fc_supported(n, Nin, Nout)) return 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int ksplit = sms / ((Nout + 255) / 256);
    if (ksplit < 1) ksplit = 1;
    const int kslabs = Nin / BK;
    if (ksplit > kslabs / 8) ksplit = kslabs / 8 > 0 ? kslabs / 8 : 1;
    return (size_t)ksplit * n * Nout;
}

extern "C" size_t dRk_tensor_fc_packed_floats(int Nin, int Nout)
{
    if (Nin <= 0 || Nout <= 0 || Nin % BK != 0) return 0;
    return (size_t)((Nout + 255) / 256) * 256 * (size_t)Nin;
}

/* [n tile][K slab][256 output columns][32 inputs]: block (nt, ks) holds w[ks*32 + e][nt*256 + r] at [r][e]; columns past Nout are zeros */
extern "C" int dRk_tensor_fc_pack_weights(const float *w, float *wpacked, int Nin, int Nout)
{
    if (!w || !wpacked || Nin <= 0 || Nout <= 0 || Nin % BK != 0) return -1;
    const int ntiles = (Nout + 255) / 256, kslabs = Nin / BK;
    for (int nt = 0; nt < ntiles; nt++)
        for (int ks = 0; ks < kslabs; ks++) {
            float *blk = wpacked + ((size_t)nt * kslabs + ks) * 256 * BK;
            for (int e = 0; e < BK; e++) {
                const float *src = w + (size_t)(ks * BK + e) * Nout + (size_t)nt * 256;
                const int valid = Nout - nt * 256 < 256 ? Nout - nt * 256 : 256;
                for (int r = 0; r < valid; r++) blk[(size_t)r * BK + e] = src[r];
                for (int r = valid; r < 256; r++) blk[(size_t)r * BK + e] = 0.0f;
            }
        }
    return 0;
}

static int tensor_fc_ksplit(int Nin, int Nout, int x3, int sms)
{
    const int kslabs = (x3 ? 3 : 1) * (Nin / BK);
    int ksplit = sms / ((Nout + 255) / 256);
    if (ksplit < 1) ksplit = 1;
    if (ksplit > kslabs / 8) ksplit = kslabs / 8 > 0 ? kslabs / 8 : 1;
    return ksplit;
}

static dRk_TensorFcPlan *tensor_fc_plan(const float *in, const float *wpacked, const float *bias, float *out, float *scratch,
                                        int n, int Nin, int Nout, int act, int x3, int *status)
{
    if (!dRk_tensor_fc_supported(n, Nin, Nout) || !scratch) return NULL;
    if (((uintptr_t)in % 16) || ((uintptr_t)wpacked % 16) || ((uintptr_t)scratch % 16)) return NULL;
    PFN_encodeTiled enc = get_encode();
    if (!enc) return NULL;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dRk_TensorFcPlan *fp = (dRk_TensorFcPlan *)calloc(1, sizeof(dRk_TensorFcPlan));
    if (!fp) return NULL;
    dRk_TensorConvPlan *pl = &fp->conv;
    UmmaParams &p = pl->p;
    /* three-pass mode: the head of the scratch holds the (high | low) activations, the partial sums follow */
    float *in2 = x3 ? scratch : NULL;
    float *partial = x3 ? scratch + (((size_t)n * 2 * Nin + 3) & ~(size_t)3) : scratch;
    p.n = n; p.W = 1; p.H = 1; p.Cin = Nin; p.CinPad = Nin; p.Cout = Nout;
    p.taps = 1; p.kw = 1; p.pad = 0;
    p.x3cat = x3 ? Nin / BK : 0;
    p.kslabs = (x3 ? 3 : 1) * (Nin / BK);
    p.S = 0; p.TW = BM; p.TH = 1; p.tiles_x = p.tiles_y = 1;
    p.total_sub = n; p.m_tiles = 1; p.n_tiles = (Nout + 255) / 256;
    p.bias = NULL; p.out = partial; p.ldo = Nout; p.coff = 0; p.act = 0; p.pool = 0; p.status = status;
    p.ksplit = tensor_fc_ksplit(Nin, Nout, x3, sms);
    p.kper = (p.kslabs + p.ksplit - 1) / p.ksplit;
    p.ksplit = (p.kslabs + p.kper - 1) / p.kper;          /* no empty parts */
    p.split_stride = (long long)n * Nout;
    pl->BN = 256;
    p.stage_tx = A_STAGE_BYTES + 256 * BK * 4;
    const CUtensorMapDataType dt = x3 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32;
    const cuuint64_t Kw = (cuuint64_t)(x3 ? 2 * Nin : Nin);
    const cuuint32_t ones[2] = {1, 1};
    const cuuint64_t adims[2] = {Kw, (cuuint64_t)n}, astr[1] = {Kw * 4};
    const cuuint32_t abox[2] = {BK, BM};
    CUresult r = enc(&pl->mapA, dt, 2, (void *)(x3 ? in2 : in), adims, astr, abox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    /* the packed weights as a 32-wide matrix whose rows are the blocks' rows one after another */
    p.bpacked = 1;
    const cuuint64_t bdims[2] = {(cuuint64_t)BK, (cuuint64_t)p.n_tiles * (x3 ? 2 : 1) * (Nin / BK) * 256}, bstr[1] = {(cuuint64_t)BK * 4};
    const cuuint32_t bbox[2] = {BK, 256};
    if (r == CUDA_SUCCESS)
        r = enc(&pl->mapB, dt, 2, (void *)wpacked, bdims, bstr, bbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "tensor fc plan: tensor map rejected (%d)\n", (int)r); free(fp); return NULL; }
    const long long tiles = (long long)p.n_tiles * p.ksplit;
    pl->grid = (int)(tiles < sms ? tiles : sms);
    fp->bias = bias; fp->in = in; fp->out = out; fp->scratch = partial; fp->in2 = in2; fp->n = n; fp->Nin = Nin; fp->Nout = Nout; fp->act = act;
    return fp;
}

extern "C" dRk_TensorFcPlan *dRk_tensor_fc_plan(const float *in, const float *wpacked, const float *bias, float *out, float *scratch,
                                                int n, int Nin, int Nout, int act, int *status)
{
    return tensor_fc_plan(in, wpacked, bias, out, scratch, n, Nin, Nout, act, 0, status);
}

/* FP32-accurate variant: every product as hi x hi + hi x lo + lo x hi of TF32 halves (three passes of the K loop); the weights
 * are packed as high and low blocks, the activations are split into (high | low) rows at the head of `scratch` by every run */
extern "C" size_t dRk_tensor_fc_x3_packed_floats(int Nin, int Nout) { return 2 * dRk_tensor_fc_packed_floats(Nin, Nout); }

extern "C" size_t dRk_tensor_fc_x3_scratch_floats(int n, int Nin, int Nout)
{
    if (!dRk_tensor_fc_supported(n, Nin, Nout)) return 0;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return (((size_t)n * 2 * Nin + 3) & ~(size_t)3) + (size_t)tensor_fc_ksplit(Nin, Nout, 1, sms) * n * Nout;
}

/* [n tile][2 * K slabs][256][32]: the slabs of the high parts (upper 19 bits of the weight), then those of the remainders */
extern "C" int dRk_tensor_fc_x3_pack_weights(const float *w, float *wpacked, int Nin, int Nout)
{
    if (!w || !wpacked || Nin <= 0 || Nout <= 0 || Nin % BK != 0) return -1;
    const int ntiles = (Nout + 255) / 256, kslabs = Nin / BK;
    for (int nt = 0; nt < ntiles; nt++)
        for (int ks = 0; ks < kslabs; ks++) {
            float *hi = wpacked + ((size_t)nt * 2 * kslabs + ks) * 256 * BK, *lo = hi + (size_t)kslabs * 256 * BK;
            const int valid = Nout - nt * 256 < 256 ? Nout - nt * 256 : 256;
            for (int e = 0; e < BK; e++) {
                const float *src = w + (size_t)(ks * BK + e) * Nout + (size_t)nt * 256;
                for (int r = 0; r < 256; r++) {
                    float h = 0.0f, l = 0.0f;
                    if (r < valid) {
                        uint32_t bits;
                        memcpy(&bits, &src[r], 4);
                        bits &= 0xffffe000u;
                        memcpy(&h, &bits, 4);
                        l = src[r] - h;
                    }
                    hi[(size_t)r * BK + e] = h;
                    lo[(size_t)r * BK + e] = l;
                }
            }
        }
    return 0;
}

extern "C" dRk_TensorFcPlan *dRk_tensor_fc_x3_plan(const float *in, const float *wpacked2, const float *bias, float *out, float *scratch,
                                                   int n, int Nin, int Nout, int act, int *status)
{
    return tensor_fc_plan(in, wpacked2, bias, out, scratch, n, Nin, Nout, act, 1, status);
}

/* rows of (high | low) halves: out[r][c] = upper 19 bits of in[r][c], out[r][K + c] = the remainder (exact) */
__global__ void k_split_hi_lo(const float *__restrict__ in, float *__restrict__ out, int rows, int K)
{
    drk_dep_trigger();
    drk_dep_wait();
    const size_t total = (size_t)rows * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / K, c = i - r * K;
        const float v = in[i];
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        out[r * 2 * K + c] = h;
        out[r * 2 * K + K + c] = v - h;
    }
}

extern "C" int dRk_tensor_fc_run(dRk_stream stream, dRk_TensorFcPlan *fp)
{
    if (!fp) return -1;
    if (fp->in2) {
        const size_t total = (size_t)fp->n * fp->Nin;
        drk_launch_dep(k_split_hi_lo, dim3(drk_blocks(total, 256, 148u * 8u)), dim3(256), 0, drk_stream(stream), fp->in, fp->in2, fp->n, fp->Nin);
        DRK_COUNT_LAUNCH();
        const int rc0 = DRK_LAUNCH_RESULT();
        if (rc0) return rc0;
    }
    int rc = launch_umma<256>(drk_stream(stream), &fp->conv);
    if (rc) return rc;
    return drk_fc_reduce_launch(drk_stream(stream), fp->scratch, fp->bias, fp->out, fp->n * fp->Nout, fp->Nout, fp->conv.p.ksplit, fp->act);
}

extern "C" void dRk_tensor_fc_free(dRk_TensorFcPlan *fp) { free(fp); }

/*
 * Winograd F(2x2,3x3) with the transform-domain products on the tensor cores (TF32 mode).
 *
 * The reference's algorithm (Kernels/dR_winograd2.cl:23-254: input transform :64-157, product :177-189, output
 * transform :198-217; filter transform src/dR_nodes_conv2d.c:1162-1240) split at its two seams: the FP32 transform kernels of
 * k_winograd.cu write V[16][Tp][Cin] and read M[16][Tp][Cout] (Tp = tile count rounded up to whole 128-row GEMM tiles), and the
 * sixteen products M_k = V_k U_k run as ONE launch of the flat tensor GEMM above: the sixteen V_k are stacked on M, and every
 * Tp / 128 row tiles the filter operand moves on to the next U_k (UmmaParams::bgroup_*).  2.25x fewer multiplications than
 * the direct tensor kernels, paid for with V and M passing through memory (16 * T * (Cin + Cout) floats written and read):
 * it is a candidate for the autotuner, not the planner's static choice.  Layers larger than the scratch cap run in image chunks.
 */
#include "k_gemm_f32.cuh"

#define TWINO_SCRATCH_CAP ((size_t)1 << 28)     /* floats (1 GiB) */

struct dRk_TensorWinogradPlan {
    dRk_TensorConvPlan gemm[2];                 /* full chunks, tail chunk */
    size_t T[2], Tp[2];
    int imgs[2], nfull;
    const float *in, *bias;
    float *out, *V, *M;
    int n, W, H, Cin, Cout, act, ldi, ldo, coff;
    int f4x3;                                   /* 0: F(2x2,3x3) with TF32 products; 1: F(4x4,3x3) with three-pass (FP32-accurate) products */
    int pool;                                   /* F(4x4): the output transform evaluates a following 2x2/2 max pooling */
};

static size_t twino_tiles(int W, int H) { return (size_t)((W + 1) / 2) * ((H + 1) / 2); }
static size_t twino_pad(size_t T) { return (T + BM - 1) / BM * BM; }
static int twino_chunk(int n, int W, int H, int Cin, int Cout)
{
    const size_t per = 16 * twino_tiles(W, H) * (size_t)(Cin + Cout);
    size_t c = (TWINO_SCRATCH_CAP - 16 * (size_t)BM * (Cin + Cout)) / per;     /* room for the padding rows */
    if (c < 1) c = 1;
    if (c > (size_t)n) c = (size_t)n;
    const size_t chunks = ((size_t)n + c - 1) / c;          /* equal chunks rather than full ones and a short last one */
    c = ((size_t)n + chunks - 1) / chunks;
    return (int)c;
}

extern "C" int dRk_tensor_winograd_supported(int W, int H, int Cin, int Cout)
{
    return dRk_tensor_conv_supported(W, H, Cin, Cout, 3, 3) && Cin >= 8 && twino_pad(twino_tiles(W, H)) * 16 <= 0x7fffffffull / 2;
}

extern "C" size_t dRk_tensor_winograd_scratch_floats(int n, int W, int H, int Cin, int Cout)
{
    if (n <= 0 || !dRk_tensor_winograd_supported(W, H, Cin, Cout)) return 0;
    return 16 * twino_pad(twino_tiles(W, H) * twino_chunk(n, W, H, Cin, Cout)) * (size_t)(Cin + Cout);
}

extern "C" size_t dRk_tensor_winograd_packed_floats(int Cin, int Cout) { return (size_t)16 * Cout * Cin; }

/* U_k = (G g G^T)_k per (input, output) channel pair from the reference's [Cin][Cout][3][3] filters, stored [16][Cout][Cin]
 * (K contiguous): G = [[1,0,0],[.5,.5,.5],[.5,-.5,.5],[0,0,1]] (src/dR_nodes_conv2d.c:1173-1176) */
extern "C" int dRk_tensor_winograd_pack_weights(const float *w, float *dst, int Cin, int Cout)
{
    static const float G[4][3] = {{1.f, 0.f, 0.f}, {.5f, .5f, .5f}, {.5f, -.5f, .5f}, {0.f, 0.f, 1.f}};
    if (!w || !dst || Cin <= 0 || Cout <= 0) return -1;
    for (int c = 0; c < Cin; c++)
        for (int o = 0; o < Cout; o++) {
            const float *g = w + ((size_t)c * Cout + o) * 9;
            float t[4][3];
            for (int i = 0; i < 4; i++)
                for (int j = 0; j < 3; j++) t[i][j] = G[i][0] * g[0 * 3 + j] + G[i][1] * g[1 * 3 + j] + G[i][2] * g[2 * 3 + j];
            for (int i = 0; i < 4; i++)
                for (int j = 0; j < 4; j++)
                    dst[((size_t)(i * 4 + j) * Cout + o) * Cin + c] = t[i][0] * G[j][0] + t[i][1] * G[j][1] + t[i][2] * G[j][2];
        }
    return 0;
}

/* the flat GEMM of one chunk: A = V [P*Tp][Kw], B = U [P*Cout][Kw], D = M [P*Tp][Cout]; P transform positions stacked on M.
 * x3: rows are Kw = 2*Cin wide, (high | low) halves, and the K loop makes the three passes hi x hi, hi x lo, lo x hi */
static int twino_gemm_plan(dRk_TensorConvPlan *pl, const float *V, const float *U, float *M, size_t Tp, int P, int x3, int Cin, int Cout,
                           int *status, int sms)
{
    PFN_encodeTiled enc = get_encode();
    if (!enc) return -1;
    memset(pl, 0, sizeof *pl);
    UmmaParams &p = pl->p;
    p.n = 1; p.W = 1; p.H = 1; p.Cin = Cin; p.Cout = Cout;
    p.CinPad = (Cin + BK - 1) / BK * BK;
    p.taps = 1; p.kw = 1; p.pad = 0;
    p.x3cat = x3 ? Cin / BK : 0;
    p.kslabs = x3 ? 3 * p.x3cat : p.CinPad / BK;
    p.S = 0; p.TW = BM; p.TH = 1; p.tiles_x = p.tiles_y = 1;
    p.total_sub = (long long)((size_t)P * Tp);
    p.m_tiles = (int)((size_t)P * Tp / BM);
    p.bias = NULL; p.out = M; p.ldo = Cout; p.coff = 0; p.act = 0; p.pool = 0; p.status = status;
    p.ksplit = 1; p.kper = p.kslabs; p.split_stride = 0;
    p.bgroup_tiles = (int)(Tp / BM); p.bgroup_rows = Cout;
    pl->in = V; pl->wT = U; pl->sms = sms;
    pl->BN = pick_bn(Cout, p.m_tiles, sms);
    p.n_tiles = (Cout + pl->BN - 1) / pl->BN;
    p.stage_tx = A_STAGE_BYTES + pl->BN * BK * 4;
    const cuuint64_t Kw = (cuuint64_t)(x3 ? 2 * Cin : Cin);
    const CUtensorMapDataType dt = x3 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32;   /* the halves are used bit for bit */
    const cuuint32_t ones[2] = {1, 1};
    const cuuint64_t adims[2] = {Kw, (cuuint64_t)P * Tp}, str[1] = {Kw * 4};
    const cuuint32_t abox[2] = {BK, BM};
    CUresult r = enc(&pl->mapA, dt, 2, (void *)V, adims, str, abox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    const cuuint64_t bdims[2] = {Kw, (cuuint64_t)P * Cout};
    const cuuint32_t bbox[2] = {BK, (cuuint32_t)pl->BN};
    if (r == CUDA_SUCCESS)
        r = enc(&pl->mapB, dt, 2, (void *)U, bdims, str, bbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "tensor winograd plan: tensor map rejected (%d)\n", (int)r); return -1; }
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    pl->grid = (int)(tiles < sms ? tiles : sms);
    return 0;
}

extern "C" dRk_TensorWinogradPlan *dRk_tensor_winograd_plan(const float *in, const float *U, const float *bias, float *out, float *scratch,
                                                            int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff, int *status)
{
    if (n <= 0 || !scratch || !dRk_tensor_winograd_supported(W, H, Cin, Cout)) return NULL;
    if (ldi < Cin || ldo < coff + Cout || ((uintptr_t)scratch % 16) || ((uintptr_t)U % 16)) return NULL;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dRk_TensorWinogradPlan *wp = (dRk_TensorWinogradPlan *)calloc(1, sizeof(dRk_TensorWinogradPlan));
    if (!wp) return NULL;
    wp->in = in; wp->bias = bias; wp->out = out; wp->n = n; wp->W = W; wp->H = H; wp->Cin = Cin; wp->Cout = Cout;
    wp->act = act; wp->ldi = ldi; wp->ldo = ldo; wp->coff = coff;
    const int chunk = twino_chunk(n, W, H, Cin, Cout);
    wp->imgs[0] = chunk; wp->nfull = n / chunk; wp->imgs[1] = n - wp->nfull * chunk;
    wp->V = scratch;
    wp->M = scratch + 16 * twino_pad(twino_tiles(W, H) * chunk) * (size_t)Cin;
    for (int i = 0; i < 2; i++) {
        if (wp->imgs[i] == 0) continue;
        wp->T[i] = twino_tiles(W, H) * wp->imgs[i];
        wp->Tp[i] = twino_pad(wp->T[i]);
        if (twino_gemm_plan(&wp->gemm[i], wp->V, U, wp->M, wp->Tp[i], 16, 0, Cin, Cout, status, sms) != 0) { free(wp); return NULL; }
    }
    return wp;
}

/*
 * Winograd F(4x4,3x3) with FP32-accurate products on the tensor cores: the transforms of k_winograd.cu in FP32 around ONE launch of
 * the flat GEMM over the 36 transform positions, every product evaluated as hi x hi + hi x lo + lo x hi of TF32 halves (the input
 * transform writes V as (high | low) rows, the filters are packed the same way).  A quarter of the direct sum's multiplications,
 * three MMAs each: 0.75 MMA per direct multiplication where the direct three-pass kernel spends 3.  The algorithm of
 * conv2dwinograd2 (Kernels/dR_winograd2.cl:23-254) at the larger tile size, in the FP32 class's error bound.
 */
static size_t twino4_tiles(int W, int H) { return (size_t)((W + 3) / 4) * ((H + 3) / 4); }
static int twino4_chunk(int n, int W, int H, int Cin, int Cout)
{
    const size_t per = 36 * twino4_tiles(W, H) * (size_t)(2 * Cin + Cout);
    size_t c = (TWINO_SCRATCH_CAP - 36 * (size_t)BM * (2 * Cin + Cout)) / per;
    if (c < 1) c = 1;
    if (c > (size_t)n) c = (size_t)n;
    const size_t chunks = ((size_t)n + c - 1) / c;          /* equal chunks rather than full ones and a short last one */
    c = ((size_t)n + chunks - 1) / chunks;
    return (int)c;
}

extern "C" int dRk_tensor_winograd4_x3_supported(int W, int H, int Cin, int Cout)
{
    return dRk_tensor_conv_supported(W, H, Cin, Cout, 3, 3) && Cin >= BK && Cin % BK == 0 && Cin <= 1024 &&
           twino_pad(twino4_tiles(W, H)) * 36 <= 0x7fffffffull / 2;
}

extern "C" size_t dRk_tensor_winograd4_x3_scratch_floats(int n, int W, int H, int Cin, int Cout)
{
    if (n <= 0 || !dRk_tensor_winograd4_x3_supported(W, H, Cin, Cout)) return 0;
    return 36 * twino_pad(twino4_tiles(W, H) * twino4_chunk(n, W, H, Cin, Cout)) * (size_t)(2 * Cin + Cout);
}

extern "C" size_t dRk_tensor_winograd4_x3_packed_floats(int Cin, int Cout) { return (size_t)36 * Cout * 2 * Cin; }

/* U = G g G^T in double (G of F(4x4,3x3)), stored [36][Cout][2*Cin]: the upper 19 bits of the FP32 value, then what is left of the
 * double value.  w is the reference's [Cin][Cout][3][3] filter array. */
extern "C" int dRk_tensor_winograd4_x3_pack_weights(const float *w, float *dst, int Cin, int Cout)
{
    if (!w || !dst || Cin <= 0 || Cout <= 0) return -1;
    static const double G[6][3] = {{1.0 / 4, 0, 0}, {-1.0 / 6, -1.0 / 6, -1.0 / 6}, {-1.0 / 6, 1.0 / 6, -1.0 / 6},
                                   {1.0 / 24, 1.0 / 12, 1.0 / 6}, {1.0 / 24, -1.0 / 12, 1.0 / 6}, {0, 0, 1}};
    for (int c = 0; c < Cin; c++)
        for (int o = 0; o < Cout; o++) {
            const float *g = w + ((size_t)c * Cout + o) * 9;
            double t[6][3];
            for (int i = 0; i < 6; i++)
                for (int j = 0; j < 3; j++) t[i][j] = G[i][0] * g[0 * 3 + j] + G[i][1] * g[1 * 3 + j] + G[i][2] * g[2 * 3 + j];
            for (int i = 0; i < 6; i++)
                for (int j = 0; j < 6; j++) {
                    const double u = t[i][0] * G[j][0] + t[i][1] * G[j][1] + t[i][2] * G[j][2];
                    const float uf = (float)u;
                    uint32_t bits;
                    memcpy(&bits, &uf, 4);
                    bits &= 0xffffe000u;
                    float hi;
                    memcpy(&hi, &bits, 4);
                    float *row = dst + ((size_t)(i * 6 + j) * Cout + o) * (2 * (size_t)Cin);
                    row[c] = hi;
                    row[Cin + c] = (float)(u - (double)hi);
                }
        }
    return 0;
}

extern "C" dRk_TensorWinogradPlan *dRk_tensor_winograd4_x3_plan(const float *in, const float *U2, const float *bias, float *out, float *scratch,
                                                                int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff,
                                                                int pool, int *status)
{
    if (n <= 0 || !scratch || !dRk_tensor_winograd4_x3_supported(W, H, Cin, Cout)) return NULL;
    if (ldi < Cin || ldo < coff + Cout || ((uintptr_t)scratch % 16) || ((uintptr_t)U2 % 16)) return NULL;
    if (pool && (pool != 1 || (W & 1) || (H & 1))) return NULL;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dRk_TensorWinogradPlan *wp = (dRk_TensorWinogradPlan *)calloc(1, sizeof(dRk_TensorWinogradPlan));
    if (!wp) return NULL;
    wp->in = in; wp->bias = bias; wp->out = out; wp->n = n; wp->W = W; wp->H = H; wp->Cin = Cin; wp->Cout = Cout;
    wp->act = act; wp->ldi = ldi; wp->ldo = ldo; wp->coff = coff; wp->f4x3 = 1; wp->pool = pool;
    const int chunk = twino4_chunk(n, W, H, Cin, Cout);
    wp->imgs[0] = chunk; wp->nfull = n / chunk; wp->imgs[1] = n - wp->nfull * chunk;
    wp->V = scratch;
    wp->M = scratch + 36 * twino_pad(twino4_tiles(W, H) * chunk) * (size_t)(2 * Cin);
    for (int i = 0; i < 2; i++) {
        if (wp->imgs[i] == 0) continue;
        wp->T[i] = twino4_tiles(W, H) * wp->imgs[i];
        wp->Tp[i] = twino_pad(wp->T[i]);
        if (twino_gemm_plan(&wp->gemm[i], wp->V, U2, wp->M, wp->Tp[i], 36, 1, Cin, Cout, status, sms) != 0) { free(wp); return NULL; }
    }
    return wp;
}

extern "C" int dRk_tensor_winograd_run(dRk_stream stream, dRk_TensorWinogradPlan *wp)
{
    if (!wp) return -1;
    cudaStream_t st = drk_stream(stream);
    int b0 = 0;
    for (int c = 0; c < wp->nfull + (wp->imgs[1] ? 1 : 0); c++) {
        const int i = c < wp->nfull ? 0 : 1;
        const float *src = wp->in + (size_t)b0 * wp->H * wp->W * wp->ldi;
        float *dst = wp->out + (size_t)b0 * (wp->pool ? (wp->H / 2) * (wp->W / 2) : wp->H * wp->W) * wp->ldo;
        int rc = wp->f4x3 ? drk_wino4_input_launch(st, src, wp->V, wp->W, wp->H, wp->Cin, wp->ldi, wp->T[i], wp->Tp[i], 1)
                          : drk_wino_input_launch(st, src, wp->V, wp->imgs[i], wp->W, wp->H, wp->Cin, wp->ldi, wp->T[i], wp->Tp[i]);
        if (rc) return rc;
        dRk_TensorConvPlan *g = &wp->gemm[i];
        switch (g->BN) {
        case 256: rc = launch_umma<256>(st, g); break;
        case 128: rc = launch_umma<128>(st, g); break;
        default: rc = launch_umma<64>(st, g); break;
        }
        if (rc) return rc;
        rc = wp->f4x3 ? drk_wino4_output_launch(st, wp->M, wp->bias, dst, wp->W, wp->H, wp->Cout, wp->ldo, wp->coff, wp->T[i], wp->Tp[i], wp->act, wp->pool)
                      : drk_wino_output_launch(st, wp->M, wp->bias, dst, wp->W, wp->H, wp->Cout, wp->ldo, wp->coff, wp->T[i], wp->Tp[i], wp->act);
        if (rc) return rc;
        b0 += wp->imgs[i];
    }
    return 0;
}

extern "C" void dRk_tensor_winograd_free(dRk_TensorWinogradPlan *wp) { free(wp); }
