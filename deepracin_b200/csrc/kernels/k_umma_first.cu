/*
 * Tensor-core 3x3 stride-1 convolution for very few input channels (Cin <= 4: the RGB first layer of
 * VGG / SqueezeNet) in TF32 mode.  With K = 9*Cin <= 36 there is nothing for TMA to tile (a pixel is
 * 12 bytes), so the im2col operand is built in shared memory by producer warps:
 *     D[o][pixel] = sum_k Wt[o][k] * P[pixel][k],   k = (ky*3 + kx)*Cin + c,
 * M = output channels (<= 128, rows past Cout are zeros), N = 256 consecutive pixels of the flattened
 * (image, y, x) index, K padded with zeros to whole 128-byte swizzle rows.  The filter tile is written once
 * per CTA; every tile of pixels then costs ceil(9*Cin/8) tcgen05.mma instructions, so the layer is bound by
 * writing its output: algorithmic bytes = n*H*W*(Cin + Cout)*4.
 * Replaces the reference's Winograd launch for such layers (src/dR_nodes_conv2d.c:36-53 sends every 3x3
 * stride-1 filter to conv2dwinograd2, Kernels/dR_winograd2.cl:23-254).  A 2x2/2 max or average pooling node
 * behind the layer (src/dR_nodes_pooling.c:138-183) can be evaluated in the epilogue, and a Slice -> scalar op ->
 * Concat preamble in front of it by the gather (see FirstInMap).
 *
 * Persistent CTAs, 17 warps: warp 0 issues the MMAs and owns TMEM; warps 1-8 are the epilogue (a lane owns an
 * output channel, two warps share each 32-lane quarter of TMEM and split the 256 pixel columns; a store
 * instruction of a warp writes the 128 contiguous bytes of 32 channels of one pixel); warps 9-16 gather
 * patches: a thread reads the 9*Cin inputs of a pixel (zeros outside the image), rounds them to TF32 and
 * writes the pixel's row in the 128-byte-swizzle pattern the MMA descriptor expects, then makes the writes
 * visible to the async proxy and arrives on the stage's mbarrier.  Two TMEM accumulators overlap the epilogue
 * of a tile with the gather and MMAs of the next.  Every wait is bounded; on expiry the CTA flags an abort,
 * writes a code to `status`, and all roles leave (no asynchronous copies are ever in flight here).
 */
#include <stdio.h>
#include <string.h>
#include "k_common.cuh"
#include "k_umma.cuh"

#define FIRST_N 256
#define FIRST_EPI_WARPS 8
#define FIRST_PROD_WARPS 8
#define FIRST_PROD_THREADS (FIRST_PROD_WARPS * 32)
#define FIRST_THREADS ((1 + FIRST_EPI_WARPS + FIRST_PROD_WARPS) * 32)

/* G = pixel groups stacked on the M axis: with Cout <= 64 rows 0-63 hold the channels of pixels [0,256) of a tile and rows
 * 64-127 the channels of pixels [256,512), through block-diagonal filters (group g multiplies only the K slabs of group g),
 * so that all four 32-lane quarters of TMEM -- hence all epilogue warps -- carry output. */
template <int CIN, int G>
struct FirstCfg {
    static constexpr int K = 9 * CIN;
    /* two more K columns carry the bias: every patch row holds 1.0 there and the filter row the bias split into a TF32 high part
       and the TF32 of the remainder (exact to 2^-21 of the bias), so the accumulator leaves the MMA with the bias added and the
       epilogue -- which is what bounds this kernel -- saves an addition per output.  They fit the zero padding of the last slab. */
    static constexpr int KB = K + 2;
    static constexpr int KS = (KB + BK - 1) / BK;                  /* 128-byte slabs per pixel patch */
    static constexpr int NMMA = (KB + 7) / 8;                      /* MMAs (K = 8) per group */
    static constexpr int CP = BM / G;                              /* rows (channels) per group */
    static constexpr int SLABS = G * KS;
    static constexpr int A_BYTES = SLABS * BM * BK * 4;
    static constexpr int B_STAGE = SLABS * FIRST_N * BK * 4;
    static constexpr int NB = B_STAGE <= 32 * 1024 ? 3 : 2;
    static constexpr int SMEM_BYTES = A_BYTES + NB * B_STAGE + 1024 + 256;
};

/* Optional affine channel map applied while gathering: input channel j of the convolution is channel ch[j] of the source
 * pixel times scale[j] plus shift[j] (zero padding stays zero), ch a permutation of 0..Cin-1.  Evaluates a Slice -> scalar
 * op -> Concat preamble (mean subtraction, channel reordering) inside the first layer instead of in a kernel of its own.
 * The gather keeps the source's channel order (compile-time load offsets: run-time offsets made it 1.5x slower) and the
 * permutation goes into the filter tile's K columns, built once per CTA: inv[c] = the convolution channel that reads
 * source channel c; scale and shift are stored per source channel. */
struct FirstInMap {
    int use;
    int inv[4];
    float scale[4], shift[4];
};

__device__ __forceinline__ uint32_t to_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

/* byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled K-major slab */
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

/* stores 32 consecutive pixels of one channel: activation clamp (the bias came through the MMA), pixel stride ldo */
__device__ __forceinline__ float *store32(float *optr, const uint32_t (&r)[32], float lo, float hi, size_t ldo, long long left, bool chok)
{
    if (chok) {
        if (left >= 32) {
#pragma unroll
            for (int j = 0; j < 32; j++) optr[j * ldo] = fminf(fmaxf(__uint_as_float(r[j]), lo), hi);
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (j < left) optr[j * ldo] = fminf(fmaxf(__uint_as_float(r[j]), lo), hi);
        }
    }
    return optr + 32 * ldo;
}

template <int CIN, int G, bool MAPPED>
__global__ void __launch_bounds__(FIRST_THREADS, 1)
k_umma_conv_first(const float *__restrict__ in, const float *__restrict__ wT, const float *__restrict__ bias, float *__restrict__ out,
                  int n, int W, int H, int Cout, int act, int ldi, int ldo, int coff, int pool, int *status, const FirstInMap map)
{
    using C = FirstCfg<CIN, G>;
    constexpr int TILE_PX = G * FIRST_N;
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t a_base = base, b_base = base + C::A_BYTES;
    const uint32_t bars = b_base + C::NB * C::B_STAGE;
    constexpr int NBARS = 2 * C::NB + 5;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + C::A_BYTES + C::NB * C::B_STAGE + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto bfull = [&](int s) { return bars + 8u * s; };
    auto bempty = [&](int s) { return bars + 8u * (C::NB + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * C::NB + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * C::NB + 2 + a); };
    const uint32_t drain_bar = bars + 8u * (2 * C::NB + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total_px = (long long)n * H * W;
    /* pooled mode (G = 2): a column is position f of the flattened (image, row pair, x) index; group 0 computes the pixel
       of row 2j, group 1 the pixel below it, and pooled pixel f/2 takes the four values of columns f, f+1 of both groups.
       The accumulator rows are then ordered so that both groups of a channel sit in one 32-lane quarter of TMEM, 16 lanes
       apart (row = 32*(ch/16) + 16*group + ch%16): the vertical half of the window is one warp shuffle. */
    const long long total_f = pool ? total_px / 2 : 0;
    const int total_tiles = pool ? (int)((total_f + FIRST_N - 1) / FIRST_N) : (int)((total_px + TILE_PX - 1) / TILE_PX);
    /* which 32-lane quarters of TMEM hold output channels: quarter q covers rows 32q..32q+31, row r = group*CP + channel */
    int active_quarters = 0;
    for (int q = 0; q < 4; q++) active_quarters += ((G == 2 && pool) ? q * 16 : (q * 32) % C::CP) < Cout ? 1 : 0;
    constexpr int TMEM_COLS = 2 * FIRST_N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NB; s++) { mbar_init(bfull(s), FIRST_PROD_THREADS); mbar_init(bempty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * active_quarters); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    /* filter tile: [128 rows][SLABS*32] TF32, block diagonal over the groups, zeros past Cout and past K */
    for (int i = threadIdx.x; i < BM * C::SLABS * 8; i += FIRST_THREADS) {
        const int chunk_all = i % (C::SLABS * 8), row = i / (C::SLABS * 8);
        const int slab = chunk_all >> 3, chunk = chunk_all & 7;
        const int grp = slab / C::KS, ks = slab - grp * C::KS;
        int ch;                                                     /* the channel row `row` computes for group `grp`, or -1 */
        if (G == 2 && pool) ch = ((row >> 4) & 1) == grp ? (row >> 5) * 16 + (row & 15) : -1;
        else ch = (row >= grp * C::CP && row < (grp + 1) * C::CP) ? row - grp * C::CP : -1;
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = ks * BK + chunk * 4 + e;
            int kw = k;                                             /* column of the packed filters this K position multiplies */
            if (MAPPED && k < C::K) { const int tap = k / CIN; kw = tap * CIN + map.inv[k - tap * CIN]; }
            float wv = 0.0f;
            if (ch >= 0 && ch < Cout) {
                if (k < C::K) wv = __ldg(wT + (size_t)ch * C::K + kw);
                else if (k < C::KB && bias) {
                    const float bfull = __ldg(bias + ch);
                    const float bhi = __uint_as_float(to_tf32(bfull));
                    wv = k == C::K ? bhi : bfull - bhi;
                }
            }
            /* 2x2 average pooling: the 1/4 goes into the filters and the bias (a power of two: exact, and it commutes with the clamp) */
            v[e] = to_tf32(pool == 2 ? 0.25f * wv : wv);
        }
        *reinterpret_cast<uint4 *>(gen + slab * (BM * BK * 4) + swz(row, chunk)) = make_uint4(v[0], v[1], v[2], v[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    drk_dep_wait();                 /* the filter tile and set-up above overlap the previous kernel; its outputs are visible from here on */

    if (warp == 0) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(FIRST_N);
            int bs = 0;
            uint32_t bph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, status, 2)) { ok = false; break; }
                if (!mbar_wait(bfull(bs), bph, abort_flag, status, 3)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * FIRST_N);
#pragma unroll
                for (int grp = 0; grp < G; grp++)
#pragma unroll
                    for (int i = 0; i < C::NMMA; i++) {
                        const int slab = grp * C::KS + (i >> 2), j = i & 3;
                        const uint64_t adesc = make_smem_desc(a_base + slab * (BM * BK * 4));
                        const uint64_t bdesc = make_smem_desc(b_base + bs * C::B_STAGE + slab * (FIRST_N * BK * 4));
                        umma_tf32(d_tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (grp | i) ? 1u : 0u);
                    }
                umma_commit(bempty(bs));
                umma_commit(tfull_bar(acc));
                if (++bs == C::NB) { bs = 0; bph ^= 1u; }
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else if (warp <= FIRST_EPI_WARPS) {
        const int quarter = warp & 3, half = (warp - 1) >> 2;
        const int row = quarter * 32 + lane;
        const bool pooled = G == 2 && pool;
        const int grp = pooled ? (lane >> 4) : row / C::CP;
        const int ch = pooled ? quarter * 16 + (lane & 15) : row - grp * C::CP;
        if ((pooled ? quarter * 16 : (quarter * 32) % C::CP) < Cout) {
            const bool chok = ch < Cout;
            const float lo = act ? 0.0f : -INFINITY, hi = act ? FLT_MAX : INFINITY;       /* the bias is already in the accumulator */
            int it = 0;
            if (pooled) {
                for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, it++) {
                    const int acc = it & 1;
                    const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                    if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, status, 4)) break;
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * FIRST_N + half * (FIRST_N / 2));
                    const long long f0 = (long long)t * FIRST_N + half * (FIRST_N / 2);
                    /* pooled pixels are consecutive: (f0 + c0)/2 + k.  A lane holds the horizontal halves of its own row (group 0:
                       row 2j, group 1: row 2j+1) for all 16 of them; of every two neighbours the lane of group 0 finishes the
                       even one and the lane of group 1 the odd one, so ONE shuffle per two pixels hands each lane the half it
                       lacks, and every lane stores only what it finished. */
                    float *optr = out + (size_t)((f0 >> 1) + grp) * ldo + coff + (chok ? ch : 0);
                    long long left = (total_f >> 1) - (f0 >> 1) - grp;
#pragma unroll 1
                    for (int c0 = 0; c0 < FIRST_N / 2; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(taddr + (uint32_t)c0, r);
#pragma unroll
                        for (int k = 0; k < 16; k += 2) {
                            const float a0 = fminf(fmaxf(__uint_as_float(r[2 * k]), lo), hi), b0 = fminf(fmaxf(__uint_as_float(r[2 * k + 1]), lo), hi);
                            const float a1 = fminf(fmaxf(__uint_as_float(r[2 * k + 2]), lo), hi), b1 = fminf(fmaxf(__uint_as_float(r[2 * k + 3]), lo), hi);
                            const float h0 = pool == 2 ? a0 + b0 : fmaxf(a0, b0), h1 = pool == 2 ? a1 + b1 : fmaxf(a1, b1);
                            const float got = __shfl_xor_sync(0xffffffffu, grp ? h0 : h1, 16);
                            const float mine = grp ? h1 : h0;
                            const float o = pool == 2 ? mine + got : fmaxf(mine, got);
                            if (chok && k < left) optr[(size_t)k * ldo] = o;
                        }
                        optr += 16 * (size_t)ldo;
                        left -= 16;
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(acc));
                }
            } else
            for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, status, 4)) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * FIRST_N + half * (FIRST_N / 2));
                const long long g0 = (long long)t * TILE_PX + grp * FIRST_N + half * (FIRST_N / 2);
                float *optr = out + (size_t)g0 * ldo + coff + (chok ? ch : 0);
                /* four 32-column chunks, the TMEM load of the next chunk in flight while this one is stored */
                uint32_t r0[32], r1[32];
                tmem_ld32_nowait(taddr, r0);
                tmem_ld_wait();
                tmem_ld32_nowait(taddr + 32u, r1);
                optr = store32(optr, r0, lo, hi, (size_t)ldo, total_px - g0, chok);
                tmem_ld_wait();
                tmem_ld32_nowait(taddr + 64u, r0);
                optr = store32(optr, r1, lo, hi, (size_t)ldo, total_px - g0 - 32, chok);
                tmem_ld_wait();
                tmem_ld32_nowait(taddr + 96u, r1);
                optr = store32(optr, r0, lo, hi, (size_t)ldo, total_px - g0 - 64, chok);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));         /* the accumulator is in registers: the MMAs of the tile after next may start */
                store32(optr, r1, lo, hi, (size_t)ldo, total_px - g0 - 96, chok);
            }
        }
    } else {
        const int col = threadIdx.x - (FIRST_EPI_WARPS + 1) * 32;           /* 0..255: the B row this thread fills */
        const bool small = total_px < 0x7fffffffll;
        int bs = 0;
        uint32_t bph = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            if (!mbar_wait(bempty(bs), bph ^ 1u, abort_flag, status, 1)) break;
            uint8_t *stage = gen + C::A_BYTES + bs * C::B_STAGE;
            uint32_t v[G][C::KS * BK];
#pragma unroll
            for (int grp = 0; grp < G; grp++) {
#pragma unroll
                for (int k = 0; k < C::KS * BK; k++) v[grp][k] = 0u;
                long long g;
                int x, y;
                bool inside;
                if (G == 2 && pool) {
                    const long long f = (long long)t * FIRST_N + col;
                    inside = f < total_f;
                    const int hh = H >> 1;
                    if (small) {                                    /* 32-bit divisions: a 64-bit one costs as much as the rest of the gather */
                        const unsigned fu = (unsigned)f, jq = fu / (unsigned)W, img = jq / (unsigned)hh;
                        x = (int)(fu - jq * (unsigned)W);
                        y = 2 * (int)(jq - img * (unsigned)hh) + grp;
                        g = ((long long)img * H + y) * W + x;
                    } else {
                        const long long jq = f / W;
                        x = (int)(f - jq * W);
                        const long long img = jq / hh;
                        y = 2 * (int)(jq - img * hh) + grp;
                        g = (img * H + y) * W + x;
                    }
                } else {
                    g = (long long)t * TILE_PX + grp * FIRST_N + col;
                    inside = g < total_px;
                    if (small) {
                        const unsigned gu = (unsigned)g, q = gu / (unsigned)W;
                        x = (int)(gu - q * (unsigned)W);
                        y = (int)(q % (unsigned)H);
                    } else {
                        const long long q = g / W;
                        x = (int)(g - q * W);
                        y = (int)(q % H);
                    }
                }
                if (inside) {
                    v[grp][C::K] = v[grp][C::K + 1] = 0x3f800000u;           /* 1.0 in the two bias columns */
                    const float *pix = in + (size_t)g * ldi;                 /* the centre pixel */
#pragma unroll
                    for (int ky = 0; ky < 3; ky++) {
                        const int iy = y + ky - 1;
                        const bool yok = iy >= 0 && iy < H;
#pragma unroll
                        for (int kx = 0; kx < 3; kx++) {
                            const int ix = x + kx - 1;
                            const bool pok = yok && ix >= 0 && ix < W;
                            const float *p = pix + ((ky - 1) * W + (kx - 1)) * ldi;
#pragma unroll
                            for (int c = 0; c < CIN; c++) {
                                float t = pok ? __ldg(p + c) : 0.0f;
                                if (MAPPED) t = pok ? fmaf(t, map.scale[c], map.shift[c]) : 0.0f;
                                v[grp][(ky * 3 + kx) * CIN + c] = __float_as_uint(t);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int grp = 0; grp < G; grp++)
#pragma unroll
                for (int ck = 0; ck < C::KS * 8; ck++) {
                    const int slab = grp * C::KS + (ck >> 3), chunk = ck & 7;
                    uint4 o;
                    if (ck * 4 < C::KB) o = make_uint4(to_tf32(__uint_as_float(v[grp][ck * 4])), to_tf32(__uint_as_float(v[grp][ck * 4 + 1])),
                                                      to_tf32(__uint_as_float(v[grp][ck * 4 + 2])), to_tf32(__uint_as_float(v[grp][ck * 4 + 3])));
                    else o = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4 *>(stage + slab * (FIRST_N * BK * 4) + swz(col, chunk)) = o;
                }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bfull(bs));
            if (++bs == C::NB) { bs = 0; bph ^= 1u; }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int CIN, int G, bool MAPPED>
static int launch_first_m(cudaStream_t st, const float *in, const float *wT, const float *bias, float *out, int n, int W, int H, int Cout,
                        int act, int ldi, int ldo, int coff, int pool, int *status, int sms, const FirstInMap &map)
{
    static bool attr_done[64];                      /* the opt-in shared-memory size is a per-device function attribute */
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_umma_conv_first<CIN, G, MAPPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, FirstCfg<CIN, G>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    if (pool && G != 2) return -1;
    const long long tiles = pool ? ((long long)n * (H / 2) * W + FIRST_N - 1) / FIRST_N : ((long long)n * H * W + G * FIRST_N - 1) / (G * FIRST_N);
    if (tiles <= 0 || tiles > 0x7fffffffll) return -1;
    const int grid = (int)(tiles < sms ? tiles : sms);
    drk_launch_dep(k_umma_conv_first<CIN, G, MAPPED>, dim3(grid), dim3(FIRST_THREADS), FirstCfg<CIN, G>::SMEM_BYTES, st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, map);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

template <int CIN, int G>
static int launch_first(cudaStream_t st, const float *in, const float *wT, const float *bias, float *out, int n, int W, int H, int Cout,
                        int act, int ldi, int ldo, int coff, int pool, int *status, int sms, const FirstInMap &map)
{
    return map.use ? launch_first_m<CIN, G, true>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map)
                   : launch_first_m<CIN, G, false>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map);
}

/* 1 if this kernel takes the layer shape */
int drk_umma_first_supported(int Cin, int Cout, int kw, int kh)
{
    return kw == 3 && kh == 3 && Cin >= 1 && Cin <= 4 && Cout >= 16 && Cout <= BM && Cout % 4 == 0;
}

/* 1 if the 2x2/2 pooling (max or average) that follows the layer can be evaluated in this kernel's epilogue */
int drk_umma_first_can_pool(int W, int H, int Cin, int Cout)
{
    return Cin <= 3 && Cout <= 64 && (W % 2) == 0 && (H % 2) == 0;
}

/* wT: [Cout][9*Cin] with k = (ky*3 + kx)*Cin + c; in: N-HWC with pixel stride ldi; pool: 0 none, 1 max 2x2/2, 2 average 2x2/2
 * (`out` is then the (W/2) x (H/2) pooled tensor) */
int drk_umma_first_launch(cudaStream_t st, const float *in, const float *wT, const float *bias, float *out, int n, int W, int H, int Cin,
                          int Cout, int act, int ldi, int ldo, int coff, int pool, int *status, int sms, const int *map_ch, const float *map_scale,
                          const float *map_shift)
{
    FirstInMap map;
    memset(&map, 0, sizeof map);
    if (map_ch) {
        map.use = 1;
        for (int j = 0; j < Cin && j < 4; j++) {
            const int c = map_ch[j];
            if (c < 0 || c >= Cin) return -1;
            map.inv[c] = j; map.scale[c] = map_scale[j]; map.shift[c] = map_shift[j];
        }
    }
    if (pool && !drk_umma_first_can_pool(W, H, Cin, Cout)) return -1;
    const bool two = Cout <= 64;                     /* two pixel groups on the M axis */
    switch (Cin) {
    case 1: return two ? launch_first<1, 2>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map)
                       : launch_first<1, 1>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map);
    case 2: return two ? launch_first<2, 2>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map)
                       : launch_first<2, 1>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map);
    case 3: return two ? launch_first<3, 2>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map)
                       : launch_first<3, 1>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map);
    case 4: return launch_first<4, 1>(st, in, wT, bias, out, n, W, H, Cout, act, ldi, ldo, coff, pool, status, sms, map);
    }
    return -1;
}
