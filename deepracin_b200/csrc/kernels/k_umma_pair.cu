/*
 * Tensor-core 3x3 stride-1 convolution for layers with at most 64 output channels (VGG conv1_2,
 * SqueezeNet's 64-channel expand layers) in TF32 mode.  A tcgen05.mma with N = 256 occupies the tensor pipe for
 * 128 clocks whether M is 64 or 128 (microbenchmark), so the transposed product of k_umma_conv_swap (M = channels, N = 256 pixels) wastes half
 * of every instruction when Cout <= 64.  Here the two halves of M hold the same channels for two
 * vertically adjacent output rows:
 *     rows  0..63  : out[o][2j  ][x]      rows 64..127 : out[o][2j+1][x]
 * Both rows read input rows 2j-1 .. 2j+2; input row 2j-1+i (i = 0..3) is tap ky = i of the upper output row
 * and tap ky = i-1 of the lower one.  With the input split by row parity into an even and an odd plane
 * (two TMA maps over the same N-HWC tensor, row stride doubled), the pixels of input row 2j-1+i for
 * j = 0..15 are consecutive rows of one plane's haloed block, i.e. one B operand read through a shifted
 * descriptor start as in the halo kernels, and the filter tile of (i, kx) stacks W[ky=i][kx] over
 * W[ky=i-1][kx] (zeros where ky falls outside 0..2).  Twelve (i, kx) products per 32-channel slab cover what
 * takes eighteen in the unpaired kernel: 1.5x fewer MMA instructions per output pixel.
 * Replaces conv2dwinograd2 (Kernels/dR_winograd2.cl:23-254) for these layers; bound: tensor pipe;
 * algorithmic FLOPs = 2*9*Cin*Cout*n*H*W.
 *
 * A tile is 14 x 32 output pixels (N = 256 columns = 16 row pairs x 16-pixel pitch, 14 valid).  6 warps:
 * warp 0 TMA producer (two plane blocks per slab through a ring of three slots, twelve filter tiles per slab
 * through a ring of seven, issued in the order the MMA issuer consumes them),
 * warp 1 MMA issuer and TMEM owner, warps 2-5 epilogue: quarters 0/1 of TMEM hold the upper rows, 2/3 the
 * lower rows of the same channels.  The fused 2x2 max pooling needs both: the lower-row warp passes its
 * horizontal maxima to the upper-row warp of the same channels through a small double-buffered
 * shared-memory exchange guarded by mbarriers.  Every wait is bounded; on expiry the CTA flags an abort,
 * reports a code through `status`, drains its in-flight copies, frees TMEM and returns.
 *
 * X3 = true: FP32-accurate evaluation ("3xTF32", as k_umma_conv_swap<true>): every plane is multiplied three times into the
 * same accumulator -- by the filter tiles as loaded (the MMA reads their upper 19 bits), by the tiles of the filters' low
 * parts (mapWlo), and, with the plane's own low part x - hi(x) as the other operand, by the filter tiles again.  Four extra
 * warps write that low part into a buffer of its own while the first two passes run; the plane ring is one slot shorter to
 * make room for it.  Tensor maps are plain FLOAT32 in this mode.
 */
#include <stdio.h>
#include "k_common.cuh"
#include "k_umma.cuh"

#define PAIR_SPLIT_WARPS 4                              /* X3 mode only */
#define PAIR_THREADS(X3) (192 + ((X3) ? PAIR_SPLIT_WARPS * 32 : 0))
/* Two block geometries, chosen per layer (UmmaParams P, TW, TH = row pairs per tile, ncols = P * TH):
 *   P = 16, 14 valid pixels, 16 row pairs: N = 256, 14 x 32 output pixels per tile (0.875 of the columns are pixels);
 *   P = 30, 28 valid pixels,  8 row pairs: N = 240, 28 x 16 output pixels per tile (0.933). */
#define PAIR_N 256
#define PAIR_PLANE_SLOT (35 * 1024)                     /* 280 rows: (TH + 1) * P <= 272 loaded, taps of idle columns read a few rows further */
#define PAIR_NH 3                                       /* ring of plane slots: odd and even planes of a slab are separate stages (X3: two, the third slot holds the low part) */
#define PAIR_W_BYTES (BM * BK * 4)
#define PAIR_NW 7
#define PAIR_X_FLOATS (2 * 7 * 32)                      /* one exchange buffer: 2 pooled rows x 7 pooled pixels x 32 lanes */
#define PAIR_X_BYTES (2 * 2 * PAIR_X_FLOATS * 4)        /* two warp pairs x two buffers */
#define PAIR_SMEM (PAIR_NH * PAIR_PLANE_SLOT + PAIR_NW * PAIR_W_BYTES + PAIR_X_BYTES + 1024 + 512)

template <bool X3>
__global__ void __launch_bounds__(PAIR_THREADS(X3), 1)
k_umma_conv_pair(const __grid_constant__ CUtensorMap mapO, const __grid_constant__ CUtensorMap mapE, const __grid_constant__ CUtensorMap mapW,
                 const __grid_constant__ CUtensorMap mapWlo, const UmmaParams p)
{
    constexpr int NH = X3 ? PAIR_NH - 1 : PAIR_NH;      /* plane slots in the ring */
    constexpr int PASSES = X3 ? 3 : 1;
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t h_base = base, w_base = base + PAIR_NH * PAIR_PLANE_SLOT;
    const uint32_t x_off = PAIR_NH * PAIR_PLANE_SLOT + PAIR_NW * PAIR_W_BYTES;
    float *xbuf = reinterpret_cast<float *>(gen + x_off);
    const uint32_t bars = base + x_off + PAIR_X_BYTES;
    constexpr int NBARS = 2 * PAIR_NH + 2 * PAIR_NW + 4 + 8 + 1 + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + x_off + PAIR_X_BYTES + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto hfull = [&](int s) { return bars + 8u * s; };
    auto hempty = [&](int s) { return bars + 8u * (PAIR_NH + s); };
    auto wfull = [&](int s) { return bars + 8u * (2 * PAIR_NH + s); };
    auto wempty = [&](int s) { return bars + 8u * (2 * PAIR_NH + PAIR_NW + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 2 + a); };
    auto xfull = [&](int pr, int b) { return bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 4 + pr * 4 + b); };
    auto xempty = [&](int pr, int b) { return bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 4 + pr * 4 + 2 + b); };
    const uint32_t drain_bar = bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 4 + 8);
    const uint32_t xlo_full = bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 4 + 8 + 1);     /* X3: the low-part buffer holds the current plane's low parts */
    const uint32_t xlo_free = bars + 8u * (2 * PAIR_NH + 2 * PAIR_NW + 4 + 8 + 2);     /* X3: pass 3 of the previous plane has read it */
    const uint32_t xlo_base = h_base + NH * PAIR_PLANE_SLOT;                            /* X3: the ring's last slot */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles;
    const int per = p.tiles_x * p.tiles_y;
    constexpr int TMEM_COLS = 2 * PAIR_N;
    const uint32_t plane_bytes = (uint32_t)((p.TH + 1) * p.P * BK * 4);

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_NH; s++) { mbar_init(hfull(s), 1); mbar_init(hempty(s), 1); }
        for (int s = 0; s < PAIR_NW; s++) { mbar_init(wfull(s), 1); mbar_init(wempty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        for (int pr = 0; pr < 2; pr++)
            for (int b = 0; b < 2; b++) { mbar_init(xfull(pr, b), 1); mbar_init(xempty(pr, b), 1); }
        mbar_init(drain_bar, 1);
        mbar_init(xlo_full, PAIR_SPLIT_WARPS);
        mbar_init(xlo_free, 1);
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
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapO) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapE) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapW) : "memory");
            if (X3) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapWlo) : "memory");
            int hs = 0, ws = 0;
            uint32_t hph = 0, wph = 0;
            long long h_issued = 0, w_issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int img = t / per, rem = t - img * per;
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                const int j0 = tyi * p.TH;
                /* issue order = the MMA issuer's consumption order: odd plane, its six filter tiles, even plane, its six */
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    for (int half = 0; half < 2 && ok; half++) {
                        if (!mbar_wait(hempty(hs), hph ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
                        mbar_expect_tx(hfull(hs), plane_bytes);
                        /* odd plane rows j0-1 .. j0+15 (input rows 2j0-1, 2j0+1, ...), even plane rows j0 .. j0+16 */
                        if (half == 0) tma_load_4d(h_base + hs * PAIR_PLANE_SLOT, &mapO, ks * BK, txi * p.TW - 1, j0 - 1, img, hfull(hs));
                        else tma_load_4d(h_base + hs * PAIR_PLANE_SLOT, &mapE, ks * BK, txi * p.TW - 1, j0, img, hfull(hs));
                        h_issued++;
                        if (++hs == NH) { hs = 0; hph ^= 1u; }
                        for (int pq = 0; pq < 6 * PASSES && ok; pq++) {             /* X3: the filter tiles, their low parts, the filter tiles again */
                            const int q = pq % 6;
                            const int i = half + 2 * (q / 3), kx = q % 3;           /* input row 2j-1+i: i = 0, 2 live in the odd plane, 1, 3 in the even */
                            if (!mbar_wait(wempty(ws), wph ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                            mbar_expect_tx(wfull(ws), PAIR_W_BYTES);
                            tma_load_2d(w_base + ws * PAIR_W_BYTES, (X3 && pq / 6 == 1) ? &mapWlo : &mapW, (i * 3 + kx) * p.CinPad + ks * BK, 0, wfull(ws));
                            w_issued++;
                            if (++ws == PAIR_NW) { ws = 0; wph ^= 1u; }
                        }
                    }
                }
            }
            if (!ok) {
                long long pend = h_issued < NH ? h_issued : NH;
                int s = hs; uint32_t ph = hph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = NH - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(hfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
                pend = w_issued < PAIR_NW ? w_issued : PAIR_NW;
                s = ws; ph = wph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = PAIR_NW - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(wfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(p.ncols);
            int hs = 0, ws = 0;
            uint32_t hph = 0, wph = 0, xph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * PAIR_N);
                for (int ks = 0; ks < p.kslabs && ok; ks++) {
                    for (int half = 0; half < 2 && ok; half++) {
                        if (!mbar_wait(hfull(hs), hph, abort_flag, p.status, 6)) { ok = false; break; }
                        uint32_t plane = h_base + hs * PAIR_PLANE_SLOT;
                        for (int pq = 0; pq < 6 * PASSES && ok; pq++) {
                            if (X3 && pq == 12) {
                                /* passes 0 and 1 (plane as loaded) are issued; pass 2 reads its low part, which the splitter warps wrote */
                                if (!mbar_wait(xlo_full, xph, abort_flag, p.status, 12)) { ok = false; break; }
                                tc_fence_after();
                                plane = xlo_base;
                            }
                            if (!mbar_wait(wfull(ws), wph, abort_flag, p.status, 3)) { ok = false; break; }
                            tc_fence_after();
                            /* input row 2j-1+i with i = half + 2*(q/3): the second three products read one block row further down */
                            const int q = pq % 6;
                            const int down = q / 3, kx = q - down * 3;
                            const uint64_t adesc = make_smem_desc(w_base + ws * PAIR_W_BYTES);
                            const uint64_t bdesc = make_smem_desc(plane + (uint32_t)((down * p.P + kx) * BK * 4));
#pragma unroll
                            for (int j = 0; j < BK / 8; j++)
                                umma_tf32(d_tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (ks | half | pq | j) ? 1u : 0u);
                            umma_commit(wempty(ws));
                            if (++ws == PAIR_NW) { ws = 0; wph ^= 1u; }
                        }
                        if (X3) { if (ok) umma_commit(xlo_free); xph ^= 1u; }
                        if (ok) umma_commit(hempty(hs));
                        if (++hs == NH) { hs = 0; hph ^= 1u; }
                    }
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else if (warp < 6) {
        const int quarter = warp & 3;
        const int lower = quarter >> 1;                          /* 0: output rows 2j, 1: rows 2j+1 */
        const int pr = quarter & 1;                              /* channels pr*32 .. pr*32+31 */
        const int ch = pr * 32 + lane;
        const bool chok = ch < p.Cout;
        const float bv = (p.bias && chok) ? __ldg(p.bias + ch) : 0.0f;
        const float lo = p.act ? 0.0f : -INFINITY, hi = p.act ? FLT_MAX : INFINITY;
        float *obase = p.out + p.coff + ch;
        float *xb = xbuf + pr * 2 * PAIR_X_FLOATS;
        int it = 0;
        uint32_t gc = 0;                                         /* chunks exchanged so far (pooled mode) */
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int img = t / per, rem = t - img * per;
            const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
            const int x0 = txi * p.TW;
            if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * PAIR_N);
            if (p.P != 16) {
                /* 30-pixel pitch: a row pair is one 32-column TMEM load at column j * P (28 pixels of it are output) */
#pragma unroll 1
                for (int j = 0; j < p.TH && ok; j++) {
                    uint32_t r[32];
                    tmem_ld32(taddr + (uint32_t)(j * p.P), r);
                    const int jrow = tyi * p.TH + j;
                    if (p.pool) {
                        float h[14];
#pragma unroll
                        for (int px = 0; px < 14; px++) h[px] = fmaxf(__uint_as_float(r[2 * px]), __uint_as_float(r[2 * px + 1]));
                        const int b = (int)(gc & 1u);
                        const uint32_t xph = (gc >> 1) & 1u;
                        float *xs = xb + b * PAIR_X_FLOATS + lane;
                        if (lower) {
                            if (!mbar_wait_warp(xempty(pr, b), xph ^ 1u, abort_flag, p.status, 7)) { ok = false; break; }
#pragma unroll
                            for (int k = 0; k < 14; k++) xs[k * 32] = h[k];
                            __syncwarp();
                            if (lane == 0) mbar_arrive(xfull(pr, b));
                        } else {
                            if (!mbar_wait_warp(xfull(pr, b), xph, abort_flag, p.status, 8)) { ok = false; break; }
#pragma unroll
                            for (int k = 0; k < 14; k++) h[k] = fmaxf(h[k], xs[k * 32]);
                            __syncwarp();
                            if (lane == 0) mbar_arrive(xempty(pr, b));
                            if (chok && jrow < (p.H >> 1)) {
                                float *orow = obase + (((size_t)img * (p.H >> 1) + jrow) * (size_t)(p.W >> 1) + (x0 >> 1)) * p.ldo;
                                const int nx = min(14, (p.W >> 1) - (x0 >> 1));
#pragma unroll
                                for (int px = 0; px < 14; px++) {
                                    if (px < nx) *orow = fminf(fmaxf(h[px] + bv, lo), hi);
                                    orow += p.ldo;
                                }
                            }
                        }
                        gc++;
                    } else if (chok) {
                        const int y = 2 * jrow + lower;
                        if (y < p.H) {
                            float *optr = obase + (((size_t)img * p.H + y) * p.W + x0) * (size_t)p.ldo;
                            const int nx = min(p.TW, p.W - x0);
#pragma unroll
                            for (int dx = 0; dx < 28; dx++) {
                                if (dx < nx) *optr = fminf(fmaxf(__uint_as_float(r[dx]) + bv, lo), hi);
                                optr += p.ldo;
                            }
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < PAIR_N && ok; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                const int jrow = tyi * p.TH + (c0 >> 4);             /* this chunk holds row pairs jrow and jrow + 1 */
                if (p.pool) {
                    /* pooled row = row pair; horizontal maxima first, then the lower-row warp hands its values to the upper-row warp */
                    float h[14];
#pragma unroll
                    for (int dy = 0; dy < 2; dy++)
#pragma unroll
                        for (int px = 0; px < 7; px++)
                            h[dy * 7 + px] = fmaxf(__uint_as_float(r[dy * 16 + 2 * px]), __uint_as_float(r[dy * 16 + 2 * px + 1]));
                    const int b = (int)(gc & 1u);
                    const uint32_t xph = (gc >> 1) & 1u;
                    float *xs = xb + b * PAIR_X_FLOATS + lane;
                    if (lower) {
                        if (!mbar_wait_warp(xempty(pr, b), xph ^ 1u, abort_flag, p.status, 7)) { ok = false; break; }
#pragma unroll
                        for (int k = 0; k < 14; k++) xs[k * 32] = h[k];
                        __syncwarp();
                        if (lane == 0) mbar_arrive(xfull(pr, b));
                    } else {
                        if (!mbar_wait_warp(xfull(pr, b), xph, abort_flag, p.status, 8)) { ok = false; break; }
#pragma unroll
                        for (int k = 0; k < 14; k++) h[k] = fmaxf(h[k], xs[k * 32]);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(xempty(pr, b));
                        if (chok) {
#pragma unroll
                            for (int dy = 0; dy < 2; dy++) {
                                const int yo = jrow + dy;
                                if (yo >= (p.H >> 1)) break;
                                float *orow = obase + (((size_t)img * (p.H >> 1) + yo) * (size_t)(p.W >> 1) + (x0 >> 1)) * p.ldo;
                                const int nx = min(7, (p.W >> 1) - (x0 >> 1));
#pragma unroll
                                for (int px = 0; px < 7; px++) {
                                    if (px < nx) *orow = fminf(fmaxf(h[dy * 7 + px] + bv, lo), hi);
                                    orow += p.ldo;
                                }
                            }
                        }
                    }
                    gc++;
                } else if (chok) {
#pragma unroll
                    for (int dy = 0; dy < 2; dy++) {
                        const int y = 2 * (jrow + dy) + lower;
                        if (y >= p.H) break;
                        float *optr = obase + (((size_t)img * p.H + y) * p.W + x0) * (size_t)p.ldo;
                        const int nx = min(14, p.W - x0);
#pragma unroll
                        for (int dx = 0; dx < 14; dx++) {
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
        /* splitter warps: the low part of every plane into the low-part buffer, while passes 0 and 1 of that plane run */
        const int sw = warp - 6;
        int hs = 0;
        uint32_t hph = 0, xph = 0;
        bool ok = true;
        const int chunks = (int)(plane_bytes / 16);
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            for (int kh = 0; kh < 2 * p.kslabs; kh++) {
                /* the plane was written by TMA: wait on its barrier (visibility); the buffer is free once pass 2 of the plane before
                   has read it (first use: the wait on the preceding phase returns at once) */
                if (!mbar_wait_warp(hfull(hs), hph, abort_flag, p.status, 10)) { ok = false; break; }
                if (!mbar_wait_warp(xlo_free, xph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                const uint4 *blk = reinterpret_cast<const uint4 *>(gen + hs * PAIR_PLANE_SLOT);
                uint4 *lo = reinterpret_cast<uint4 *>(gen + NH * PAIR_PLANE_SLOT);
                for (int i = sw * 32 + lane; i < chunks; i += PAIR_SPLIT_WARPS * 32) {
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
                if (++hs == NH) { hs = 0; hph ^= 1u; }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

/* Picks the block geometry for a W x H image (see the top of the file): the one with the larger share of MMA columns that
 * are output pixels.  Returns that share; P, TW, TJ (row pairs per tile) through the pointers. */
double drk_umma_pair_geometry(int W, int H, int *P, int *TW, int *TJ)
{
    const int geo[2][3] = {{16, 14, 16}, {30, 28, 8}};
    double best = -1.0;
    for (int g = 0; g < 2; g++) {
        const int pitch = geo[g][0], tw = geo[g][1], tj = geo[g][2];
        const double tx = (W + tw - 1) / tw, ty = (H + 2 * tj - 1) / (2 * tj);
        const double fill = (double)W * H / (tx * ty * 2 * pitch * tj);
        if (fill > best + 1e-9) { best = fill; *P = pitch; *TW = tw; *TJ = tj; }
    }
    return best;
}

double drk_umma_pair_fill(int W, int H)
{
    int P, TW, TJ;
    return drk_umma_pair_geometry(W, H, &P, &TW, &TJ);
}

/* mapWlo: the filters' low parts (three-pass mode, x3 != 0); otherwise unused (pass mapW) */
int drk_umma_pair_launch(cudaStream_t st, const CUtensorMap *mapO, const CUtensorMap *mapE, const CUtensorMap *mapW, const CUtensorMap *mapWlo,
                         const UmmaParams *p, int grid, int x3)
{
    static bool attr_done[64];                      /* the opt-in shared-memory size is a per-device function attribute */
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_umma_conv_pair<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_umma_conv_pair<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    if (x3) drk_launch_dep(k_umma_conv_pair<true>, dim3(grid), dim3(PAIR_THREADS(1)), PAIR_SMEM, st, *mapO, *mapE, *mapW, *mapWlo, *p);
    else drk_launch_dep(k_umma_conv_pair<false>, dim3(grid), dim3(PAIR_THREADS(0)), PAIR_SMEM, st, *mapO, *mapE, *mapW, *mapW, *p);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}
