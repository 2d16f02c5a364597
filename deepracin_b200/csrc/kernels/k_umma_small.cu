/*
 * Tensor-core 3x3 stride-1 convolution for layers with at most four input channels (the RGB first layer of VGG-16 and
 * SqueezeNet) in TF32 mode, without a gather.  Replaces conv2dwinograd2 (Kernels/dR_winograd2.cl:23-254) for these layers;
 * bound: HBM (the output is written once: n*H*W*Cout*4 bytes; with a fused 2x2 pool a quarter of that).
 *
 * A pixel of such a layer is 12 bytes, which TMA cannot tile, so a first pass (k_pad_c4) rewrites the input as
 * [n][H][W][4] floats (16 bytes per pixel, channel 3 = 0), evaluating an optional affine channel map on the way -- the
 * Slice / scalar-op / Concat preamble of the example graphs (examples/squeezenet-v1.1/squeezenet_whole/graph.dr:7-41).
 * In that layout a haloed (TH+2) x P pixel block is one 4-D TMA box of 16-byte rows, and it already IS the im2col
 * operand: tcgen05's K-major layout without swizzle is built from core matrices of 8 rows x 16 bytes, the row being one
 * pixel here.  Output pixel j (block row r, column x: j = r*P + x) and tap (ky, kx) read block pixel j + ky*P + kx, i.e.
 * the 8-pixel core matrix of tap (ky, kx) starts (ky*P + kx) * 16 bytes into the block, and the core matrix of the next tap
 * in the row starts 16 bytes after it: the descriptor's K stride (leading byte offset) is 16 bytes, its stride between
 * 8-pixel groups 128 bytes, and consecutive core matrices overlap in memory.  One MMA (K = 8) covers two taps of a filter
 * row; a filter row is taps kx = 0, 1 and kx = 2, 3 with zero weights for the fourth: six MMAs of N = P*TH pixels per tile,
 * M = output channels (transposed product, epilogue as in k_umma_conv_swap: a lane owns a channel).  The filters
 * [128][12 chunks x 4 floats] stay in shared memory for the CTA's lifetime.
 *
 * Persistent CTAs, 10 warps: warp 0 TMA producer (blocks through a ring of 8 slots), warp 1 MMA issuer and TMEM owner,
 * warps 2-9 epilogue (two per TMEM lane quarter, alternating block rows).  Fused 2x2/2 max or average pooling.  Every wait
 * is bounded; on expiry the CTA flags an abort, reports a code through `status`, drains its copies, frees TMEM and returns.
 */
#include <stdio.h>
#include "k_common.cuh"
#include "k_umma.cuh"

#define C4_THREADS 320
#define C4_EPI_WARPS 8
#define C4_NH 8                         /* block slots */
#define C4_SLOT 6144                    /* (8 + 2) rows x 32 pixels x 16 B = 5120, plus room for the taps of the last idle columns */
#define C4_W_CHUNK (BM * 16)            /* one filter chunk: 128 rows x 16 bytes */
#define C4_W_BYTES (12 * C4_W_CHUNK)
#define C4_N 256
#define C4_SMEM (C4_NH * C4_SLOT + C4_W_BYTES + 1024 + 512)

/* K-major operand without swizzle: core matrices of 8 rows x 16 bytes; lbo = bytes between core matrices along K,
 * sbo = bytes between 8-row groups */
__device__ __forceinline__ uint64_t make_smem_desc_noswz(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

struct PadMap {
    int use, ch[4];
    float scale[4], shift[4];
};

/* [pixels][ldi >= Cin] -> [pixels][4], channel c = scale[c] * in[ch[c]] + shift[c] (identity without a map), channels >= Cin zero */
__global__ void k_pad_c4(const float *__restrict__ in, float4 *__restrict__ out, size_t pixels, int Cin, int ldi, const PadMap m)
{
    drk_dep_trigger();
    drk_dep_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pixels; i += (size_t)gridDim.x * blockDim.x) {
        const float *px = in + i * (size_t)ldi;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; c++)
            if (c < Cin) v[c] = m.use ? fmaf(__ldg(px + m.ch[c]), m.scale[c], m.shift[c]) : __ldg(px + c);
        out[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

__global__ void __launch_bounds__(C4_THREADS, 1)
k_umma_conv_c4(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW, const UmmaParams p)
{
    extern __shared__ uint8_t smem_raw[];
    drk_dep_trigger();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t h_base = base, w_base = base + C4_NH * C4_SLOT;
    const uint32_t bars = w_base + C4_W_BYTES;
    constexpr int NBARS = 2 * C4_NH + 6;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + C4_NH * C4_SLOT + C4_W_BYTES + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    auto hfull = [&](int s) { return bars + 8u * s; };
    auto hempty = [&](int s) { return bars + 8u * (C4_NH + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * C4_NH + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * C4_NH + 2 + a); };
    const uint32_t wfull = bars + 8u * (2 * C4_NH + 4);
    const uint32_t drain_bar = bars + 8u * (2 * C4_NH + 5);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles;
    const int per = p.tiles_x * p.tiles_y;
    constexpr int TMEM_COLS = 2 * C4_N;
    const uint32_t block_bytes = (uint32_t)((p.TH + 2) * p.P * 16);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C4_NH; s++) { mbar_init(hfull(s), 1); mbar_init(hempty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), C4_EPI_WARPS); }
        mbar_init(wfull, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    /* what lies behind a block in its slot is read by the taps of the last columns (into idle accumulator columns, and with
       the zero weights of the fourth tap into real ones): it must hold finite numbers */
    for (int i = threadIdx.x; i < C4_NH * (C4_SLOT / 16); i += C4_THREADS) reinterpret_cast<uint4 *>(gen)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapX) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&mapW) : "memory");
            /* the filters are constants: requested before this grid waits for the one before it */
            mbar_expect_tx(wfull, C4_W_BYTES);
            for (int q = 0; q < 12; q++) tma_load_2d(w_base + q * C4_W_CHUNK, &mapW, q * 4, 0, wfull);
            drk_dep_wait();
            int hs = 0;
            uint32_t hph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int img = t / per, rem = t - img * per;
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                if (!mbar_wait(hempty(hs), hph ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
                mbar_expect_tx(hfull(hs), block_bytes);
                tma_load_4d(h_base + hs * C4_SLOT, &mapX, 0, txi * p.TW - 1, tyi * p.TH - 1, img, hfull(hs));
                issued++;
                if (++hs == C4_NH) { hs = 0; hph ^= 1u; }
            }
            if (!ok) {
                long long pend = issued < C4_NH ? issued : C4_NH;
                int s = hs; uint32_t ph = hph;
                for (long long i = 0; i < pend; i++) {
                    if (--s < 0) { s = C4_NH - 1; ph ^= 1u; }
                    const long long t0 = clock64();
                    while (!mbar_try(hfull(s), ph) && clock64() - t0 < WAIT_CYCLES) { }
                }
                const long long t0 = clock64();
                while (!mbar_try(wfull, 0) && clock64() - t0 < WAIT_CYCLES) { }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(p.ncols);
            int hs = 0;
            uint32_t hph = 0;
            int it = 0;
            bool ok = mbar_wait(wfull, 0, abort_flag, p.status, 3);
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                if (!mbar_wait(hfull(hs), hph, abort_flag, p.status, 6)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C4_N);
                const uint32_t blk = h_base + hs * C4_SLOT;
#pragma unroll
                for (int g = 0; g < 6; g++) {
                    const int ky = g >> 1, half = g & 1;                /* taps (ky, 2*half) and (ky, 2*half + 1) */
                    const uint64_t adesc = make_smem_desc_noswz(w_base + (uint32_t)((ky * 4 + half * 2) * C4_W_CHUNK), C4_W_CHUNK, 128);
                    const uint64_t bdesc = make_smem_desc_noswz(blk + (uint32_t)((ky * p.P + half * 2) * 16), 16, 128);
                    umma_tf32(d_tmem, adesc, bdesc, idesc, g ? 1u : 0u);
                }
                umma_commit(hempty(hs));
                umma_commit(tfull_bar(acc));
                if (++hs == C4_NH) { hs = 0; hph ^= 1u; }
            }
            if (!ok) umma_drain(drain_bar);
        }
    } else {
        drk_dep_wait();             /* the epilogue's stores must follow the previous grid's reads of the output buffer */
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int ch = quarter * 32 + lane;                 /* the output channel this lane owns */
        const bool chok = ch < p.Cout;
        const float bv = (p.bias && chok) ? __ldg(p.bias + ch) : 0.0f;
        const float lo = p.act ? 0.0f : -INFINITY, hi = p.act ? FLT_MAX : INFINITY;
        float *obase = p.out + p.coff + ch;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int img = t / per, rem = t - img * per;
            const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
            const int x0 = txi * p.TW;
            if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * C4_N);
            /* a block row is one 32-column TMEM load at column row * P; the two warps of a quarter take alternate rows (row pairs
               when a 2x2 pool is fused).  Warp-wide loads: every lane executes them, lanes past Cout only skip the stores. */
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
                        float v;
                        if (p.pool == 1) {          /* bias and activation are monotone: the maximum commutes with them */
                            v = fmaxf(fmaxf(__uint_as_float(r0[2 * px]), __uint_as_float(r0[2 * px + 1])),
                                      fmaxf(__uint_as_float(r1[2 * px]), __uint_as_float(r1[2 * px + 1])));
                            v = fminf(fmaxf(v + bv, lo), hi);
                        } else {                    /* average of the four activated values */
                            v = 0.25f * (fminf(fmaxf(__uint_as_float(r0[2 * px]) + bv, lo), hi) + fminf(fmaxf(__uint_as_float(r0[2 * px + 1]) + bv, lo), hi) +
                                         fminf(fmaxf(__uint_as_float(r1[2 * px]) + bv, lo), hi) + fminf(fmaxf(__uint_as_float(r1[2 * px + 1]) + bv, lo), hi));
                        }
                        if (px < nx) *orow = v;
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

/* ------------------------------------------------------------------------------------------------ host side */
int drk_umma_c4_supported(int Cin, int Cout, int kw, int kh)
{
    return kw == 3 && kh == 3 && Cin >= 1 && Cin <= 4 && Cout >= 16 && Cout <= BM && Cout % 4 == 0;
}

/* Block geometry: rows of P = 30 (28 valid) or 32 (up to 30 valid) pixels, TH of them, N = P * TH <= 256 a multiple of 16; the
 * one with the larger share of columns that are output pixels (an even TH when a 2x2 pool is fused). */
double drk_umma_c4_geometry(int W, int H, int pool, int *P, int *TW, int *TH)
{
    double best = -1.0;
    const int pitches[2] = {30, 32};
    for (int pi = 0; pi < 2; pi++) {
        const int pitch = pitches[pi];
        const int tw = pitch == 30 ? 28 : (W < 30 ? ((W + 1) & ~1) : 30);
        if (tw < 2 || tw > pitch - 2) continue;
        for (int th = 8; th >= 2; th--) {
            const int ncols = pitch * th;
            if (ncols % 16 || ncols > C4_N) continue;
            if (pool && (th & 1)) continue;
            const double tx = (W + tw - 1) / tw, ty = (H + th - 1) / th;
            const double fill = (double)W * H / (tx * ty * ncols);
            if (fill > best + 1e-9) { best = fill; *P = pitch; *TW = tw; *TH = th; }
        }
    }
    return best;
}

size_t drk_umma_c4_packed_floats(void) { return (size_t)BM * 48; }

/* [128 rows][12 chunks x 4]: chunk ky*4 + kx holds channels 0..3 of tap (ky, kx); kx = 3, channels >= Cin and rows >= Cout are zero */
int drk_umma_c4_pack_weights(const float *w, float *dst, int Cin, int Cout)
{
    memset(dst, 0, drk_umma_c4_packed_floats() * sizeof(float));
    for (int o = 0; o < Cout; o++)
        for (int c = 0; c < Cin; c++)
            for (int ky = 0; ky < 3; ky++)
                for (int kx = 0; kx < 3; kx++)
                    dst[(size_t)o * 48 + (ky * 4 + kx) * 4 + c] = w[((size_t)c * Cout + o) * 9 + ky * 3 + kx];
    return 0;
}

int drk_umma_c4_pad_launch(cudaStream_t st, const float *in, float *padded, size_t pixels, int Cin, int ldi, const int *map_ch, const float *map_scale,
                           const float *map_shift)
{
    PadMap m;
    memset(&m, 0, sizeof m);
    if (map_ch) {
        m.use = 1;
        for (int c = 0; c < Cin; c++) { m.ch[c] = map_ch[c]; m.scale[c] = map_scale[c]; m.shift[c] = map_shift[c]; }
    }
    drk_launch_dep(k_pad_c4, dim3(drk_blocks(pixels, 256, 148u * 16u)), dim3(256), 0, st, in, reinterpret_cast<float4 *>(padded), pixels, Cin, ldi, m);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

int drk_umma_c4_launch(cudaStream_t st, const CUtensorMap *mapX, const CUtensorMap *mapW, const UmmaParams *p, int grid)
{
    static bool attr_done[64];                      /* the opt-in shared-memory size is a per-device function attribute */
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_umma_conv_c4, cudaFuncAttributeMaxDynamicSharedMemorySize, C4_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    drk_launch_dep(k_umma_conv_c4, dim3(grid), dim3(C4_THREADS), C4_SMEM, st, *mapX, *mapW, *p);
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}
