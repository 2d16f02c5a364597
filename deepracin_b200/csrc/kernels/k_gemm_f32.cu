/*
 * Exact-FP32 (FFMA) GEMM core of the CNN-layer path, used three ways:
 *   - implicit-GEMM convolution: A rows are output pixels gathered on the fly from the
 *     N-HWC input (zero padded), B is the packed filter matrix [kh*kw*Cin][Cout];
 *   - dense GEMM for the 16 transform-domain products of the Winograd path;
 *   - dense split-K GEMM for fully connected layers at larger batch sizes.
 * CTA tile BM x BN x 16, 256 threads, TM x TN accumulators per thread, operands staged in
 * shared memory (A stored k-major so both operands are read as float4), next tile
 * prefetched into registers while the current one is multiplied.  Bound: FP32 FFMA issue
 * rate for K >= ~100, HBM for the first VGG layer (K = 27).
 */
#include "k_common.cuh"
#include "k_gemm_f32.cuh"

#define BK 16

template <int BM, int BN, int TM, int TN, bool CONV>
/* two CTAs per SM for the 128 x 128 convolution variant (128 registers without spills); the dense variant would spill at that limit */
__global__ void __launch_bounds__(256, BM == 128 ? (CONV ? 2 : 1) : 3) k_gemm_f32(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias,
                                                  float *__restrict__ C, int M, int N, int K, int lda, int ldb, int ldc, int coff, int act,
                                                  size_t strideA, size_t strideB, size_t strideC, int vecA, int vecB, int vecC, drk_ConvGeom g)
{
    constexpr int LDA_S = BM + 4;
    constexpr int A_UNITS = BM * BK / 4 / 256 > 0 ? BM * BK / 4 / 256 : 1;   /* float4 units per thread */
    constexpr int B_UNITS = BN * BK / 4 / 256 > 0 ? BN * BK / 4 / 256 : 1;
    constexpr int A_ACTIVE = BM * BK / 4;   /* total units */
    constexpr int B_ACTIVE = BN * BK / 4;
    constexpr int RCH = TM / 4, CCH = TN / 4;
    __shared__ __align__(16) float As[2][BK][LDA_S];
    __shared__ __align__(16) float Bs[2][BK][BN];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    A += (size_t)blockIdx.z * strideA;
    B += (size_t)blockIdx.z * strideB;
    C += (size_t)blockIdx.z * strideC;

    /* per-thread description of the A rows it stages */
    /* unit i of a thread is float4 number tid + 256*i of the tile: its row is tid/4 + 64*i and its K segment (tid%4)*4 for
       every i, so only what is expensive to recompute is kept in registers (two CTAs per SM need <= 128 of them) */
    const int a_kseg0 = (tid % (BK / 4)) * 4, a_row0 = tid / (BK / 4);
#define a_kseg(i) a_kseg0
#define a_row(i) (a_row0 + (i) * (256 / (BK / 4)))
    bool a_ok[A_UNITS];
    size_t a_base[A_UNITS];             /* dense: row offset; conv: image offset */
    int a_iy0[A_UNITS], a_ix0[A_UNITS];
#pragma unroll
    for (int i = 0; i < A_UNITS; i++) {
        const int u = tid + i * 256;
        const int m = m0 + a_row(i);
        a_ok[i] = u < A_ACTIVE && m < M;
        a_base[i] = 0; a_iy0[i] = 0; a_ix0[i] = 0;
        if (a_ok[i]) {
            if (CONV) {
                const int ox = m % g.Wo;
                const int t = m / g.Wo;
                const int oy = t % g.Ho;
                const int b = t / g.Ho;
                a_base[i] = (size_t)b * g.H * g.W;
                a_iy0[i] = oy * g.sy - g.py;
                a_ix0[i] = ox * g.sx - g.px;
            } else {
                a_base[i] = (size_t)m * lda;
            }
        }
    }
    const int b_n0 = (tid % (BN / 4)) * 4, b_krow0 = tid / (BN / 4);
#define b_n(i) b_n0
#define b_krow(i) (b_krow0 + (i) * (256 / (BN / 4)))

    float4 ra[A_UNITS], rb[B_UNITS];

    auto load_tiles = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_UNITS; i++) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int k = k0 + a_kseg(i);
            if (a_ok[i] && k < K) {
                if (CONV) {
                    if (vecA) {
                        const int tap = k / g.Cin, c = k - tap * g.Cin;
                        const int ky = tap / g.kw, kx = tap - ky * g.kw;
                        const int iy = a_iy0[i] + ky, ix = a_ix0[i] + kx;
                        if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W)
                            v = *reinterpret_cast<const float4 *>(A + (a_base[i] + (size_t)iy * g.W + ix) * g.ldi + c);
                    } else {
                        float t[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            t[j] = 0.f;
                            const int kk = k + j;
                            if (kk < K) {
                                const int tap = kk / g.Cin, c = kk - tap * g.Cin;
                                const int ky = tap / g.kw, kx = tap - ky * g.kw;
                                const int iy = a_iy0[i] + ky, ix = a_ix0[i] + kx;
                                if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) t[j] = A[(a_base[i] + (size_t)iy * g.W + ix) * g.ldi + c];
                            }
                        }
                        v = make_float4(t[0], t[1], t[2], t[3]);
                    }
                } else {
                    const float *p = A + a_base[i] + k;
                    if (vecA && k + 3 < K) v = *reinterpret_cast<const float4 *>(p);
                    else {
                        v.x = p[0];
                        if (k + 1 < K) v.y = p[1];
                        if (k + 2 < K) v.z = p[2];
                        if (k + 3 < K) v.w = p[3];
                    }
                }
            }
            ra[i] = v;
        }
#pragma unroll
        for (int i = 0; i < B_UNITS; i++) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int k = k0 + b_krow(i), n = n0 + b_n(i);
            if (tid + i * 256 < B_ACTIVE && k < K && n < N) {
                const float *p = B + (size_t)k * ldb + n;
                if (vecB && n + 3 < N) v = *reinterpret_cast<const float4 *>(p);
                else {
                    v.x = p[0];
                    if (n + 1 < N) v.y = p[1];
                    if (n + 2 < N) v.z = p[2];
                    if (n + 3 < N) v.w = p[3];
                }
            }
            rb[i] = v;
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_UNITS; i++) {
            if (tid + i * 256 < A_ACTIVE) {
                As[buf][a_kseg(i) + 0][a_row(i)] = ra[i].x;
                As[buf][a_kseg(i) + 1][a_row(i)] = ra[i].y;
                As[buf][a_kseg(i) + 2][a_row(i)] = ra[i].z;
                As[buf][a_kseg(i) + 3][a_row(i)] = ra[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < B_UNITS; i++)
            if (tid + i * 256 < B_ACTIVE) *reinterpret_cast<float4 *>(&Bs[buf][b_krow(i)][b_n(i)]) = rb[i];
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    const int numKT = (K + BK - 1) / BK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    int cur = 0;
    for (int kt = 0; kt < numKT; kt++) {
        if (kt + 1 < numKT) load_tiles((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], b[TN];
#pragma unroll
            for (int r = 0; r < RCH; r++) {
                const float4 t = *reinterpret_cast<const float4 *>(&As[cur][k][r * (BM / RCH) + ty * 4]);
                a[r * 4 + 0] = t.x; a[r * 4 + 1] = t.y; a[r * 4 + 2] = t.z; a[r * 4 + 3] = t.w;
            }
#pragma unroll
            for (int c = 0; c < CCH; c++) {
                const float4 t = *reinterpret_cast<const float4 *>(&Bs[cur][k][c * (BN / CCH) + tx * 4]);
                b[c * 4 + 0] = t.x; b[c * 4 + 1] = t.y; b[c * 4 + 2] = t.z; b[c * 4 + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < numKT) {
            store_tiles(cur ^ 1);
            __syncthreads();
            cur ^= 1;
        }
    }

    /* epilogue: bias, activation, store at (pixel stride ldc, channel offset coff) */
#pragma unroll
    for (int r = 0; r < RCH; r++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = m0 + r * (BM / RCH) + ty * 4 + i;
            if (m >= M) continue;
            float *crow = C + (size_t)m * ldc + coff;
#pragma unroll
            for (int c = 0; c < CCH; c++) {
                const int n = n0 + c * (BN / CCH) + tx * 4;
                if (n >= N) continue;
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float t = acc[r * 4 + i][c * 4 + j];
                    if (bias && n + j < N) t += bias[n + j];
                    v[j] = drk_act(t, act);
                }
                if (vecC && n + 3 < N) *reinterpret_cast<float4 *>(crow + n) = make_float4(v[0], v[1], v[2], v[3]);
                else {
#pragma unroll
                    for (int j = 0; j < 4; j++) if (n + j < N) crow[n + j] = v[j];
                }
            }
        }
}

#undef a_kseg
#undef a_row
#undef b_n
#undef b_krow

/*
 * The same product for 16-byte-aligned operands (every VGG / Winograd / fully connected shape), with asynchronous staging:
 * both operand tiles go from global to shared memory by cp.async (16 bytes per request, zero fill past the edges and for
 * the convolution's padding) through a ring of STAGES buffers, one __syncthreads per 16-deep K tile, no staging registers.
 * A is kept as it lies in memory -- [row][k], K contiguous -- and read back with 128-bit loads along K (four K steps per
 * load); the two row groups of a warp read two addresses (broadcast), B is read as in the kernel above.  128 x 128 x 16
 * tiles, 8 x 8 accumulators per thread held as 8 x 4 column pairs and updated with the packed FFMA2 of sm_100 (two IEEE FMAs per
 * instruction: the scalar version of this loop was bound by register-port conflicts of its 64 FFMAs per K step, ncu: dispatch
 * stalls on 0.8 of the issued instructions, FMA pipe 60 % active; packed: 71 %), two CTAs per SM.
 * Measured on 256->256 @56x56 batch 64: Winograd 2.74 -> 2.42 ms, direct 5.51 -> 5.22 ms.
 */
#define AS_STAGES 4
#define AS_APITCH (BK + 4)          /* floats per staged A row: 16 + 4 keeps rows 16-byte aligned and spreads banks */
/* NCH = 64-column chunks per CTA tile (BN = 64 or 128), MR = 64-row groups (BM = 64 or 128; 64 for GEMMs of at most 64 rows: a
   fully connected layer at batch 17..64) */
#define AS_SMEM(NCH, MR) (AS_STAGES * (64 * (MR) * AS_APITCH + BK * 64 * (NCH)) * 4)

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

template <bool CONV, int NCH, int MR>
__global__ void __launch_bounds__(256, 2) k_gemm_f32_async(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias,
                                                           float *__restrict__ C, int M, int N, int K, int lda, int ldb, int ldc, int coff, int act,
                                                           size_t strideA, size_t strideB, size_t strideC, int vecC, drk_ConvGeom g)
{
    extern __shared__ __align__(16) float smem_f[];
    float *As = smem_f;                                         /* [STAGES][BM][APITCH] */
    constexpr int AS_BN = 64 * NCH, AS_BM = 64 * MR;
    float *Bs = smem_f + AS_STAGES * AS_BM * AS_APITCH;         /* [STAGES][BK][BN] */
    const uint32_t as_u = (uint32_t)__cvta_generic_to_shared(As), bs_u = (uint32_t)__cvta_generic_to_shared(Bs);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * AS_BM, n0 = blockIdx.x * AS_BN;
    A += (size_t)blockIdx.z * strideA;
    B += (size_t)blockIdx.z * strideB;
    C += (size_t)blockIdx.z * strideC;

    /* staging assignment: A unit i = row tid/4 + 64 i, K segment (tid%4)*4; B unit i = K row tid/(BN/4) + 8 i (one unit covers
       all 16 rows when BN = 64), columns (tid%(BN/4))*4 */
    const int a_kseg = (tid & 3) * 4, a_row0 = tid >> 2;
    const int b_n = (tid % (AS_BN / 4)) * 4, b_k0 = tid / (AS_BN / 4);
    bool a_ok[MR];
    size_t a_base[MR];
    int a_iy0[MR], a_ix0[MR];
#pragma unroll
    for (int i = 0; i < MR; i++) {
        const int m = m0 + a_row0 + 64 * i;
        a_ok[i] = m < M;
        a_base[i] = 0; a_iy0[i] = 0; a_ix0[i] = 0;
        if (a_ok[i]) {
            if (CONV) {
                const int ox = m % g.Wo;
                const int t = m / g.Wo;
                const int oy = t % g.Ho;
                a_base[i] = (size_t)(t / g.Ho) * g.H * g.W;
                a_iy0[i] = oy * g.sy - g.py;
                a_ix0[i] = ox * g.sx - g.px;
            } else {
                a_base[i] = (size_t)m * lda;
            }
        }
    }
    const int bn_bytes = (n0 + b_n < N) ? 4 * min(4, N - n0 - b_n) : 0;

    auto stage_load = [&](int kt, int slot) {
        const int k = kt * BK + a_kseg;
#pragma unroll
        for (int i = 0; i < MR; i++) {
            const float *src = A;
            int bytes = 0;
            if (a_ok[i] && k < K) {
                if (CONV) {
                    const int tap = k / g.Cin, c = k - tap * g.Cin;
                    const int ky = tap / g.kw, kx = tap - ky * g.kw;
                    const int iy = a_iy0[i] + ky, ix = a_ix0[i] + kx;
                    if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) { src = A + (a_base[i] + (size_t)iy * g.W + ix) * g.ldi + c; bytes = 16; }
                } else {
                    src = A + a_base[i] + k;
                    bytes = 4 * min(4, K - k);
                }
            }
            cp_async16(as_u + (uint32_t)(((slot * AS_BM + a_row0 + 64 * i) * AS_APITCH + a_kseg) * 4), src, bytes);
        }
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            const int kr = kt * BK + b_k0 + 8 * i;
            const bool ok = kr < K && bn_bytes > 0;
            cp_async16(bs_u + (uint32_t)(((slot * BK + b_k0 + 8 * i) * AS_BN + b_n) * 4), ok ? (const void *)(B + (size_t)kr * ldb + n0 + b_n) : (const void *)B, ok ? bn_bytes : 0);
        }
    };

    /* accumulators as pairs of neighbouring columns: one packed FFMA2 (fma.rn.f32x2, two IEEE round-to-nearest FMAs, the same
       results as two scalar ones) per pair halves the instruction and register-port traffic of the 8 x 8 outer product */
    float2 acc[4 * MR][2 * NCH];
#pragma unroll
    for (int i = 0; i < 4 * MR; i++)
#pragma unroll
        for (int j = 0; j < 2 * NCH; j++) acc[i][j] = make_float2(0.f, 0.f);

    const int numKT = (K + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < AS_STAGES - 1; s++) {
        if (s < numKT) stage_load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < numKT; kt++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(AS_STAGES - 2) : "memory");
        __syncthreads();                    /* tile kt has landed for everyone; everyone is done with the slot refilled below */
        if (kt + AS_STAGES - 1 < numKT) stage_load(kt + AS_STAGES - 1, (kt + AS_STAGES - 1) % AS_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int slot = kt % AS_STAGES;
        const float *as = As + (size_t)slot * AS_BM * AS_APITCH;
        const float *bs = Bs + (size_t)slot * BK * AS_BN;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 4) {
            float4 a4[4 * MR];
#pragma unroll
            for (int r = 0; r < MR; r++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    a4[r * 4 + i] = *reinterpret_cast<const float4 *>(as + (r * 64 + ty * 4 + i) * AS_APITCH + kk);
#pragma unroll
            for (int k4 = 0; k4 < 4; k4++) {
                float2 b[2 * NCH];
#pragma unroll
                for (int c = 0; c < NCH; c++) {
                    const float4 t = *reinterpret_cast<const float4 *>(bs + (kk + k4) * AS_BN + c * 64 + tx * 4);
                    b[c * 2 + 0] = make_float2(t.x, t.y); b[c * 2 + 1] = make_float2(t.z, t.w);
                }
#pragma unroll
                for (int i = 0; i < 4 * MR; i++) {
                    const float av = k4 == 0 ? a4[i].x : k4 == 1 ? a4[i].y : k4 == 2 ? a4[i].z : a4[i].w;
                    const float2 a2 = make_float2(av, av);
#pragma unroll
                    for (int j = 0; j < 2 * NCH; j++) acc[i][j] = __ffma2_rn(a2, b[j], acc[i][j]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
    for (int r = 0; r < MR; r++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = m0 + r * 64 + ty * 4 + i;
            if (m >= M) continue;
            float *crow = C + (size_t)m * ldc + coff;
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                const int n = n0 + c * 64 + tx * 4;
                if (n >= N) continue;
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 pr = acc[r * 4 + i][c * 2 + (j >> 1)];
                    float t = (j & 1) ? pr.y : pr.x;
                    if (bias && n + j < N) t += bias[n + j];
                    v[j] = drk_act(t, act);
                }
                if (vecC && n + 3 < N) *reinterpret_cast<float4 *>(crow + n) = make_float4(v[0], v[1], v[2], v[3]);
                else {
#pragma unroll
                    for (int j = 0; j < 4; j++) if (n + j < N) crow[n + j] = v[j];
                }
            }
        }
}

template <bool CONV, int NCH, int MR>
static int launch_async(cudaStream_t st, dim3 grid, const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int lda, int ldb,
                        int ldc, int coff, int act, size_t sA, size_t sB, size_t sC, int vecC, const drk_ConvGeom &g)
{
    static bool attr_done[64];                      /* the opt-in shared-memory size is a per-device function attribute */
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm_f32_async<CONV, NCH, MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, AS_SMEM(NCH, MR));
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    k_gemm_f32_async<CONV, NCH, MR><<<grid, 256, AS_SMEM(NCH, MR), st>>>(A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g);
    return 0;
}

static bool aligned16(const void *p) { return ((uintptr_t)p % 16) == 0; }

int drk_gemm_f32_launch(cudaStream_t st, const float *A, const float *B, const float *bias, float *C, int M, int N, int K,
                        int lda, int ldb, int ldc, int coff, int act, int batch, size_t sA, size_t sB, size_t sC, const drk_ConvGeom *geom)
{
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -1;
    drk_ConvGeom g;
    memset(&g, 0, sizeof g);
    int vecA;
    if (geom) {
        g = *geom;
        vecA = g.Cin % 4 == 0 && g.ldi % 4 == 0 && aligned16(A);
    } else {
        vecA = lda % 4 == 0 && aligned16(A) && sA % 4 == 0;
    }
    const int vecB = ldb % 4 == 0 && aligned16(B) && sB % 4 == 0;
    const int vecC = ldc % 4 == 0 && coff % 4 == 0 && aligned16(C) && sC % 4 == 0;
    const long big = (long)((M + 127) / 128) * ((N + 127) / 128) * batch;
    const bool small = big < 120 || N <= 64 || M <= 64;
    dim3 grid;
    if (small) grid = dim3((N + 63) / 64, (M + 63) / 64, batch);
    else grid = dim3((N + 127) / 128, (M + 127) / 128, batch);
    if (grid.y > 65535u || grid.z > 65535u) return -2;
    if (vecA && vecB && M > 64) {
        /* 16-byte-aligned operands: the cp.async-staged kernel, 128 x 128 tiles or 128 x 64 for narrow outputs, as long as the
           launch has about a tile per SM (two CTAs per SM, 128 registers: measured 8 % faster than one CTA with 152) */
        const int nch = N <= 64 ? 1 : 2;
        const dim3 ga((N + 64 * nch - 1) / (64 * nch), (M + 127) / 128, batch);
        if ((long)ga.x * ga.y * ga.z >= 100 && ga.y <= 65535u && ga.z <= 65535u) {
            int rc;
            if (nch == 2) rc = geom ? launch_async<true, 2, 2>(st, ga, A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g)
                                    : launch_async<false, 2, 2>(st, ga, A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g);
            else rc = geom ? launch_async<true, 1, 2>(st, ga, A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g)
                           : launch_async<false, 1, 2>(st, ga, A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g);
            if (rc) return rc;
            DRK_COUNT_LAUNCH();
            return DRK_LAUNCH_RESULT();
        }
    }
    if (vecA && vecB && !geom && M > 16 && M <= 64 && N >= 128) {
        /* a short, wide product (fully connected layer at batch 17..64, batched over K slices): 64 x 128 tiles */
        const dim3 ga((N + 127) / 128, 1, batch);
        if ((long)ga.x * ga.z >= 100 && ga.z <= 65535u) {
            int rc = launch_async<false, 2, 1>(st, ga, A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecC, g);
            if (rc) return rc;
            DRK_COUNT_LAUNCH();
            return DRK_LAUNCH_RESULT();
        }
    }
    if (geom) {
        if (small) k_gemm_f32<64, 64, 4, 4, true><<<grid, 256, 0, st>>>(A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecA, vecB, vecC, g);
        else k_gemm_f32<128, 128, 8, 8, true><<<grid, 256, 0, st>>>(A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecA, vecB, vecC, g);
    } else {
        if (small) k_gemm_f32<64, 64, 4, 4, false><<<grid, 256, 0, st>>>(A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecA, vecB, vecC, g);
        else k_gemm_f32<128, 128, 8, 8, false><<<grid, 256, 0, st>>>(A, B, bias, C, M, N, K, lda, ldb, ldc, coff, act, sA, sB, sC, vecA, vecB, vecC, g);
    }
    DRK_COUNT_LAUNCH();
    return DRK_LAUNCH_RESULT();
}

extern "C" int dRk_conv2d_f32(dRk_stream stream, const float *in, const float *wpack, const float *bias, float *out,
                              int n, int W, int H, int Cin, int Cout, int kw, int kh, int sx, int sy, int act,
                              int ldi, int ldo, int coff)
{
    if (n <= 0 || W <= 0 || H <= 0 || Cin <= 0 || Cout <= 0 || kw <= 0 || kh <= 0 || sx <= 0 || sy <= 0) return -1;
    if (ldi < Cin || ldo < coff + Cout) return -3;
    if (kw == 3 && kh == 3 && sx == 1 && sy == 1) {        /* output-bound layers with a handful of input channels */
        int rc = 0;
        if (drk_conv3x3_smallcin_launch(drk_stream(stream), in, wpack, bias, out, n, W, H, Cin, Cout, act, ldi, ldo, coff, &rc)) return rc;
    }
    drk_ConvGeom g;
    g.W = W; g.H = H; g.Cin = Cin; g.kw = kw; g.kh = kh; g.sx = sx; g.sy = sy;
    g.Wo = W / sx; g.Ho = H / sy; g.px = kw / 2; g.py = kh / 2; g.ldi = ldi;
    if (g.Wo <= 0 || g.Ho <= 0) return -1;
    const long long M = (long long)n * g.Ho * g.Wo;
    if (M > 0x7fffffffLL) return -2;
    return drk_gemm_f32_launch(drk_stream(stream), in, wpack, bias, out, (int)M, Cout, kw * kh * Cin, 0, Cout, ldo, coff, act,
                               1, 0, 0, 0, &g);
}
