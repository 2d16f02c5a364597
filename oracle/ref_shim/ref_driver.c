/*
 * Reference-kernel leg of the CPU oracle -- TEST INFRASTRUCTURE ONLY.
 *
 * Compiles the reference's live OpenCL C kernel files, unmodified and in place
 * (this file #includes them from the reference checkout; nothing is copied), as
 * plain C through cl_shim.h and runs them under a small NDRange emulator:
 * work-groups are spread over OpenMP threads, the work-items of a group that
 * uses barrier() run as cooperative ucontext fibers so barrier() keeps its
 * meaning.  The host-side steps the reference performs around each kernel
 * (scheduling arithmetic, filter transform, weight transpose, host softmax sum)
 * are restated here from the cited lines so that the launch geometry and hence
 * the summation order are the reference's own.
 *
 * The emulated device limits (local memory size, max work-group size) are
 * parameters: they only change work-group shapes / summation order.
 */
#define _GNU_SOURCE
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>
#include "cl_shim.h"

#include "dR_helper.cl"
#include "dR_winograd2.cl"
#include "dR_conv2d1x1.cl"
#include "dR_fcl.cl"
#include "dR_math.cl"
#include "dR_transform.cl"
/* generated pooling kernels the reference keeps beside its SqueezeNet model */
#include "Pool3x3_10_nocopyMax"
#include "Pool2x2_9_nocopyAverage"
#include "Pool14x14_46_nocopyAverage"

#define DR_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ emulator */
typedef void (*item_fn)(void *args);

static __thread size_t t_gsz[3], t_lsz[3], t_grp[3];
static __thread size_t t_item; /* linear local id of the running work-item */
static __thread ucontext_t t_sched;
static __thread ucontext_t *t_ctx;
static __thread char *t_stacks;
static __thread int *t_done;
static __thread size_t t_cap;
static __thread item_fn t_fn;
static __thread void *t_args;
static __thread int t_in_fiber;

#define FIBER_STACK (48 * 1024)

size_t get_local_size(unsigned d) { return t_lsz[d]; }
size_t get_global_size(unsigned d) { return t_gsz[d]; }
size_t get_num_groups(unsigned d) { return t_gsz[d] / t_lsz[d]; }
size_t get_group_id(unsigned d) { return t_grp[d]; }
size_t get_local_id(unsigned d)
{
    if (d == 0) return t_item % t_lsz[0];
    if (d == 1) return (t_item / t_lsz[0]) % t_lsz[1];
    return t_item / (t_lsz[0] * t_lsz[1]);
}
size_t get_global_id(unsigned d) { return t_grp[d] * t_lsz[d] + get_local_id(d); }

void barrier(int flags)
{
    (void)flags;
    if (t_in_fiber) {
        size_t me = t_item;
        swapcontext(&t_ctx[me], &t_sched);
        t_item = me;
    }
}

static void fiber_main(unsigned idx)
{
    t_item = idx;
    t_fn(t_args);
    t_done[idx] = 1;
    t_item = idx;
    swapcontext(&t_ctx[idx], &t_sched);
}

static void ensure_fibers(size_t n)
{
    if (t_cap >= n) return;
    free(t_ctx); free(t_stacks); free(t_done);
    t_ctx = (ucontext_t *)malloc(n * sizeof(ucontext_t));
    t_stacks = (char *)malloc(n * FIBER_STACK);
    t_done = (int *)malloc(n * sizeof(int));
    t_cap = n;
}

static void run_group(item_fn fn, void *args, size_t items, int uses_barrier)
{
    t_fn = fn; t_args = args;
    if (!uses_barrier) {
        t_in_fiber = 0;
        for (size_t i = 0; i < items; i++) { t_item = i; fn(args); }
        return;
    }
    ensure_fibers(items);
    t_in_fiber = 1;
    for (size_t i = 0; i < items; i++) {
        getcontext(&t_ctx[i]);
        t_ctx[i].uc_stack.ss_sp = t_stacks + i * FIBER_STACK;
        t_ctx[i].uc_stack.ss_size = FIBER_STACK;
        t_ctx[i].uc_link = &t_sched;
        t_done[i] = 0;
        makecontext(&t_ctx[i], (void (*)(void))fiber_main, 1, (unsigned)i);
    }
    size_t left = items;
    while (left) {
        left = 0;
        for (size_t i = 0; i < items; i++) {
            if (t_done[i]) continue;
            t_item = i;
            swapcontext(&t_sched, &t_ctx[i]);
            if (!t_done[i]) left++;
        }
    }
    t_in_fiber = 0;
}

/* NDRange over gsz with work-groups of lsz (lsz NULL: implementation-chosen,
 * here one item per group, which is legal for kernels without barriers). */
static void nd_range(item_fn fn, void *args, const size_t gsz[3], const size_t lsz_in[3], int uses_barrier)
{
    size_t lsz[3] = {1, 1, 1};
    if (lsz_in) { lsz[0] = lsz_in[0]; lsz[1] = lsz_in[1]; lsz[2] = lsz_in[2]; }
    else if (!uses_barrier) { lsz[0] = gsz[0]; } /* whole x-row per group: cheaper bookkeeping */
    const size_t ng0 = gsz[0] / lsz[0], ng1 = gsz[1] / lsz[1], ng2 = gsz[2] / lsz[2];
    const long total = (long)(ng0 * ng1 * ng2);
#pragma omp parallel for schedule(dynamic, 1)
    for (long g = 0; g < total; g++) {
        for (int d = 0; d < 3; d++) { t_gsz[d] = gsz[d]; t_lsz[d] = lsz[d]; }
        t_grp[0] = (size_t)g % ng0; t_grp[1] = ((size_t)g / ng0) % ng1; t_grp[2] = (size_t)g / (ng0 * ng1);
        run_group(fn, args, lsz[0] * lsz[1] * lsz[2], uses_barrier);
    }
}

/* ---------------------------------------------------- Winograd F(2x2,3x3) */
struct wino_args {
    const float *bias, *in, *U; float *out; int act, usebias, NperDim, OPart, INumPart, O, I, bW, bH, numWGx;
    size_t lmem_floats;
};
static __thread float *t_lmem; static __thread size_t t_lmem_cap;
static float *thread_lmem(size_t floats)
{
    if (t_lmem_cap < floats) { free(t_lmem); t_lmem = (float *)malloc(floats * sizeof(float)); t_lmem_cap = floats; }
    return t_lmem;
}
static void wino_item(void *p)
{
    struct wino_args *a = (struct wino_args *)p;
    conv2dwinograd2(a->bias, a->in, a->U, a->out, thread_lmem(a->lmem_floats), a->act, a->usebias, a->NperDim,
                    a->OPart, a->INumPart, a->O, a->I, a->bW, a->bH, a->numWGx);
}

/* Scheduling arithmetic of src/dR_nodes_conv2d.c:809-1006 (the non-"wide"
 * branch; the wide kernel is never selected below 256x256 inputs). */
static void wino_schedule(int W, int H, int I, int O, long lms, long mws,
                          int *NperDimOut, int *zOut, int *zInOut, int *wgx, int *wgy)
{
    int z = 1, zIn = 1, N = 1;
    long lmem = 16L * N * N * I * 4;
    while (O / z < I / zIn) zIn *= 2;
    long nw = (long)N * N * (O / z > I / zIn ? O / z : I / zIn);
    while (lmem < lms && nw <= mws / 2 && N * 2 < W && N * 2 < H) {
        N += 1;
        lmem = 16L * N * N * I * 4;
        nw = (long)N * N * (O / z > I / zIn ? O / z : I / zIn);
    }
    if (N > 1) N--;
    while ((W % (N * 2) > (W / 10) || H % (N * 2) > (H / 10)) && N > 4) N--;
    nw = (long)N * N * (O / z > I ? O / z : I / zIn);
    while (nw > mws / 2) {
        zIn *= 2; z *= 2;
        nw = (long)N * N * (O / z > I / zIn ? O / z : I / zIn);
    }
    int width = (W % (N * 2) == 0) ? W : ((W / (N * 2)) + 1) * (N * 2);
    int height = (H % (N * 2) == 0) ? H : ((H / (N * 2)) + 1) * (N * 2);
    *NperDimOut = N; *zOut = z; *zInOut = zIn; *wgx = width / (2 * N); *wgy = height / (2 * N);
}

/* Host filter transform U = G g G^T and re-layout [I][O][16] -> [I][16][O]:
 * src/dR_nodes_conv2d.c:1162-1240 (naive matmuls of src/dR_core.c:677-723). */
static float *wino_transform_filters(const float *w, int I, int O)
{
    static const float G[12] = {1.f, 0.f, 0.f, .5f, .5f, .5f, .5f, -.5f, .5f, 0.f, 0.f, 1.f};
    float *U = (float *)malloc((size_t)16 * I * O * sizeof(float));
    for (int i = 0; i < I; i++)
        for (int o = 0; o < O; o++) {
            const float *g = w + ((size_t)i * O + o) * 9;
            float t[12], u[16];
            for (int r = 0; r < 4; r++)
                for (int c = 0; c < 3; c++) {
                    float s = 0.f;
                    for (int k = 0; k < 3; k++) s += G[r * 3 + k] * g[k * 3 + c];
                    t[r * 3 + c] = s;
                }
            for (int r = 0; r < 4; r++)
                for (int c = 0; c < 4; c++) {
                    float s = 0.f;
                    for (int k = 0; k < 3; k++) s += t[r * 3 + k] * G[c * 3 + k];
                    u[r * 4 + c] = s;
                }
            for (int k = 0; k < 16; k++) U[(size_t)i * O * 16 + (size_t)k * O + o] = u[k];
        }
    return U;
}

/* Launch geometry of src/dR_nodes_conv2d.c:1009-1132.  in/out: n images, z-major. */
DR_EXPORT int drref_conv2d_winograd(const float *in, int n, int W, int H, int I, const float *w, const float *bias,
                                    int O, int act, long lms, long mws, float *out)
{
    int N, z, zIn, wgx, wgy;
    wino_schedule(W, H, I, O, lms, mws, &N, &z, &zIn, &wgx, &wgy);
    if (16L * N * N * I * 4 > lms) return -1;
    float *U = wino_transform_filters(w, I, O);
    int maxDepth = (O / z > I) ? O / z : I / zIn;
    size_t lsz[3] = {(size_t)N * N, (size_t)maxDepth, 1};
    size_t gsz[3] = {(size_t)N * N * wgx * wgy, (size_t)maxDepth * z, 1};
    for (int b = 0; b < n; b++) {
        struct wino_args a = {bias, in + (size_t)b * W * H * I, U, out + (size_t)b * W * H * O, act ? 1 : 0,
                              bias ? 1 : 0, N, O / z, zIn, O, I, W, H, wgx, (size_t)16 * N * N * I};
        nd_range(wino_item, &a, gsz, lsz, 1);
    }
    free(U);
    return N;
}

/* ------------------------------------------------------------------ 1x1 conv */
struct c11_args { const float *bias, *in, *wt; float *out; int usebias, act, O, I, bW, bH; };
static void c11_item(void *p)
{
    struct c11_args *a = (struct c11_args *)p;
    conv2d1x1(a->bias, a->in, a->wt, a->out, thread_lmem((size_t)a->I), a->usebias, a->act, a->O, a->I, a->bW, a->bH);
}
/* Schedule src/dR_nodes_conv2d.c:1526-1603, transpose :1696-1716, launch :1605-1672. */
DR_EXPORT int drref_conv2d_1x1(const float *in, int n, int W, int H, int I, const float *w, const float *bias,
                               int O, int act, long mws, float *out)
{
    int lws = 16;
    while (lws < W && lws < H && (long)lws * lws <= mws) lws *= 2;
    lws /= 2;
    size_t gx = (W % lws == 0) ? W : ((W / lws) + 1) * lws;
    size_t gy = (H % lws == 0) ? H : ((H / lws) + 1) * lws;
    float *wt = (float *)malloc((size_t)I * O * sizeof(float));
    for (int i = 0; i < I; i++)
        for (int o = 0; o < O; o++) wt[(size_t)o * I + i] = w[(size_t)i * O + o];
    float dummy = 0.f;
    size_t lsz[3] = {(size_t)lws, (size_t)lws, 1}, gsz[3] = {gx, gy, (size_t)O};
    for (int b = 0; b < n; b++) {
        struct c11_args a = {bias ? bias : &dummy, in + (size_t)b * W * H * I, wt, out + (size_t)b * W * H * O,
                             bias ? 1 : 0, act ? 1 : 0, O, I, W, H};
        nd_range(c11_item, &a, gsz, lsz, 1);
    }
    free(wt);
    return lws;
}

/* ------------------------------------------------------------ fully connected */
struct fc1_args { const float *in, *w; float *out; int Nin, Nout, part, sx, sy, sz; };
static void fc1_item(void *p)
{
    struct fc1_args *a = (struct fc1_args *)p;
    matrixVectorMultFirst(a->in, a->w, thread_lmem((size_t)a->part), a->out, a->Nin, a->Nout, a->part, a->sx, a->sy, a->sz);
}
struct fc2_args { float *io; const float *bias; int usebias, act, Nout, parts; };
static void fc2_item(void *p)
{
    struct fc2_args *a = (struct fc2_args *)p;
    matrixVectorMultSecond(a->io, (float *)a->bias, a->usebias, a->act, a->Nout, a->parts);
}
/* Schedule src/dR_nodes_fc.c:114-199, launches :201-278.  The reference stores the
 * partial sums in the node's own output buffer; here a scratch of the needed size. */
DR_EXPORT int drref_fc(const float *in, int n, int W, int H, int C, const float *w, const float *bias, int Nout,
                       int act, long lms, long mws, float *out)
{
    const int Nin = W * H * C;
    int lws = Nout, z = Nin;
    while (lws > mws) { if (lws % 2 == 0) lws /= 2; else lws /= 2 + 1; }
    long lmem = (long)z * 4;
    while (lmem > lms) { if (z % 2 == 0) z /= 2; else z /= 2 + 1; lmem = (long)z * 4; }
    long nwg = (long)Nout / lws * Nin / z;
    while (nwg < 60 && z != 1) { if (z % 2 == 0) z /= 2; else z /= 2 + 1; nwg = (long)Nout / lws * Nin / z; }
    size_t gx = (size_t)Nout + (Nout % lws);
    size_t gy = (Nin % z != 0) ? (size_t)(Nin / z) + 1 : (size_t)(Nin / z);
    if (gx % lws != 0 || Nin % z != 0) return -1; /* shapes the reference itself mishandles */
    float dummy = 0.f;
    float *partial = (float *)malloc(gx * gy * sizeof(float));
    for (int b = 0; b < n; b++) {
        struct fc1_args a1 = {in + (size_t)b * Nin, w, partial, Nin, Nout, z, W, H, C};
        size_t g1[3] = {gx, gy, 1}, l1[3] = {(size_t)lws, 1, 1};
        nd_range(fc1_item, &a1, g1, l1, 1);
        struct fc2_args a2 = {partial, bias ? bias : &dummy, bias ? 1 : 0, act ? 1 : 0, Nout, Nin / z};
        size_t g2[3] = {(size_t)Nout, 1, 1};
        nd_range(fc2_item, &a2, g2, NULL, 0);
        memcpy(out + (size_t)b * Nout, partial, (size_t)Nout * sizeof(float));
    }
    free(partial);
    return z;
}

/* -------------------------------------------------------------------- pooling */
struct pool_args { const float *in; float *out; int W, H, C, sx, sy, sz, stx, sty, stz, which; };
static void pool_item(void *p)
{
    struct pool_args *a = (struct pool_args *)p;
    if (a->which == 0) Pool3x3_10_nocopyMax(a->in, a->out, a->W, a->H, a->C, a->sx, a->sy, a->sz, a->stx, a->sty, a->stz);
    else if (a->which == 1) Pool2x2_9_nocopyAverage(a->in, a->out, a->W, a->H, a->C, a->sx, a->sy, a->sz, a->stx, a->sty, a->stz);
    else Pool14x14_46_nocopyAverage(a->in, a->out, a->W, a->H, a->C, a->sx, a->sy, a->sz, a->stx, a->sty, a->stz);
}
/* which: 0 = 3x3 max, 1 = 2x2 average, 2 = 14x14 average (the three generated
 * kernels the reference ships); launch as src/dR_nodes_pooling.c:138-183. */
DR_EXPORT int drref_pool(const float *in, int n, int W, int H, int C, int which, int stx, int sty, float *out)
{
    int k = which == 0 ? 3 : (which == 1 ? 2 : 14);
    int Wo = (W + stx - 1) / stx, Ho = (H + sty - 1) / sty;
    size_t gsz[3] = {(size_t)Wo, (size_t)Ho, (size_t)C};
    for (int b = 0; b < n; b++) {
        struct pool_args a = {in + (size_t)b * W * H * C, out + (size_t)b * Wo * Ho * C, W, H, C, k, k, 1, stx, sty, 1, which};
        nd_range(pool_item, &a, gsz, NULL, 0);
    }
    return 0;
}

/* ------------------------------------------------------ element-wise, softmax */
struct ew_args { const float *a, *b; float *out; float s; int op; };
static void ew1_item(void *p)
{
    struct ew_args *a = (struct ew_args *)p;
    switch (a->op) {
    case 0: addScalar(a->a, a->out, a->s); break;
    case 1: subScalar(a->a, a->out, a->s); break;
    case 2: mulScalar((float *)a->a, a->out, a->s); break;
    case 3: divScalar((float *)a->a, a->out, a->s); break;
    case 4: computeLog(a->a, a->out); break;
    case 5: computeExp((float *)a->a, a->out); break;
    case 6: computeSqrt((float *)a->a, a->out); break;
    case 7: fill((float *)a->a, a->out, a->s); break;
    case 8: powScalar((float *)a->a, a->out, a->s); break;
    }
}
static void ew2_item(void *p)
{
    struct ew_args *a = (struct ew_args *)p;
    switch (a->op) {
    case 0: elemWiseAdd(a->a, a->b, a->out); break;
    case 1: elemWiseSub(a->a, a->b, a->out); break;
    case 2: elemWiseMul(a->a, a->b, a->out); break;
    case 3: elemWiseDiv(a->a, a->b, a->out); break;
    case 4: elemWisePow(a->a, a->b, a->out); break;
    }
}
/* Launch shapes of src/dR_nodes_math.c:349-376 / :99-123 (global = tensor shape). */
DR_EXPORT void drref_elemwise1(const float *in, int W, int H, int C, int op, float s, float *out)
{
    struct ew_args a = {in, NULL, out, s, op};
    size_t gsz[3] = {(size_t)W, (size_t)H, (size_t)C};
    nd_range(ew1_item, &a, gsz, NULL, 0);
}
DR_EXPORT void drref_elemwise2(const float *x, const float *y, int W, int H, int C, int op, float *out)
{
    struct ew_args a = {x, y, out, 0.f, op};
    size_t gsz[3] = {(size_t)W, (size_t)H, (size_t)C};
    nd_range(ew2_item, &a, gsz, NULL, 0);
}
/* Softmax = computeExp kernel, serial host sum, mulScalar kernel: src/dR_nodes_math.c:620-678. */
DR_EXPORT void drref_softmax(const float *in, int W, int H, int C, float *out)
{
    drref_elemwise1(in, W, H, C, 5, 0.f, out);
    float sum = 0.0f;
    for (int i = 0; i < W * H * C; i++) sum += out[i];
    sum = 1 / sum;
    drref_elemwise1(out, W, H, C, 2, sum, out);
}

/* --------------------------------------------------------- slice, crop-or-pad */
struct tr_args { const float *in; float *out; int o0, o1, o2, s0, s1, s2, i0, i1, i2, which; };
static void tr_item(void *p)
{
    struct tr_args *a = (struct tr_args *)p;
    if (a->which == 0) extractSlice(a->in, a->out, a->o0, a->o1, a->o2, a->s0, a->s1, a->s2, a->i0, a->i1, a->i2);
    else cropOrPad(a->in, a->out, a->s0, a->s1, a->s2, a->i0, a->i1, a->i2);
}
/* 1-D launches over the output: src/dR_nodes_transform.c:123-153 and the CropOrPad twin. */
DR_EXPORT void drref_slice(const float *in, int W, int H, int C, int ox, int oy, int oz, int w, int h, int c, float *out)
{
    struct tr_args a = {in, out, ox, oy, oz, w, h, c, W, H, C, 0};
    size_t gsz[3] = {(size_t)w * h * c, 1, 1};
    nd_range(tr_item, &a, gsz, NULL, 0);
}
DR_EXPORT void drref_croporpad(const float *in, int W, int H, int C, int w, int h, int c, float *out)
{
    struct tr_args a = {in, out, 0, 0, 0, w, h, c, W, H, C, 1};
    size_t gsz[3] = {(size_t)w * h * c, 1, 1};
    nd_range(tr_item, &a, gsz, NULL, 0);
}
