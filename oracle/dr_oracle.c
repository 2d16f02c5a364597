/*
 * CPU oracle for the deepRacin CNN-layer hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic the reference performs for Conv2d,
 * FullyConnected, Pooling, Softmax, element-wise math and the Slice / Concat /
 * CropOrPad copies.  It exists to check the CUDA library; nothing in the shipped
 * library links, loads or calls it.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may use it.
 *
 * Layout conventions are the reference's own: a tensor is W x H x C stored
 * "z major, x minor" (index = z*W*H + y*W + x), weights of a convolution are
 * [Cin][Cout][kh][kw], weights of a fully connected layer are [Nin][Nout] with
 * the input flattened in (y, x, z)-order.  A batch is simply `n` such tensors
 * stored back to back (the reference itself loops over images on the host).
 *
 * Pinning: this restatement is checked (tests/test_oracle.py) against
 *   - the reference's own kernel sources compiled as C (oracle/ref_shim), and
 *   - the only known answers the reference holds: the pretrained SqueezeNet
 *     graph classifying its two example images as classes 292 and 611
 *     (examples/squeezenet-v1.1/squeezenet_deployed.c:199-207).
 * FullyConnected has no fixture in the reference (VGG weights are not shipped):
 * its parity is pinned by the compiled reference kernels only.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define DR_EXPORT __attribute__((visibility("default")))

/* Zero padding rule of the reference: Kernels/dR_helper.cl:15-28. */
static inline float sample_zero(const float *img, int x, int y, int w, int h)
{
    if (x < 0 || x >= w || y < 0 || y >= h)
        return 0.0f;
    return img[(size_t)y * w + x];
}

/* ReLU / linear as the kernels write them: clamp(v, 0, FLT_MAX)
 * (Kernels/dR_conv2d1x1.cl:45-52, Kernels/dR_winograd2.cl:228-235). */
static inline float activate(double v, int act)
{
    float f = (float)v;
    if (act == 1) {
        if (!(f > 0.0f)) f = 0.0f;
        if (f > FLT_MAX) f = FLT_MAX;
    }
    return f;
}

/*
 * Convolution with "same" zero padding, correlation form, optional stride:
 *   out[o,y,x] = act(b[o] + sum_{i,ky,kx} in[i, y*sy+ky-kh/2, x*sx+kx-kw/2] * w[i,o,ky,kx])
 * Formula: include/dR_nodes_conv2d.h:47-54; output size W/sx x H/sy (integer
 * division): src/dR_nodes_conv2d.c:115-117.  Accumulates in double so that the
 * result is independent of the summation order any implementation picks.
 */
DR_EXPORT void dro_conv2d(const float *in, int n, int W, int H, int Cin,
                          const float *w, const float *bias, int kw, int kh, int Cout,
                          int sx, int sy, int act, float *out)
{
    const int Wo = W / sx, Ho = H / sy;
    const int px = kw / 2, py = kh / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; b++)
        for (int o = 0; o < Cout; o++) {
            const float *img = in + (size_t)b * W * H * Cin;
            float *dst = out + ((size_t)b * Cout + o) * Wo * Ho;
            for (int y = 0; y < Ho; y++)
                for (int x = 0; x < Wo; x++) {
                    double acc = bias ? (double)bias[o] : 0.0;
                    for (int i = 0; i < Cin; i++) {
                        const float *plane = img + (size_t)i * W * H;
                        const float *f = w + ((size_t)i * Cout + o) * kh * kw;
                        for (int ky = 0; ky < kh; ky++)
                            for (int kx = 0; kx < kw; kx++)
                                acc += (double)sample_zero(plane, x * sx + kx - px, y * sy + ky - py, W, H) *
                                       (double)f[ky * kw + kx];
                    }
                    dst[(size_t)y * Wo + x] = activate(acc, act);
                }
        }
}

/*
 * Winograd F(2x2,3x3) in the reference's own arithmetic (single precision,
 * channel-ordered accumulation), i.e. the same transform matrices and the same
 * order of operations as Kernels/dR_winograd2.cl:55-251 with the host filter
 * transform of src/dR_nodes_conv2d.c:1162-1240.  Used to bound the rounding
 * difference between transform-domain and direct evaluation.
 */
static void wino_filter_transform(const float *g, float *u)
{
    /* U = G g G^T, G = [[1,0,0],[.5,.5,.5],[.5,-.5,.5],[0,0,1]] */
    static const float G[4][3] = {{1.f, 0.f, 0.f}, {.5f, .5f, .5f}, {.5f, -.5f, .5f}, {0.f, 0.f, 1.f}};
    float t[4][3];
    for (int r = 0; r < 4; r++)
        for (int c = 0; c < 3; c++) {
            float s = 0.f;
            for (int k = 0; k < 3; k++) s += G[r][k] * g[k * 3 + c];
            t[r][c] = s;
        }
    for (int r = 0; r < 4; r++)
        for (int c = 0; c < 4; c++) {
            float s = 0.f;
            for (int k = 0; k < 3; k++) s += t[r][k] * G[c][k];
            u[r * 4 + c] = s;
        }
}

DR_EXPORT void dro_conv2d_winograd(const float *in, int n, int W, int H, int Cin,
                                   const float *w, const float *bias, int Cout, int act, float *out)
{
    float *U = (float *)malloc((size_t)Cin * Cout * 16 * sizeof(float));
    for (int i = 0; i < Cin; i++)
        for (int o = 0; o < Cout; o++)
            wino_filter_transform(w + ((size_t)i * Cout + o) * 9, U + ((size_t)i * Cout + o) * 16);
    const int tx = (W + 1) / 2, ty = (H + 1) / 2;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; b++)
        for (int t = 0; t < tx * ty; t++) {
            const float *img = in + (size_t)b * W * H * Cin;
            const int ox = (t % tx) * 2, oy = (t / tx) * 2;
            float *V = (float *)malloc((size_t)Cin * 16 * sizeof(float));
            for (int i = 0; i < Cin; i++) {
                const float *p = img + (size_t)i * W * H;
                float d[4][4], m[16];
                for (int r = 0; r < 4; r++)
                    for (int c = 0; c < 4; c++) d[r][c] = sample_zero(p, ox - 1 + c, oy - 1 + r, W, H);
                /* rows: B^T d with B^T = [[1,0,-1,0],[0,1,1,0],[0,-1,1,0],[0,-1,0,1]] */
                for (int c = 0; c < 4; c++) {
                    m[0 + c] = d[0][c] - d[2][c];
                    m[4 + c] = d[1][c] + d[2][c];
                    m[8 + c] = -d[1][c] + d[2][c];
                    m[12 + c] = -d[1][c] + d[3][c];
                }
                /* columns: (.) B */
                for (int r = 0; r < 4; r++) {
                    float a0 = m[r * 4], a1 = m[r * 4 + 1], a2 = m[r * 4 + 2], a3 = m[r * 4 + 3];
                    V[i * 16 + r * 4 + 0] = a0 - a2;
                    V[i * 16 + r * 4 + 1] = a1 + a2;
                    V[i * 16 + r * 4 + 2] = -a1 + a2;
                    V[i * 16 + r * 4 + 3] = -a1 + a3;
                }
            }
            for (int o = 0; o < Cout; o++) {
                float m[16];
                for (int k = 0; k < 16; k++) m[k] = 0.f;
                for (int i = 0; i < Cin; i++) {
                    const float *u = U + ((size_t)i * Cout + o) * 16;
                    for (int k = 0; k < 16; k++) m[k] = fmaf(V[i * 16 + k], u[k], m[k]);
                }
                float s[8];
                for (int r = 0; r < 4; r++) {
                    s[r * 2 + 0] = m[r * 4 + 0] + m[r * 4 + 1] + m[r * 4 + 2];
                    s[r * 2 + 1] = m[r * 4 + 1] - m[r * 4 + 2] + m[r * 4 + 3];
                }
                float y00 = s[0] + s[2] + s[4], y01 = s[1] + s[3] + s[5];
                float y10 = s[2] - s[4] + s[6], y11 = s[3] - s[5] + s[7];
                if (bias) { y00 += bias[o]; y01 += bias[o]; y10 += bias[o]; y11 += bias[o]; }
                float *dst = out + ((size_t)b * Cout + o) * W * H;
                dst[(size_t)oy * W + ox] = activate(y00, act);
                if (ox + 1 < W) dst[(size_t)oy * W + ox + 1] = activate(y01, act);
                if (oy + 1 < H) {
                    dst[(size_t)(oy + 1) * W + ox] = activate(y10, act);
                    if (ox + 1 < W) dst[(size_t)(oy + 1) * W + ox + 1] = activate(y11, act);
                }
            }
            free(V);
        }
    free(U);
}

/*
 * Fully connected layer: out[o] = act(b[o] + sum_k in_hwc[k] * w[k*Nout + o]) where
 * in_hwc[k] reads the z-major input through the (y,x,z)-order mapping of
 * Kernels/dR_helper.cl:131-142 (used at Kernels/dR_fcl.cl:78); linear output is
 * clamp(v,-FLT_MAX,FLT_MAX) (Kernels/dR_fcl.cl:116-119).
 */
DR_EXPORT void dro_fc(const float *in, int n, int W, int H, int C, const float *w,
                      const float *bias, int Nout, int act, float *out)
{
    const int Nin = W * H * C;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; b++)
        for (int o = 0; o < Nout; o++) {
            const float *img = in + (size_t)b * Nin;
            double acc = bias ? (double)bias[o] : 0.0;
            for (int k = 0; k < Nin; k++) {
                int z = k % C, x = (k / C) % W, y = (k / C) / W;
                acc += (double)img[(size_t)z * W * H + (size_t)y * W + x] * (double)w[(size_t)k * Nout + o];
            }
            float f = (float)acc;
            if (act == 1) { if (!(f > 0.f)) f = 0.f; }
            if (f > FLT_MAX) f = FLT_MAX;
            if (f < -FLT_MAX) f = -FLT_MAX;
            out[(size_t)b * Nout + o] = f;
        }
}

/*
 * Pooling as generated by src/dR_nodes_pooling.c:277-401: the window of output
 * (x,y,z) starts at (x*stx, y*sty, z*stz) (top-left anchored), reads outside the
 * image in x/y return 0 and take part in the result, max starts at -FLT_MAX,
 * average always divides by the full window size.  Output size is ceil(in/stride)
 * per axis (src/dR_nodes_pooling.c:186-224).  Channels past the end read as 0
 * here (the reference does not bound-check z).
 */
DR_EXPORT void dro_pool(const float *in, int n, int W, int H, int C, int sx, int sy, int sz,
                        int stx, int sty, int stz, int type, float *out)
{
    const int Wo = (W + stx - 1) / stx, Ho = (H + sty - 1) / sty, Co = (C + stz - 1) / stz;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < n; b++)
        for (int z = 0; z < Co; z++)
            for (int y = 0; y < Ho; y++)
                for (int x = 0; x < Wo; x++) {
                    const float *img = in + (size_t)b * W * H * C;
                    float res = type == 0 ? -FLT_MAX : 0.0f;
                    for (int dz = 0; dz < sz; dz++)
                        for (int dy = 0; dy < sy; dy++)
                            for (int dx = 0; dx < sx; dx++) {
                                int iz = z * stz + dz;
                                float v = iz < C ? sample_zero(img + (size_t)iz * W * H, x * stx + dx, y * sty + dy, W, H) : 0.f;
                                if (type == 0) res = res > v ? res : v;
                                else res += v;
                            }
                    if (type != 0) res = res / (float)(sx * sy * sz);
                    out[(((size_t)b * Co + z) * Ho + y) * Wo + x] = res;
                }
}

/*
 * Softmax exactly as src/dR_nodes_math.c:620-678 does it: exp of every element,
 * a serial single-precision sum over the WHOLE tensor on the host, then a multiply
 * by 1/sum.  No maximum is subtracted, so logits above ~88 overflow.
 */
DR_EXPORT void dro_softmax(const float *in, int n, int len, float *out)
{
    for (int b = 0; b < n; b++) {
        const float *x = in + (size_t)b * len;
        float *y = out + (size_t)b * len;
        float sum = 0.0f;
        for (int i = 0; i < len; i++) { y[i] = expf(x[i]); sum += y[i]; }
        float inv = 1 / sum;
        for (int i = 0; i < len; i++) y[i] = y[i] * inv;
    }
}

/* Element-wise ops with a scalar; op codes of include/dR_nodes_math.h:82-92,
 * kernels Kernels/dR_math.cl:176-342. */
DR_EXPORT void dro_elemwise1(const float *in, size_t len, int op, float s, float *out)
{
    for (size_t i = 0; i < len; i++) {
        float v = in[i], r;
        switch (op) {
        case 0: r = v + s; break;
        case 1: r = v - s; break;
        case 2: r = v * s; break;
        case 3: r = v / s; break;
        case 4: r = logf(v); break;
        case 5: r = expf(v); break;
        case 6: r = sqrtf(v); break;
        case 7: r = s; break;
        case 8: r = powf(v, s); break;
        default: r = v;
        }
        out[i] = r;
    }
}

/* Element-wise binary ops; codes of include/dR_nodes_math.h:10-16,
 * kernels Kernels/dR_math.cl:30-125. */
DR_EXPORT void dro_elemwise2(const float *a, const float *b, size_t len, int op, float *out)
{
    for (size_t i = 0; i < len; i++) {
        float r;
        switch (op) {
        case 0: r = a[i] + b[i]; break;
        case 1: r = a[i] - b[i]; break;
        case 2: r = a[i] * b[i]; break;
        case 3: r = a[i] / b[i]; break;
        case 4: r = powf(a[i], b[i]); break;
        default: r = a[i];
        }
        out[i] = r;
    }
}

/* Slice: out[z,y,x] = in[oz+z, oy+y, ox+x] (Kernels/dR_transform.cl:5-25). */
DR_EXPORT void dro_slice(const float *in, int n, int W, int H, int C, int ox, int oy, int oz,
                         int w, int h, int c, float *out)
{
    for (int b = 0; b < n; b++)
        for (int z = 0; z < c; z++)
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w; x++)
                    out[(((size_t)b * c + z) * h + y) * w + x] =
                        in[(((size_t)b * C + oz + z) * H + oy + y) * W + ox + x];
}

/* CropOrPad: same coordinates, zero outside the source in x/y
 * (Kernels/dR_transform.cl:32-48); channels past the source read 0 here. */
DR_EXPORT void dro_croporpad(const float *in, int n, int W, int H, int C, int w, int h, int c, float *out)
{
    for (int b = 0; b < n; b++)
        for (int z = 0; z < c; z++)
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w; x++)
                    out[(((size_t)b * c + z) * h + y) * w + x] =
                        z < C ? sample_zero(in + ((size_t)b * C + z) * W * H, x, y, W, H) : 0.0f;
}

/*
 * Concat of one input into the output at a running offset along dim (0=x,1=y,2=z);
 * the caller walks the inputs in list order (src/dR_nodes_transform.c:377-401,
 * 468-553).  `off` is the sum of the earlier inputs' extents along dim.
 */
DR_EXPORT void dro_concat_place(const float *in, int n, int w, int h, int c, int dim, int off,
                                int W, int H, int C, float *out)
{
    for (int b = 0; b < n; b++)
        for (int z = 0; z < c; z++)
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w; x++) {
                    int X = x + (dim == 0 ? off : 0), Y = y + (dim == 1 ? off : 0), Z = z + (dim == 2 ? off : 0);
                    out[(((size_t)b * C + Z) * H + Y) * W + X] = in[(((size_t)b * c + z) * h + y) * w + x];
                }
}
