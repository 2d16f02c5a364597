/*
 * Operator-level C ABI of the CUDA kernels (sm_100a).  Plain pointers and sizes only;
 * every pointer is a DEVICE pointer unless stated, `stream` is a cudaStream_t passed as
 * void*.  Every function only enqueues work and returns 0 or a cudaError_t value
 * (negative values: argument errors).  These are the entry points the graph nodes call;
 * each replaces one OpenCL kernel + its host-side `*_compute` launcher of the reference.
 *
 * Activations are N-HWC: element (image b, row y, column x, channel c) of a W x H x C
 * tensor lives at ((b*H + y)*W + x)*ld + c, ld >= C being the pixel stride in floats.
 */
#ifndef DR_KERNELS_H
#define DR_KERNELS_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef void *dRk_stream;

/* Interface layout <-> internal layout.  The reference's buffers are [C][H][W]
 * (include/deepRACIN.h:61); its Python layer transposes on the host
 * (python/deepracin/__init__.py.in:458-462, 487-489). */
int dRk_chw_to_hwc(dRk_stream stream, const float *src, float *dst, int n, int W, int H, int C);
int dRk_hwc_to_chw(dRk_stream stream, const float *src, float *dst, int n, int W, int H, int C);

/*
 * Convolution, exact FP32 (FFMA) implicit GEMM over M = n*Ho*Wo pixels, N = Cout,
 * K = kh*kw*Cin; fused bias and ReLU(clamp to [0,FLT_MAX]) / linear.  Any odd or even
 * filter size and any stride; padding and anchoring as include/dR_nodes_conv2d.h:47-54.
 * Replaces the generated direct kernel (src/dR_nodes_conv2d.c:481-773, launcher :364-420)
 * and, for 1x1 filters, Kernels/dR_conv2d1x1.cl:4-53 (launcher :1605-1672).
 *   wpack : [kh*kw*Cin][Cout], row k = (ky*kw + kx)*Cin + c
 *   ldi   : pixel stride of `in`;  ldo/coff : pixel stride / channel offset of `out`
 */
int dRk_conv2d_f32(dRk_stream stream, const float *in, const float *wpack, const float *bias, float *out,
                   int n, int W, int H, int Cin, int Cout, int kw, int kh, int sx, int sy, int act,
                   int ldi, int ldo, int coff);

/*
 * Winograd F(2x2,3x3) convolution, exact FP32, as three launches: input transform
 * V = B^T d B per 4x4 tile, 16 transform-domain GEMMs M_k = V_k U_k, inverse transform
 * A^T M A + bias + activation.  Transform matrices are the reference's
 * (Kernels/dR_winograd2.cl:55-251); U = G g G^T is computed on the host as in
 * src/dR_nodes_conv2d.c:1162-1240 and passed as [16][Cin][Cout].
 * scratch must hold dRk_winograd_scratch_floats() floats.
 */
size_t dRk_winograd_scratch_floats(int n, int W, int H, int Cin, int Cout);
int dRk_conv2d_winograd_f32(dRk_stream stream, const float *in, const float *U, const float *bias, float *out,
                            float *scratch, int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff);

/*
 * The same convolution (conv2dwinograd2, Kernels/dR_winograd2.cl:23-254) as Winograd F(4x4,3x3) in FP32: 6x6 input tiles,
 * 36 transform-domain GEMMs, 4x4 outputs per tile; 4x fewer multiplications than the direct sum (F(2x2,3x3): 2.25x) at an
 * error of about 1e-5 of max|ref| (inside the FP32 class bound of 1e-4, above F(2x2,3x3)'s 1e-6).  U = G g G^T as
 * [36][Cin][Cout] from dRk_winograd4_pack_weights (w is the reference's [Cin][Cout][3][3] filter array);
 * scratch must hold dRk_winograd4_scratch_floats() floats.  pool = 1: the 2x2/2 max pooling that follows the layer
 * (src/dR_nodes_pooling.c:138-183) is evaluated by the output transform and out is the pooled [n][H/2][W/2] tensor (W, H even).
 */
size_t dRk_winograd4_scratch_floats(int n, int W, int H, int Cin, int Cout);
int dRk_winograd4_pack_weights(const float *w, float *U, int Cin, int Cout);
int dRk_conv2d_winograd4_f32(dRk_stream stream, const float *in, const float *U, const float *bias, float *out,
                             float *scratch, int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff, int pool);

/*
 * Fully connected layer out[b][o] = act(bias[o] + sum_k in[b][k] * w[k][o]); `in` is the
 * N-HWC activation, whose flattening is exactly the (y,x,z) order the reference's kernel
 * reads through mapToDepthMajor (Kernels/dR_fcl.cl:59-120, Kernels/dR_helper.cl:131-142).
 * Weight-streaming split-K kernel for small batches (partials in `scratch`, reduced by a
 * second launch like the reference's matrixVectorMultSecond), FFMA GEMM for large ones.
 * Linear output is clamped to [-FLT_MAX, FLT_MAX], ReLU to [0, FLT_MAX].
 */
size_t dRk_fc_scratch_floats(int n, int Nin, int Nout);
int dRk_fc_f32(dRk_stream stream, const float *in, const float *w, const float *bias, float *out, float *scratch,
               int n, int Nin, int Nout, int act);

/*
 * dRk_fc_f32 for callers that must not allocate device memory while running (embedders with a memory
 * budget frozen after start-up, plug-in hosts that own every device allocation).  No counterpart in the
 * reference.  The split-K scratch is a fixed 8 MiB array inside the library (2 Mi floats, resident on
 * every GPU that loads the library); shapes needing more (dRk_fc_scratch_floats) are refused with -4.
 * The first call on a device resolves the array's address -- make it before any stream capture; calls
 * share the array, so calls that may overlap on the GPU race.  The stream's device must be the current device (-6 otherwise).
 * Allocates nothing.
 */
int dRk_fc_f32_noalloc(dRk_stream stream, const float *in, const float *w, const float *bias, float *out,
                       int n, int Nin, int Nout, int act);

/* out[i] = (float)in[i] for 8-bit image samples (both pointers 16-byte aligned); replaces the host-side cast of the reference's
 * examples (examples/vgg16/vgg_deployed.c:153-157). */
int dRk_u8_to_f32(dRk_stream stream, const unsigned char *in, float *out, size_t count);

/* Max / average pooling with the reference's window rule (src/dR_nodes_pooling.c:277-401,
 * launcher :138-183): top-left anchored windows, zero reads outside, average over the full
 * window.  type 0 = max, 1 = average.  Output is dense N-HWC of ceil(in/stride) per axis. */
int dRk_pool(dRk_stream stream, const float *in, float *out, int n, int W, int H, int C, int sx, int sy, int sz,
             int stx, int sty, int stz, int type, int ldi);

/* Softmax over each image's whole tensor, one fused kernel: exp(x - max) / sum.  Equal to
 * the reference's computeExp + host sum + mulScalar (src/dR_nodes_math.c:620-678) wherever
 * that is finite. */
int dRk_softmax(dRk_stream stream, const float *in, float *out, int n, int len);

/* Element-wise ops; op codes of include/dR_nodes_math.h:10-16 and :82-92
 * (Kernels/dR_math.cl:30-342). */
int dRk_elemwise1(dRk_stream stream, const float *in, float *out, size_t len, int op, float scalar);
int dRk_elemwise2(dRk_stream stream, const float *a, const float *b, float *out, size_t len, int op);

/* Slice (Kernels/dR_transform.cl:5-25), CropOrPad (:32-48) and the placement of one Concat
 * input at a running offset along dim 0=x / 1=y / 2=z (generated kernel,
 * src/dR_nodes_transform.c:468-553).  Shapes are (W,H,C) of source and destination. */
int dRk_slice(dRk_stream stream, const float *in, float *out, int n, int W, int H, int C, int ox, int oy, int oz,
              int w, int h, int c, int ldi);
int dRk_croporpad(dRk_stream stream, const float *in, float *out, int n, int W, int H, int C, int w, int h, int c, int ldi);
int dRk_concat_place(dRk_stream stream, const float *in, float *out, int n, int w, int h, int c, int dim, int off,
                     int W, int H, int C, int ldi);

/* Fused Slice -> scalar element-wise chain -> Concat along channels: output channel j of every pixel is
 * source channel ch[j] of src[j] (pixel stride ld[j]) pushed through up to 4 scalar ops (codes of
 * dRk_elemwise1) in order.  Replaces extractSlice + the scalar kernels + the generated concat kernel
 * (Kernels/dR_transform.cl:5-25, Kernels/dR_math.cl:176-260, src/dR_nodes_transform.c:468-553) for that pattern. */
#define DRK_CHANNEL_MAP_MAX 16
typedef struct {
    const float *src[DRK_CHANNEL_MAP_MAX];
    int ld[DRK_CHANNEL_MAP_MAX], ch[DRK_CHANNEL_MAP_MAX], nops[DRK_CHANNEL_MAP_MAX];
    int op[DRK_CHANNEL_MAP_MAX][4];
    float scalar[DRK_CHANNEL_MAP_MAX][4];
    int cout;
} drk_ChannelMap;
int dRk_channel_map(dRk_stream stream, const drk_ChannelMap *map, float *out, size_t pixels);

/*
 * Tensor-core convolution / GEMM: tcgen05.mma kind::tf32 with FP32 accumulators in TMEM,
 * operands staged by TMA (cp.async.bulk.tensor) into 128B-swizzled shared memory.
 * The plan object owns the CUtensorMap descriptors for one layer shape + buffer set.
 *   in   : N-HWC, dense (ldi == Cin), Cin a multiple of 4 and >= 8; or 3x3 filters with Cin <= 4 and
 *          16 <= Cout <= 128 (first-layer kernel: the patch operand is gathered by producer warps, no TMA)
 *   wT   : [Cout][kh*kw*CinPad] (K contiguous), k = (ky*kw + kx)*CinPad + c, CinPad = dRk_tensor_conv_cin_pad(Cin):
 *          Cin rounded up to a multiple of 32 with the padding filled with zeros, or Cin itself when Cin <= 4
 * Returns NULL if the shape is not supported by the tensor path (caller falls back to FFMA).
 * `status` is a device int the kernel writes a non-zero code to if a bounded wait runs out.
 * fuse_pool2 = 1 (3x3 layers, even W and H): the epilogue stores the maximum over each 2x2 pixel window,
 * i.e. `out` is the (W/2) x (H/2) result of the 2x2/2 max-pooling node that follows the convolution;
 * fuse_pool2 = 2: the same with the average (first-layer kernel only).  dRk_tensor_conv_can_fuse_pool tells
 * whether the kernel picked for a shape can do it (pool_type 1 max, 2 average).
 */
typedef struct dRk_TensorConvPlan dRk_TensorConvPlan;
/* 1 if the tensor path can evaluate this layer shape (stride 1, 1x1 or 3x3, channel counts it can tile). */
int dRk_tensor_conv_supported(int W, int H, int Cin, int Cout, int kw, int kh);
int dRk_tensor_conv_cin_pad(int Cin);
int dRk_tensor_conv_can_fuse_pool(int W, int H, int Cin, int Cout, int kw, int kh, int pool_type);
/* Packing of the reference's [Cin][Cout][kh][kw] filters (include/dR_nodes_conv2d.h:78-80) into the `wT` layout of the
 * tensor kernel that the planner picks for this layer shape: the rows above, except that layers with Cout <= 64 whose image
 * tiles well into 14 x 32 blocks use [128][12*CinPad] (two output rows stacked on M, see k_umma_pair.cu).
 * _packed_floats returns the size of `dst` (0: shape not supported); _pack_weights returns 0 on success. */
size_t dRk_tensor_conv_packed_floats(int W, int H, int Cin, int Cout, int kw, int kh);
int dRk_tensor_conv_pack_weights(const float *w, float *dst, int W, int H, int Cin, int Cout, int kw, int kh);
dRk_TensorConvPlan *dRk_tensor_conv_plan(const float *in, const float *wT, const float *bias, float *out,
                                         int n, int W, int H, int Cin, int Cout, int kw, int kh, int act,
                                         int ldo, int coff, int fuse_pool2, int *status);
/* Few-channel first layers only (Cin <= 4): the convolution then reads channel ch[c] of a source with pixel stride ldi,
 * times scale[c] plus shift[c], as its input channel c (ch a permutation of 0..Cin-1); `in` of the plan is that source.  Replaces a Slice -> scalar op ->
 * Concat preamble (examples/squeezenet-v1.1/squeezenet_whole/graph.dr:7-41) in front of the layer.  -1 if the plan is for
 * another kernel. */
int dRk_tensor_conv_set_input_map(dRk_TensorConvPlan *plan, int ldi, const int *ch, const float *scale, const float *shift);
/* FP32-accurate 3x3 stride-1 convolution on the tensor cores ("3xTF32"): every product x*w is evaluated as
 * hi(x)*hi(w) + hi(x)*lo(w) + lo(x)*hi(w) with hi() = the 19 bits a TF32 MMA reads, in three passes into one FP32 accumulator
 * (transposed kernel, or the row-pair kernel for at most 64 output channels; FLOAT32 tensor maps, the low part of the activations
 * computed in shared memory).  Error bound as the
 * exact-FP32 kernels (1e-4 * max|ref| per layer) at a third of the TF32 kernels' rate.  Same reference kernel as dRk_tensor_conv
 * (conv2dwinograd2, Kernels/dR_winograd2.cl:23-254).  wT2 = filters + their low parts, dRk_tensor_conv_x3_pack_weights;
 * the returned plan runs and is freed with dRk_tensor_conv_run / dRk_tensor_conv_free. */
int dRk_tensor_conv_x3_supported(int W, int H, int Cin, int Cout);
size_t dRk_tensor_conv_x3_packed_floats(int W, int H, int Cin, int Cout);
int dRk_tensor_conv_x3_pack_weights(const float *w, float *dst, int W, int H, int Cin, int Cout);
dRk_TensorConvPlan *dRk_tensor_conv_x3_plan(const float *in, const float *wT2, const float *bias, float *out, int n, int W, int H,
                                            int Cin, int Cout, int act, int ldo, int coff, int fuse_pool2, int *status);
/* Planner introspection, no device needed: the kernel (1 flat 1x1, 2 plain, 3 halo, 4 transposed, 5 row pair, 6 few-channel
 * first layer; 0 = shape or pooling not supported) and block geometry a plan for this layer on a GPU with `sms` SMs would use. */
int dRk_tensor_conv_describe(int n, int W, int H, int Cin, int Cout, int kw, int kh, int fuse_pool2, int sms,
                             int *P, int *TW, int *TH, int *ncols);
/* The same for a plan that was built: what its launches actually run. */
int dRk_tensor_conv_plan_describe(const dRk_TensorConvPlan *plan, int *P, int *TW, int *TH, int *ncols);
int dRk_tensor_conv_run(dRk_stream stream, dRk_TensorConvPlan *plan);
void dRk_tensor_conv_free(dRk_TensorConvPlan *plan);

/* Winograd F(2x2,3x3) with its sixteen transform-domain products on the tensor cores (TF32 operands, FP32 accumulate; the
 * transforms stay FP32): the algorithm of conv2dwinograd2 (Kernels/dR_winograd2.cl:23-254) with the product step (:177-189) as
 * one batched tcgen05 GEMM.  3x3 stride-1 layers with Cin % 4 == 0, Cin >= 8, Cout % 4 == 0, Cout >= 16.  U is the transformed
 * filter tensor [16][Cout][Cin] from dRk_tensor_winograd_pack_weights (G g G^T, src/dR_nodes_conv2d.c:1162-1240); scratch holds
 * dRk_tensor_winograd_scratch_floats() floats; in / out are N-HWC with pixel strides ldi / ldo, out at channel offset coff. */
typedef struct dRk_TensorWinogradPlan dRk_TensorWinogradPlan;
int dRk_tensor_winograd_supported(int W, int H, int Cin, int Cout);
size_t dRk_tensor_winograd_scratch_floats(int n, int W, int H, int Cin, int Cout);
size_t dRk_tensor_winograd_packed_floats(int Cin, int Cout);
int dRk_tensor_winograd_pack_weights(const float *w, float *dst, int Cin, int Cout);
dRk_TensorWinogradPlan *dRk_tensor_winograd_plan(const float *in, const float *U, const float *bias, float *out, float *scratch,
                                                 int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff, int *status);
/* The same algorithm as Winograd F(4x4,3x3) with FP32-accurate products: 36 transform positions, every product as three TF32 MMAs
 * (hi x hi, hi x lo, lo x hi) over operands stored as (high | low) halves; FP32-class error bound (1e-4 of max|ref|).  Cin a
 * multiple of 32; U2 from dRk_tensor_winograd4_x3_pack_weights ([36][Cout][2*Cin]); pool = 1 evaluates a following 2x2/2 max pooling
 * in the output transform (out is then the pooled tensor).  Run and free with dRk_tensor_winograd_run / _free. */
int dRk_tensor_winograd4_x3_supported(int W, int H, int Cin, int Cout);
size_t dRk_tensor_winograd4_x3_scratch_floats(int n, int W, int H, int Cin, int Cout);
size_t dRk_tensor_winograd4_x3_packed_floats(int Cin, int Cout);
int dRk_tensor_winograd4_x3_pack_weights(const float *w, float *dst, int Cin, int Cout);
dRk_TensorWinogradPlan *dRk_tensor_winograd4_x3_plan(const float *in, const float *U2, const float *bias, float *out, float *scratch,
                                                     int n, int W, int H, int Cin, int Cout, int act, int ldi, int ldo, int coff,
                                                     int pool, int *status);
int dRk_tensor_winograd_run(dRk_stream stream, dRk_TensorWinogradPlan *plan);
void dRk_tensor_winograd_free(dRk_TensorWinogradPlan *plan);

/* Fully connected layer on the tensor cores (TF32 inputs, FP32 accumulate) for batches of 16..128 with
 * Nin % 32 == 0 and Nout % 4 == 0 (>= 64): split-K flat GEMM + the reduce step of dRk_fc_f32.  wpacked comes from
 * dRk_tensor_fc_pack_weights (w is the reference's [Nin][Nout] matrix; dRk_tensor_fc_packed_floats() floats): every
 * 256-column x 32-row block the kernel fetches in one TMA request is one contiguous 32 KiB run, so the weight stream reads
 * DRAM sequentially.  scratch holds dRk_tensor_fc_scratch_floats() floats.  Same reference kernels as dRk_fc_f32. */
typedef struct dRk_TensorFcPlan dRk_TensorFcPlan;
int dRk_tensor_fc_supported(int n, int Nin, int Nout);
size_t dRk_tensor_fc_scratch_floats(int n, int Nin, int Nout);
size_t dRk_tensor_fc_packed_floats(int Nin, int Nout);
int dRk_tensor_fc_pack_weights(const float *w, float *wpacked, int Nin, int Nout);
dRk_TensorFcPlan *dRk_tensor_fc_plan(const float *in, const float *wpacked, const float *bias, float *out, float *scratch,
                                     int n, int Nin, int Nout, int act, int *status);
/* The same with FP32-accurate products (three TF32 passes over high and low halves; DR_MATH_FP32_TENSOR mode): weights from
 * dRk_tensor_fc_x3_pack_weights (twice the floats), scratch of dRk_tensor_fc_x3_scratch_floats() floats (its head holds the
 * activations split into halves by every run).  Run and free as below. */
size_t dRk_tensor_fc_x3_packed_floats(int Nin, int Nout);
size_t dRk_tensor_fc_x3_scratch_floats(int n, int Nin, int Nout);
int dRk_tensor_fc_x3_pack_weights(const float *w, float *wpacked2, int Nin, int Nout);
dRk_TensorFcPlan *dRk_tensor_fc_x3_plan(const float *in, const float *wpacked2, const float *bias, float *out, float *scratch,
                                        int n, int Nin, int Nout, int act, int *status);
int dRk_tensor_fc_run(dRk_stream stream, dRk_TensorFcPlan *plan);
void dRk_tensor_fc_free(dRk_TensorFcPlan *plan);

/* Test support for the bounded waits of the tensor-core kernels (no counterpart in the reference, whose failure path is
 * the return code of its OpenCL calls, src/dR_clwrap.c:874-883): one CTA waits at most `limit_cycles` SM clocks on a
 * barrier nothing arrives at, through the kernels' own wait function; it then writes code 9 to `status`, as a kernel
 * whose wait ran out does, and returns.  result (device int[3]): [0] outcome of that wait (0 = ran out), [1] outcome of
 * a wait on a barrier that was arrived at (1), [2] how long the first wait took, in units of 1024 clocks. */
int dRk_bounded_wait_probe(dRk_stream stream, int *status, long long limit_cycles, int *result);

/* Measurement support: the FP32 FMA rate of this GPU from registers (an 8 x 8 outer product per thread, the inner step of the
 * FFMA GEMM, no memory traffic; packed = 1: FFMA2, 0: scalar FFMA), best of three launches of `iters` iterations over every SM.
 * The yardstick the FFMA kernels' fractions are quoted against; sink is device scratch of at least 1024 floats per SM.
 * Synchronises the stream. */
int dRk_ffma_rate_probe(dRk_stream stream, float *sink, size_t sink_floats, int packed, int iters, double *tflops);

/* Debug switches of the library (environment variables DRK_NO_PAIR, DRK_NO_SWAP, DRK_NO_HALO, DRK_NO_INPUT_MAP,
 * DRK_NO_DEP_LAUNCH; read once per process): each takes one kernel variant or launch feature out of use so that two runs can
 * be timed against each other.  None changes results beyond rounding order.  No counterpart in the reference. */
typedef struct { int no_pair, no_swap, no_halo, no_input_map, no_dep_launch; } drk_DebugSwitches;
const drk_DebugSwitches *dRk_debug_switches(void);

/* Number of kernel launches issued through this ABI by the calling thread since the last reset. */
long dRk_launch_count(void);
void dRk_launch_count_reset(void);
#ifdef __cplusplus
}
#endif
#endif
