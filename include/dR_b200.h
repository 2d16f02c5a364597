/*
 * Additions of the CUDA build to the deepRacin API.  None of these has a counterpart in
 * the reference: its tensors have no batch dimension (a batch is a host loop of
 * dR_feedData + dR_apply, examples/vgg16/vgg_deployed.c:141-166), its kernel variant is
 * fixed by filter shape (src/dR_nodes_conv2d.c:36-81) and it runs on one device.
 */
#ifndef DR_B200_H
#define DR_B200_H
#include "dR_types.h"
#ifdef __cplusplus
extern "C" {
#endif
enum dR_MathMode {
    DR_MATH_FP32 = 0,   /* every contraction in FP32 FFMA (validation-grade, the default) */
    DR_MATH_TF32 = 1,   /* dense contractions on the tcgen05 tensor cores with TF32 inputs, FP32 accumulate */
    DR_MATH_FP32_TENSOR = 2 /* FP32-accurate results from the tensor cores: 3x3 layers evaluate every product in three TF32 passes
                               (high x high, high x low, low x high parts; error bound of the FP32 class), the rest runs DR_MATH_FP32 */
};
enum dR_InterfaceLayout {
    DR_LAYOUT_CHW = 0,  /* reference layout of feed/output buffers: [C][H][W] per image */
    DR_LAYOUT_HWC = 1   /* [H][W][C] per image: no layout conversion on feed/fetch */
};
/* Images per dR_apply; feed and output buffers hold n tensors back to back.  Before dR_prepare. */
gboolean dR_setBatchSize(dR_Graph *net, gint n);
gboolean dR_setMathMode(dR_Graph *net, gint mode);
gboolean dR_setInterfaceLayout(dR_Graph *net, gint layout);
/* Force a kernel family for one convolution node (dR_ConvAlgo); DR_CONV_AUTO restores the rule. */
gboolean dR_setConvAlgo(dR_Node *node, gint algo);
/* Graph-wide override, and switch for timing the legal variants of every conv during dR_prepare. */
gboolean dR_setGraphConvAlgo(dR_Graph *net, gint algo);
gboolean dR_setAutotune(dR_Graph *net, gboolean on);
gboolean dR_setFusion(dR_Graph *net, gboolean on);
gboolean dR_setCudaGraph(dR_Graph *net, gboolean on);
/* CUDA device ordinal used by dR_initCL. */
gboolean dR_setDevice(dR_Graph *net, gint ordinal);
/* Blocks until everything issued on the graph's stream has finished. */
gboolean dR_synchronize(dR_Graph *net);
/* dR_apply bracketed by events on the graph's own stream; returns milliseconds (<0 on failure). */
gdouble dR_applyTimed(dR_Graph *net, gint iterations);
/* Kernel family / arithmetic a prepared convolution node runs (dR_ConvAlgo; 0 FP32 FFMA, 1 TF32 tensor cores, 2 three-pass TF32). */
gint dR_getConvAlgo(dR_Node *node);
gint dR_getConvTensor(dR_Node *node);
/* The tensor-core kernel a convolution node's launches run once it has been applied (numbering and geometry of
 * dRk_tensor_conv_describe: geom = {pitch, valid pixels per block row, block rows, MMA columns}); 0 if it runs an FP32 kernel. */
gint dR_getConvTensorKernel(dR_Node *node, gint geom[4]);
/* Last per-node GPU time in ms (profilingGPU runs), and number of kernels one dR_apply launches. */
gdouble dR_getNodeGpuMs(dR_Node *node);
gint dR_getLaunchCount(dR_Graph *net);
/* Non-zero if a kernel reported a device-side status (bounded wait ran out, ...) since the last call. */
gint dR_getDeviceStatus(dR_Graph *net);
/* Exercises the failure path of the tensor-core kernels without a failure: a one-CTA kernel waits at most
 * `limitMicroseconds` (at the GPU's maximum clock) on a barrier nothing arrives at, gives up the way a stuck kernel
 * would (code 9 in the graph's status word, read by dR_getDeviceStatus) and returns.  result as dRk_bounded_wait_probe.
 * The graph must be prepared; blocks until the probe has finished. */
gboolean dR_probeBoundedWait(dR_Graph *net, gint limitMicroseconds, gint result[3]);
/* Measurement support: the FP32 FMA rate of the graph's GPU from registers (dRk_ffma_rate_probe; packed: FFMA2, else scalar
 * FFMA), in TFLOP/s -- the yardstick for the FFMA kernels.  The graph must be prepared; blocks for a few milliseconds. */
gboolean dR_probeFfmaRate(dR_Graph *net, gboolean packed, gdouble *tflops);
/* Double-buffered feeding: dR_feedDataAsync copies on a second stream into the feed node's other interface
 * buffer while the previous batch is still being computed; the next dR_apply waits for that copy and reads it.
 * Before dR_prepare; not combined with CUDA-graph replay or caller-supplied feed buffers. */
gboolean dR_setFeedOverlap(dR_Graph *net, gboolean on);
/* Feed / fetch with pinned host memory and no implicit synchronisation. */
gboolean dR_feedDataAsync(dR_Graph *net, dR_Node *feednode, gfloat *pinned, size_t numfloats);
gboolean dR_fetchOutputAsync(dR_Graph *net, gint outputIndex, gfloat *pinned, size_t numfloats);
/* The same feed from 8-bit samples (decoded image bytes in the graph's interface layout, batchSize images back to back): a
 * quarter of the bytes cross the host link, the cast to float happens on the device ((float)byte, what the reference's examples
 * compute on the host, examples/vgg16/vgg_deployed.c:153-157).  The first call allocates the device staging buffer. */
gboolean dR_feedDataU8Async(dR_Graph *net, dR_Node *feednode, const unsigned char *pinned, size_t numbytes);
void *dR_allocPinned(size_t bytes);
void dR_freePinned(void *p);
/* Planning without a device: dR_prepare runs scheduling, fusion planning, variant selection and the buffer
 * planner with placeholder addresses and uploads nothing; dR_apply then refuses to run.  For host-side
 * inspection and tests of the planner; never a compute path. */
gboolean dR_setDryRun(dR_Graph *net, gboolean on);
/* Introspection of a prepared graph: execution order, and where each node's activations live. */
gint dR_getScheduleLength(dR_Graph *net);
gint dR_getScheduledNodeId(dR_Graph *net, gint position);
size_t dR_getNodeActAddress(dR_Node *node);
gint dR_getNodeActFloats(dR_Node *node);
gint dR_getNodeChannelStride(dR_Node *node);
gint dR_getNodeChannelOffset(dR_Node *node);
gint dR_getStreamBufferCount(dR_Graph *net);
size_t dR_getScratchFloats(dR_Graph *net);
/* Library identification: returns a static string naming the build (arch, kernels). */
const char *dR_b200_version(void);
#ifdef __cplusplus
}
#endif
#endif
