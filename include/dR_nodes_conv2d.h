/*
 * Conv2d node: out[z,y,x] = act(b[z] + sum_{k,j,i} in[k, y*sy+j, x*sx+i] * w[k,z,j+kh/2,i+kw/2])
 * with zero padding outside the input, output size (W/sx, H/sy, Cout)
 * (reference include/dR_nodes_conv2d.h:45-86, src/dR_nodes_conv2d.c:12-256).
 */
#ifndef DR_LAYERS_CONV2D_H
#define DR_LAYERS_CONV2D_H
#include "dR_types.h"

typedef struct dR_Conv2d_Data dR_Conv2d_Data;

/* Which CUDA kernel family evaluates a convolution node. */
enum dR_ConvAlgo {
    DR_CONV_AUTO = 0,       /* static rule (or the autotuner's pick when enabled) */
    DR_CONV_DIRECT = 1,     /* FP32 FFMA implicit-GEMM evaluation of the direct sum; any filter/stride */
    DR_CONV_WINOGRAD = 2,   /* F(2x2,3x3): transform, 16 transform-domain GEMMs, inverse transform */
    DR_CONV_ONEBYONE = 3,   /* 1x1 stride 1 as one GEMM over pixels */
    DR_CONV_TENSOR = 4,     /* tcgen05 TF32 implicit GEMM (TMA-fed, TMEM accumulators) */
    DR_CONV_TENSOR_WINOGRAD = 5, /* Winograd with the transform-domain GEMMs on the tcgen05 tensor cores: F(2x2,3x3) with TF32 products in TF32 mode,
                                    F(4x4,3x3) with three-pass (FP32-accurate) products in DR_MATH_FP32_TENSOR mode */
    DR_CONV_WINOGRAD4 = 6   /* F(4x4,3x3) in FP32: 36 transform-domain GEMMs, 4x fewer multiplications, error about 1e-5 of max|ref| */
};
#define DR_CONV_ALGOS 7
typedef enum dR_ConvAlgo dR_ConvAlgo;

struct dR_Conv2d_Data {
    dR_Shape4 shape;            /* [kw, kh, Cin, Cout] */
    dR_Shape4 stride;           /* [., sx, sy, .] */
    dR_Shape3 ishape;
    dR_ActivationType activation;
    gboolean useBias;
    gboolean hasVariables;
    gfloat *weights;            /* host copy, [Cin][Cout][kh][kw] */
    gfloat *biases;             /* host copy, [Cout] */
    cl_mem weightsBuf;          /* device weights packed for the chosen kernel */
    cl_mem biasBuf;
    /* ---- b200 ---- */
    gint algo;                  /* requested dR_ConvAlgo */
    gint chosenAlgo;            /* what dR_prepare settled on */
    gint chosenTensor;          /* 1: TF32 tensor-core arithmetic, 0: exact FP32 FFMA */
    cl_mem weightsBufAlt;       /* second packing kept for the autotuner's alternative */
    void *tmaDescs;             /* host block of CUtensorMap descriptors (tensor path) */
    gdouble tunedMs[DR_CONV_ALGOS]; /* measured ms per dR_ConvAlgo (0 = not measured) */
};

#ifdef __cplusplus
extern "C" {
#endif
/* reference include/dR_nodes_conv2d.h:70 */
dR_Node *dR_Conv2d(dR_Graph *net, dR_Node *inputnode, dR_Shape4 *filtershape, dR_Shape4 *stride,
                   dR_ActivationType activation, gboolean useBias);
/* reference include/dR_nodes_conv2d.h:86 -- copies weights [Cin][Cout][kh][kw] and bias [Cout] */
void dR_Conv2d_setVariables(dR_Node *node, gfloat *weights, gfloat *biases);
#ifdef __cplusplus
}
#endif

gboolean dR_conv2d_compute(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_schedule(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_propagateShape(dR_Graph *net, dR_Node *layer);
gint32 dR_conv2d_getRequiredOutputBufferSize(dR_Node *layer);
gboolean dR_conv2d_createKernel(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_allocateBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_fillBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_cleanupBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_conv2d_cleanupLayer(dR_Graph *net, dR_Node *layer);
gchar *dR_conv2d_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],
                               gint variableSizes[], gint *numVariables);
dR_Node *dR_conv2d_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params,
                                   gint numParams, gfloat **variables, gint numVariables);
gchar *dR_conv2d_printLayer(dR_Node *layer);
/* run one variant of this node on the stream (used by compute and by the autotuner) */
gboolean dR_conv2d_runVariant(dR_Graph *net, dR_Node *layer, gint algo, gint tensor);
#endif
