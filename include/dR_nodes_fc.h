/*
 * FullyConnected node: out[o] = act(b[o] + sum_k in_hwc[k] * w[k][o]); the input is
 * flattened in (y, x, z) order, weights are [Nin][Nout] row-major
 * (reference include/dR_nodes_fc.h:28-34, src/dR_nodes_fc.c, Kernels/dR_fcl.cl:59-120).
 */
#ifndef DR_LAYERS_FC_H
#define DR_LAYERS_FC_H
#include "dR_types.h"

typedef struct dR_FC_Data dR_FC_Data;
struct dR_FC_Data {
    dR_Shape2 shape;            /* [Nin, Nout] */
    dR_Shape3 ishape;
    dR_ActivationType activation;
    gboolean useBias;
    gboolean hasVariables;
    gfloat *weights;
    gfloat *biases;
    cl_mem weightsBuf;          /* [Nin][Nout] (also the K-major x Nout packing the GEMM kernels want) */
    cl_mem weightsBufT;         /* [Nout][Nin] packing for the tensor-core path */
    cl_mem biasBuf;
    gint splitK;                /* K partitions of the weight-streaming kernel (partials live in scratch) */
    gint chosenTensor;
    void *tmaDescs;
};

#ifdef __cplusplus
extern "C" {
#endif
dR_Node *dR_FullyConnected(dR_Graph *net, dR_Node *inputLayer, dR_Shape2 *shape, dR_ActivationType activation,
                           gboolean useBias);
void dR_FullyConnected_setVariables(dR_Node *layer, gfloat *weights, gfloat *bias);
#ifdef __cplusplus
}
#endif

gboolean dR_fc_compute(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_schedule(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_propagateShape(dR_Graph *net, dR_Node *layer);
gint32 dR_fc_getRequiredOutputBufferSize(dR_Node *layer);
gboolean dR_fc_createKernel(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_allocateBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_fillBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_cleanupBuffers(dR_Graph *net, dR_Node *layer);
gboolean dR_fc_cleanupLayer(dR_Graph *net, dR_Node *layer);
gchar *dR_fc_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],
                           gint variableSizes[], gint *numVariables);
dR_Node *dR_fc_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams,
                               gfloat **variables, gint numVariables);
gchar *dR_fc_printLayer(dR_Node *layer);
#endif
