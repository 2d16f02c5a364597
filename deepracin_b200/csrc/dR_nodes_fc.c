/*
 * FullyConnected node (reference src/dR_nodes_fc.c).  The reference's two-step
 * partitioned matrix-vector product becomes one CUDA entry point that streams the
 * [Nin][Nout] weight matrix once per batch (split-K partials in the graph's scratch,
 * reduced with bias + activation by a second launch), or a GEMM for large batches.
 */
#include "dR_nodes_fc.h"
#include "dR_core.h"
#include "dR_kernels.h"
#include "dR_b200.h"

/* reference src/dR_nodes_fc.c:6-48 */
dR_Node *dR_FullyConnected(dR_Graph *net, dR_Node *inputLayer, dR_Shape2 *sh, dR_ActivationType acttype, gboolean useB)
{
    dR_FC_Data *fc = (dR_FC_Data *)calloc(1, sizeof(dR_FC_Data));
    fc->shape = *sh;
    fc->activation = acttype;
    fc->useBias = useB;
    dR_Node *l = dR_newNode(tFullyConnected, fc);
    l->compute = dR_fc_compute;
    l->schedule = dR_fc_schedule;
    l->propagateShape = dR_fc_propagateShape;
    l->getRequiredOutputBufferSize = dR_fc_getRequiredOutputBufferSize;
    l->createKernel = dR_fc_createKernel;
    l->allocateBuffers = dR_fc_allocateBuffers;
    l->fillBuffers = dR_fc_fillBuffers;
    l->cleanupBuffers = dR_fc_cleanupBuffers;
    l->cleanupLayer = dR_fc_cleanupLayer;
    l->serializeNode = dR_fc_serializeNode;
    l->parseAppendNode = dR_fc_parseAppendNode;
    l->setVariables = dR_FullyConnected_setVariables;
    l->printLayer = dR_fc_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: Fully Connected needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

/* reference src/dR_nodes_fc.c:50-84 */
gchar *dR_fc_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    gint nv = fc->useBias ? 2 : 1;
    if (*numParams < 4 || *numVariables < nv) { g_print("SerializeNode needs space for 4 parameters and %d variables!\n", nv); return NULL; }
    if (!fc->hasVariables) { g_print("FullyConnected node %d has no weights to serialize\n", layer->layerID); return NULL; }
    *numParams = 4;
    params[0] = g_strdup_printf("%d", fc->activation);
    params[1] = g_strdup_printf("%d", fc->useBias ? 1 : 0);
    params[2] = g_strdup_printf("%d", fc->shape.s0);
    params[3] = g_strdup_printf("%d", fc->shape.s1);
    *numVariables = nv;
    variableSizes[0] = fc->shape.s0 * fc->shape.s1;
    variables[0] = fc->weights;
    if (fc->useBias) { variableSizes[1] = fc->shape.s1; variables[1] = fc->biases; }
    return "FullyConnected";
}

/* reference src/dR_nodes_fc.c:86-112 */
dR_Node *dR_fc_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape2 shape;
    if (numINodes != 1) { g_print("Parsing Error: FullyConnected Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 4 || numVariables < 1 || numVariables > 2) { g_print("Parsing Error: FullyConnected Node needs 4 Parameters and 1 or 2 Variables!\n"); return NULL; }
    gint useB = atoi(params[1]);
    if (useB && numVariables < 2) { g_print("Parsing Error: FullyConnected Node with bias needs 2 Variables!\n"); return NULL; }
    shape.s0 = atoi(params[2]); shape.s1 = atoi(params[3]);
    dR_Node *out = dR_FullyConnected(net, iNodes[0], &shape, (dR_ActivationType)atoi(params[0]), useB);
    dR_FullyConnected_setVariables(out, variables[0], useB ? variables[1] : NULL);
    return out;
}

gboolean dR_fc_schedule(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }

/* reference src/dR_nodes_fc.c:280-306 */
gboolean dR_fc_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("FullyConnected Layer with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    fc->ishape = dR_firstInput(layer)->oshape;
    if (fc->ishape.s0 * fc->ishape.s1 * fc->ishape.s2 != fc->shape.s0) {
        if (!net->config->silent) g_print("FullyConnected Layer does not match Input Size! \n");
        return FALSE;
    }
    layer->oshape.s0 = fc->shape.s1; layer->oshape.s1 = 1; layer->oshape.s2 = 1;
    return TRUE;
}

gint32 dR_fc_getRequiredOutputBufferSize(dR_Node *layer) { return layer->oshape.s0; }

gboolean dR_fc_createKernel(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    /* tensor modes, batches of 16..128: split-K GEMM on the tensor cores (2: with three-pass, FP32-accurate products); otherwise
       the FP32 weight-streaming kernels */
    fc->chosenTensor = 0;
    if (net->config->mathMode != DR_MATH_FP32 && dRk_tensor_fc_supported(net->config->batchSize, fc->shape.s0, fc->shape.s1))
        fc->chosenTensor = net->config->mathMode == DR_MATH_FP32_TENSOR ? 2 : 1;
    layer->scratchFloats = fc->chosenTensor == 2 ? dRk_tensor_fc_x3_scratch_floats(net->config->batchSize, fc->shape.s0, fc->shape.s1)
                         : fc->chosenTensor ? dRk_tensor_fc_scratch_floats(net->config->batchSize, fc->shape.s0, fc->shape.s1)
                                            : dRk_fc_scratch_floats(net->config->batchSize, fc->shape.s0, fc->shape.s1);
    return TRUE;
}

gboolean dR_fc_allocateBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    gboolean ret;
    if (!fc->hasVariables) { g_print("FullyConnected Layer %d has no weights (call dR_FullyConnected_setVariables)\n", layer->layerID); return FALSE; }
    if (fc->chosenTensor) ret = dR_createFloatBufferL(net, &fc->weightsBufT, (fc->chosenTensor == 2 ? 2 : 1) * dRk_tensor_fc_packed_floats(fc->shape.s0, fc->shape.s1));
    else ret = dR_createFloatBufferL(net, &fc->weightsBuf, (size_t)fc->shape.s0 * fc->shape.s1);
    if (fc->useBias) ret &= dR_createFloatBuffer(net, &fc->biasBuf, fc->shape.s1, CL_MEM_READ_ONLY);
    return ret;
}

gboolean dR_fc_fillBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    gboolean ret;
    if (fc->chosenTensor) {
        /* block-by-block packing for the TMA-fed B operand */
        const size_t np = (fc->chosenTensor == 2 ? 2 : 1) * dRk_tensor_fc_packed_floats(fc->shape.s0, fc->shape.s1);
        gfloat *t = (gfloat *)g_malloc(np * sizeof(gfloat));
        ret = (fc->chosenTensor == 2 ? dRk_tensor_fc_x3_pack_weights(fc->weights, t, fc->shape.s0, fc->shape.s1)
                                     : dRk_tensor_fc_pack_weights(fc->weights, t, fc->shape.s0, fc->shape.s1)) == 0 &&
              dR_uploadArray(net, "", t, 0, np * sizeof(cl_float), fc->weightsBufT);
        g_free(t);
    } else {
        ret = dR_uploadArray(net, "", fc->weights, 0, (size_t)fc->shape.s0 * fc->shape.s1 * sizeof(cl_float), fc->weightsBuf);
    }
    if (fc->useBias) ret &= dR_uploadArray(net, "", fc->biases, 0, (size_t)fc->shape.s1 * sizeof(cl_float), fc->biasBuf);
    return ret;
}

/* reference src/dR_nodes_fc.c:201-278 */
gboolean dR_fc_compute(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    if (in->act_cstride != in->oshape.s2) { g_print("FullyConnected Layer %d: input must be dense\n", layer->layerID); return FALSE; }
    dR_beginCLKernel(net);
    if (fc->chosenTensor) {
        if (!fc->tmaDescs) {
            fc->tmaDescs = (fc->chosenTensor == 2 ? dRk_tensor_fc_x3_plan : dRk_tensor_fc_plan)(
                dR_actPtr(in), (const float *)fc->weightsBufT, fc->useBias ? (const float *)fc->biasBuf : NULL, dR_actPtr(layer),
                (float *)net->scratch, net->config->batchSize, fc->shape.s0, fc->shape.s1, fc->activation == tReLU ? 1 : 0, (int *)net->statusWord);
            if (!fc->tmaDescs) { g_print("FullyConnected Layer %d: tensor-core plan could not be built\n", layer->layerID); return FALSE; }
        }
        net->clConfig->clError = dRk_tensor_fc_run(net->clConfig->clCommandQueue, (dRk_TensorFcPlan *)fc->tmaDescs);
        return dR_finishCLKernel(net, "deepRACIN:FullyConnected");
    }
    net->clConfig->clError = dRk_fc_f32(net->clConfig->clCommandQueue, dR_actPtr(in), (const float *)fc->weightsBuf,
                                        fc->useBias ? (const float *)fc->biasBuf : NULL, dR_actPtr(layer), (float *)net->scratch,
                                        net->config->batchSize, fc->shape.s0, fc->shape.s1, fc->activation == tReLU ? 1 : 0);
    return dR_finishCLKernel(net, "deepRACIN:FullyConnected");
}

gboolean dR_fc_cleanupBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    gboolean ret = TRUE;
    if (fc->weightsBuf) { ret &= dR_clMemoryBufferCleanup(net, fc->weightsBuf); fc->weightsBuf = NULL; }
    if (fc->weightsBufT) { ret &= dR_clMemoryBufferCleanup(net, fc->weightsBufT); fc->weightsBufT = NULL; }
    if (fc->tmaDescs) { dRk_tensor_fc_free((dRk_TensorFcPlan *)fc->tmaDescs); fc->tmaDescs = NULL; }
    if (fc->biasBuf) { ret &= dR_clMemoryBufferCleanup(net, fc->biasBuf); fc->biasBuf = NULL; }
    return ret;
}

gboolean dR_fc_cleanupLayer(dR_Graph *net, dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    (void)net;
    g_free(fc->weights); g_free(fc->biases); g_free(fc);
    return TRUE;
}

/* reference src/dR_nodes_fc.c:371-389 */
void dR_FullyConnected_setVariables(dR_Node *layer, gfloat *weights, gfloat *biases)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    size_t n = (size_t)fc->shape.s0 * fc->shape.s1;
    g_free(fc->weights);
    fc->weights = (gfloat *)g_malloc(n * sizeof(gfloat));
    memcpy(fc->weights, weights, n * sizeof(gfloat));
    if (fc->useBias && biases) {
        g_free(fc->biases);
        fc->biases = (gfloat *)g_malloc((size_t)fc->shape.s1 * sizeof(gfloat));
        memcpy(fc->biases, biases, (size_t)fc->shape.s1 * sizeof(gfloat));
    }
    fc->hasVariables = TRUE;
}

gchar *dR_fc_printLayer(dR_Node *layer)
{
    dR_FC_Data *fc = (dR_FC_Data *)layer->layer;
    static const char *acts[] = {"Linear", "ReLU", "Sigmoid", "Tan"};
    return g_strdup_printf("FullyConnected Layer: %d\n Input neurons: %d\n Output neurons: %d\n Activation: %s\n Use bias: %s\n",
                           layer->layerID, fc->shape.s0, fc->shape.s1, acts[fc->activation & 3], fc->useBias ? "Yes" : "No");
}
