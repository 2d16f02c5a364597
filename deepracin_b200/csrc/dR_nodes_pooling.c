/*
 * Pooling node (reference src/dR_nodes_pooling.c).  The reference generates one fully
 * unrolled OpenCL kernel per node (:277-401); here one precompiled CUDA kernel takes the
 * window and stride as arguments.
 */
#include "dR_nodes_pooling.h"
#include "dR_core.h"
#include "dR_kernels.h"

/* reference src/dR_nodes_pooling.c:5-53 */
dR_Node *dR_Pooling(dR_Graph *net, dR_Node *inputLayer, dR_Shape4 *sh, dR_Shape4 *st, dR_PoolingType type)
{
    dR_Pooling_Data *p = (dR_Pooling_Data *)calloc(1, sizeof(dR_Pooling_Data));
    p->shape = *sh;
    p->stride = *st;
    p->poolingType = type;
    dR_Node *l = dR_newNode(tPooling, p);
    l->compute = dR_pooling_compute;
    l->schedule = dR_pooling_schedule;
    l->propagateShape = dR_pooling_propagateShape;
    l->getRequiredOutputBufferSize = dR_pooling_getRequiredOutputBufferSize;
    l->createKernel = dR_pooling_createKernel;
    l->allocateBuffers = dR_pooling_allocateBuffers;
    l->fillBuffers = dR_pooling_fillBuffers;
    l->cleanupBuffers = dR_pooling_cleanupBuffers;
    l->cleanupLayer = dR_pooling_cleanupLayer;
    l->serializeNode = dR_pooling_serializeNode;
    l->parseAppendNode = dR_pooling_parseAppendNode;
    l->printLayer = dR_pooling_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: Pooling Layer needs an appropriate Inputnode \n");
    dR_appendLayer(net, l);
    return l;
}

/* reference src/dR_nodes_pooling.c:55-79 */
gchar *dR_pooling_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_Pooling_Data *p = (dR_Pooling_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 9) { g_print("SerializeNode needs space for 9 parameters and 0 variables!\n"); return NULL; }
    *numParams = 9;
    params[0] = g_strdup_printf("%d", p->poolingType);
    params[1] = g_strdup_printf("%d", p->shape.s0);
    params[2] = g_strdup_printf("%d", p->shape.s1);
    params[3] = g_strdup_printf("%d", p->shape.s2);
    params[4] = g_strdup_printf("%d", p->shape.s3);
    params[5] = g_strdup_printf("%d", p->stride.s0);
    params[6] = g_strdup_printf("%d", p->stride.s1);
    params[7] = g_strdup_printf("%d", p->stride.s2);
    params[8] = g_strdup_printf("%d", p->stride.s3);
    *numVariables = 0;
    return "Pooling";
}

/* reference src/dR_nodes_pooling.c:81-113 */
dR_Node *dR_pooling_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape4 shape, stride;
    (void)variables;
    if (numINodes != 1) { g_print("Parsing Error: Pooling Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 9 || numVariables != 0) { g_print("Parsing Error: Pooling Node needs 9 Parameters and 0 Variables!\n"); return NULL; }
    shape.s0 = atoi(params[1]); shape.s1 = atoi(params[2]); shape.s2 = atoi(params[3]); shape.s3 = atoi(params[4]);
    stride.s0 = atoi(params[5]); stride.s1 = atoi(params[6]); stride.s2 = atoi(params[7]); stride.s3 = atoi(params[8]);
    return dR_Pooling(net, iNodes[0], &shape, &stride, (dR_PoolingType)atoi(params[0]));
}

gboolean dR_pooling_schedule(dR_Graph *net, dR_Node *layer) { (void)net; ((dR_Pooling_Data *)layer->layer)->useLMEM = FALSE; return TRUE; }

static gint ceilDiv(gint a, gint b) { return (a + b - 1) / b; }

/* reference src/dR_nodes_pooling.c:186-224: ceil(in/stride) per axis, channels included */
gboolean dR_pooling_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_Pooling_Data *p = (dR_Pooling_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("Pooling Layer with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    if (p->stride.s1 <= 0 || p->stride.s2 <= 0 || p->stride.s3 <= 0 || p->shape.s1 <= 0 || p->shape.s2 <= 0 || p->shape.s3 <= 0) {
        g_print("Pooling: window and stride must be positive\n");
        return FALSE;
    }
    if (p->poolingType != tMax && p->poolingType != tAverage) { g_print("Pooling: only max and average pooling are implemented\n"); return FALSE; }
    p->ishape = dR_firstInput(layer)->oshape;
    layer->oshape.s0 = ceilDiv(p->ishape.s0, p->stride.s1);
    layer->oshape.s1 = ceilDiv(p->ishape.s1, p->stride.s2);
    layer->oshape.s2 = ceilDiv(p->ishape.s2, p->stride.s3);
    if (layer->oshape.s0 <= 0 || layer->oshape.s1 <= 0 || layer->oshape.s2 <= 0) {
        if (!net->config->silent) g_print("Pooling Shape propagates to Zero. False shape parameters! \n");
        return FALSE;
    }
    return TRUE;
}

gint32 dR_pooling_getRequiredOutputBufferSize(dR_Node *layer) { return layer->oshape.s0 * layer->oshape.s1 * layer->oshape.s2; }
gboolean dR_pooling_createKernel(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
gboolean dR_pooling_allocateBuffers(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
gboolean dR_pooling_fillBuffers(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
gboolean dR_pooling_cleanupBuffers(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
gboolean dR_pooling_cleanupLayer(dR_Graph *net, dR_Node *layer) { (void)net; g_free(layer->layer); return TRUE; }

/* reference src/dR_nodes_pooling.c:138-183 */
gboolean dR_pooling_compute(dR_Graph *net, dR_Node *layer)
{
    dR_Pooling_Data *p = (dR_Pooling_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    if (p->useLMEM) return TRUE;        /* the producing convolution already stored the pooled tensor here */
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_pool(net->clConfig->clCommandQueue, dR_actPtr(in) + in->act_coffset, dR_actPtr(layer), net->config->batchSize,
                                      p->ishape.s0, p->ishape.s1, p->ishape.s2, p->shape.s1, p->shape.s2, p->shape.s3,
                                      p->stride.s1, p->stride.s2, p->stride.s3, p->poolingType == tMax ? 0 : 1, in->act_cstride);
    return dR_finishCLKernel(net, "deepRACIN:pool");
}

gchar *dR_pooling_printLayer(dR_Node *layer)
{
    dR_Pooling_Data *p = (dR_Pooling_Data *)layer->layer;
    return g_strdup_printf("Pooling Layer: %d\n Type: %s\n Window: %dx%dx%d\n Stride: %d, %d, %d\n", layer->layerID,
                           p->poolingType == tMax ? "Max" : "Average", p->shape.s1, p->shape.s2, p->shape.s3, p->stride.s1, p->stride.s2, p->stride.s3);
}
