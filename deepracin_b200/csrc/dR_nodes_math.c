/*
 * Element-wise and softmax nodes (reference src/dR_nodes_math.c, kernels
 * Kernels/dR_math.cl).  Softmax is one fused kernel per image here; the reference runs
 * computeExp, downloads, sums on the host and runs mulScalar (:620-678).
 */
#include "dR_nodes_math.h"
#include "dR_core.h"
#include "dR_kernels.h"

static gboolean noop(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
static gboolean freeData(dR_Graph *net, dR_Node *layer) { (void)net; g_free(layer->layer); return TRUE; }
static gint32 denseSize(dR_Node *layer) { return layer->oshape.s0 * layer->oshape.s1 * layer->oshape.s2; }
static size_t batchLen(dR_Graph *net, dR_Node *layer) { return (size_t)denseSize(layer) * net->config->batchSize; }

static gboolean denseInput(dR_Node *layer, dR_Node *in)
{
    if (in->act_cstride == in->oshape.s2) return TRUE;
    g_print("Layer %d: input %d is stored strided; element-wise nodes need dense inputs\n", layer->layerID, in->layerID);
    return FALSE;
}

/* ------------------------------------------------ element-wise, two inputs */
/* reference src/dR_nodes_math.c:9-50 */
dR_Node *dR_ElemWise2Operation(dR_Graph *net, dR_Node *in1, dR_Node *in2, dR_ElemWise2OperationType op)
{
    dR_ElemWise2Op_Data *d = (dR_ElemWise2Op_Data *)calloc(1, sizeof(dR_ElemWise2Op_Data));
    d->op = op;
    dR_Node *l = dR_newNode(tElemWise2Op, d);
    l->compute = dR_elemwise2op_compute;
    l->schedule = dR_elemwise2op_schedule;
    l->propagateShape = dR_elemwise2op_propagateShape;
    l->getRequiredOutputBufferSize = dR_elemwise2op_getRequiredOutputBufferSize;
    l->createKernel = dR_elemwise2op_createKernel;
    l->allocateBuffers = dR_elemwise2op_allocateBuffers;
    l->fillBuffers = dR_elemwise2op_fillBuffers;
    l->cleanupBuffers = dR_elemwise2op_cleanupBuffers;
    l->cleanupLayer = dR_elemwise2op_cleanupLayer;
    l->serializeNode = dR_elemwise2op_serializeNode;
    l->parseAppendNode = dR_elemwise2op_parseAppendNode;
    l->printLayer = dR_elemwise2op_printLayer;
    if (in1 && in2) { dR_linkNodes(in1, l); dR_linkNodes(in2, l); }
    else g_print("Error: ElemWise2Operation node needs 2 appropriate Inputnodes\n");
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_elemwise2op_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    (void)variables; (void)variableSizes;
    if (*numParams < 1) { g_print("SerializeNode needs space for 1 parameters and 0 variables!\n"); return NULL; }
    *numParams = 1;
    params[0] = g_strdup_printf("%d", ((dR_ElemWise2Op_Data *)layer->layer)->op);
    *numVariables = 0;
    return "ElemWise2Op";
}

/* The reference's reader rejects this node unless it has ONE input (src/dR_nodes_math.c:76),
 * so a saved two-input graph cannot be re-loaded there; two inputs are accepted here. */
dR_Node *dR_elemwise2op_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    (void)variables;
    if (numINodes != 2) { g_print("Parsing Error: ElemWise2Op Node needs 2 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 1 || numVariables != 0) { g_print("Parsing Error: ElemWise2Op Node needs 1 Parameters and 0 Variables!\n"); return NULL; }
    return dR_ElemWise2Operation(net, iNodes[0], iNodes[1], (dR_ElemWise2OperationType)atoi(params[0]));
}

gboolean dR_elemwise2op_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

/* reference src/dR_nodes_math.c:125-156: both inputs must have the same shape */
gboolean dR_elemwise2op_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_ElemWise2Op_Data *d = (dR_ElemWise2Op_Data *)layer->layer;
    if (layer->previous_layers->length != 2) {
        if (!net->config->silent) g_print("Elem-wise 2-operation Node with id %d has %d inputs but needs 2!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    dR_Node *a = dR_nthInput(layer, 0), *b = dR_nthInput(layer, 1);
    if (a->oshape.s0 != b->oshape.s0 || a->oshape.s1 != b->oshape.s1 || a->oshape.s2 != b->oshape.s2) {
        if (!net->config->silent) g_print("Elem-wise 2-operation Node needs 2 input nodes with the same shape!\n");
        return FALSE;
    }
    if (d->op < tAdd || d->op > tPow) { g_print("Elem-wise 2-operation: unknown op %d\n", d->op); return FALSE; }
    d->ishape = a->oshape;
    layer->oshape = a->oshape;
    return TRUE;
}

gint32 dR_elemwise2op_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_elemwise2op_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise2op_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise2op_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise2op_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise2op_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

/* reference src/dR_nodes_math.c:99-123 */
gboolean dR_elemwise2op_compute(dR_Graph *net, dR_Node *layer)
{
    dR_ElemWise2Op_Data *d = (dR_ElemWise2Op_Data *)layer->layer;
    dR_Node *a = dR_nthInput(layer, 0), *b = dR_nthInput(layer, 1);
    if (!denseInput(layer, a) || !denseInput(layer, b)) return FALSE;
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_elemwise2(net->clConfig->clCommandQueue, dR_actPtr(a), dR_actPtr(b), dR_actPtr(layer), batchLen(net, layer), d->op);
    return dR_finishCLKernel(net, "deepRACIN:elemWise2Op");
}

gchar *dR_elemwise2op_printLayer(dR_Node *layer)
{
    static const char *ops[] = {"Add", "Sub", "Mul", "Div", "Pow"};
    dR_ElemWise2Op_Data *d = (dR_ElemWise2Op_Data *)layer->layer;
    return g_strdup_printf("Element-wise 2-operation node: %d\n Operation: %s\n", layer->layerID, ops[d->op % 5]);
}

/* ------------------------------------------------- element-wise, one input */
/* reference src/dR_nodes_math.c:259-299 */
dR_Node *dR_ElemWise1Operation(dR_Graph *net, dR_Node *inputLayer, dR_ElemWise1OperationType op, gfloat scalar)
{
    dR_ElemWise1Op_Data *d = (dR_ElemWise1Op_Data *)calloc(1, sizeof(dR_ElemWise1Op_Data));
    d->op = op;
    d->scalar = scalar;
    dR_Node *l = dR_newNode(tElemWise1Op, d);
    l->compute = dR_elemwise1op_compute;
    l->schedule = dR_elemwise1op_schedule;
    l->propagateShape = dR_elemwise1op_propagateShape;
    l->getRequiredOutputBufferSize = dR_elemwise1op_getRequiredOutputBufferSize;
    l->createKernel = dR_elemwise1op_createKernel;
    l->allocateBuffers = dR_elemwise1op_allocateBuffers;
    l->fillBuffers = dR_elemwise1op_fillBuffers;
    l->cleanupBuffers = dR_elemwise1op_cleanupBuffers;
    l->cleanupLayer = dR_elemwise1op_cleanupLayer;
    l->serializeNode = dR_elemwise1op_serializeNode;
    l->parseAppendNode = dR_elemwise1op_parseAppendNode;
    l->printLayer = dR_elemwise1op_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: ElemWise1Operation node needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

/* reference src/dR_nodes_math.c:301-318 ("%d" op, "%f" scalar) */
gchar *dR_elemwise1op_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_ElemWise1Op_Data *d = (dR_ElemWise1Op_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 2) { g_print("SerializeNode needs space for 2 parameters and 0 variables!\n"); return NULL; }
    *numParams = 2;
    params[0] = g_strdup_printf("%d", d->op);
    params[1] = g_strdup_printf("%f", d->scalar);
    *numVariables = 0;
    return "ElemWise1Op";
}

dR_Node *dR_elemwise1op_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    (void)variables;
    if (numINodes != 1) { g_print("Parsing Error: ElemWise1Op Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 2 || numVariables != 0) { g_print("Parsing Error: ElemWise1Op Node needs 2 Parameters and 0 Variables!\n"); return NULL; }
    return dR_ElemWise1Operation(net, iNodes[0], (dR_ElemWise1OperationType)atoi(params[0]), (gfloat)atof(params[1]));
}

gboolean dR_elemwise1op_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

gboolean dR_elemwise1op_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_ElemWise1Op_Data *d = (dR_ElemWise1Op_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("Elem-wise 1-operation Node with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    if (d->op < tAddS || d->op > tPowS) { g_print("Elem-wise 1-operation: unknown op %d\n", d->op); return FALSE; }
    d->ishape = dR_firstInput(layer)->oshape;
    layer->oshape = d->ishape;
    return TRUE;
}

gint32 dR_elemwise1op_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_elemwise1op_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise1op_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise1op_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise1op_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_elemwise1op_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

/* reference src/dR_nodes_math.c:349-376 */
gboolean dR_elemwise1op_compute(dR_Graph *net, dR_Node *layer)
{
    dR_ElemWise1Op_Data *d = (dR_ElemWise1Op_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    if (!denseInput(layer, in)) return FALSE;
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_elemwise1(net->clConfig->clCommandQueue, dR_actPtr(in), dR_actPtr(layer), batchLen(net, layer), d->op, d->scalar);
    return dR_finishCLKernel(net, "deepRACIN:elemWise1Op");
}

gchar *dR_elemwise1op_printLayer(dR_Node *layer)
{
    static const char *ops[] = {"AddS", "SubS", "MulS", "DivS", "Log", "Exp", "Sqrt", "Fill", "PowS"};
    dR_ElemWise1Op_Data *d = (dR_ElemWise1Op_Data *)layer->layer;
    return g_strdup_printf("Element-wise 1-operation node: %d\n Operation: %s\n Scalar: %f\n", layer->layerID, ops[d->op % 9], d->scalar);
}

/* ----------------------------------------------------------------- softmax */
/* reference src/dR_nodes_math.c:534-573 */
dR_Node *dR_Softmax(dR_Graph *net, dR_Node *inputLayer)
{
    dR_Softmax_Data *d = (dR_Softmax_Data *)calloc(1, sizeof(dR_Softmax_Data));
    dR_Node *l = dR_newNode(tSoftmax, d);
    l->compute = dR_softmax_compute;
    l->schedule = dR_softmax_schedule;
    l->propagateShape = dR_softmax_propagateShape;
    l->getRequiredOutputBufferSize = dR_softmax_getRequiredOutputBufferSize;
    l->createKernel = dR_softmax_createKernel;
    l->allocateBuffers = dR_softmax_allocateBuffers;
    l->fillBuffers = dR_softmax_fillBuffers;
    l->cleanupBuffers = dR_softmax_cleanupBuffers;
    l->cleanupLayer = dR_softmax_cleanupLayer;
    l->serializeNode = dR_softmax_serializeNode;
    l->parseAppendNode = dR_softmax_parseAppendNode;
    l->printLayer = dR_softmax_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: Softmax node needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_softmax_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    (void)layer; (void)params; (void)variables; (void)variableSizes;
    *numParams = 0;
    *numVariables = 0;
    return "Softmax";
}

dR_Node *dR_softmax_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    (void)params; (void)variables;
    if (numINodes != 1) { g_print("Parsing Error: Softmax Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 0 || numVariables != 0) { g_print("Parsing Error: Softmax Node needs 0 Parameters and 0 Variables!\n"); return NULL; }
    return dR_Softmax(net, iNodes[0]);
}

gboolean dR_softmax_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

gboolean dR_softmax_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_Softmax_Data *d = (dR_Softmax_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("Softmax Node with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    d->ishape = dR_firstInput(layer)->oshape;
    layer->oshape = d->ishape;
    return TRUE;
}

gint32 dR_softmax_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_softmax_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_softmax_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_softmax_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_softmax_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_softmax_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

gboolean dR_softmax_compute(dR_Graph *net, dR_Node *layer)
{
    dR_Node *in = dR_firstInput(layer);
    if (!denseInput(layer, in)) return FALSE;
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_softmax(net->clConfig->clCommandQueue, dR_actPtr(in), dR_actPtr(layer), net->config->batchSize, denseSize(layer));
    return dR_finishCLKernel(net, "deepRACIN:softmax");
}

gchar *dR_softmax_printLayer(dR_Node *layer) { return g_strdup_printf("Softmax node: %d\n", layer->layerID); }
