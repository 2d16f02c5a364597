/*
 * Slice, Concat and CropOrPad nodes (reference src/dR_nodes_transform.c, kernels
 * Kernels/dR_transform.cl and the generated concat kernel :468-553).
 */
#include "dR_nodes_transform.h"
#include "dR_core.h"
#include "dR_kernels.h"

static gboolean noop(dR_Graph *net, dR_Node *layer) { (void)net; (void)layer; return TRUE; }
static gboolean freeData(dR_Graph *net, dR_Node *layer) { (void)net; g_free(layer->layer); return TRUE; }
static gint32 denseSize(dR_Node *layer) { return layer->oshape.s0 * layer->oshape.s1 * layer->oshape.s2; }

/* -------------------------------------------------------------------- slice */
/* reference src/dR_nodes_transform.c:8-57; origin and shape are (x, y, z, unused) */
dR_Node *dR_Slice(dR_Graph *net, dR_Node *inputLayer, dR_Shape4 *origin, dR_Shape4 *shape)
{
    dR_Slice_Data *d = (dR_Slice_Data *)calloc(1, sizeof(dR_Slice_Data));
    d->origin = *origin;
    d->oshape = *shape;
    dR_Node *l = dR_newNode(tSlice, d);
    l->compute = dR_slice_compute;
    l->schedule = dR_slice_schedule;
    l->propagateShape = dR_slice_propagateShape;
    l->getRequiredOutputBufferSize = dR_slice_getRequiredOutputBufferSize;
    l->createKernel = dR_slice_createKernel;
    l->allocateBuffers = dR_slice_allocateBuffers;
    l->fillBuffers = dR_slice_fillBuffers;
    l->cleanupBuffers = dR_slice_cleanupBuffers;
    l->cleanupLayer = dR_slice_cleanupLayer;
    l->serializeNode = dR_slice_serializeNode;
    l->parseAppendNode = dR_slice_parseAppendNode;
    l->printLayer = dR_slice_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: Slice Node needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_slice_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_Slice_Data *d = (dR_Slice_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 8) { g_print("SerializeNode needs space for 8 parameters and 0 variables!\n"); return NULL; }
    *numParams = 8;
    params[0] = g_strdup_printf("%d", d->origin.s0); params[1] = g_strdup_printf("%d", d->origin.s1);
    params[2] = g_strdup_printf("%d", d->origin.s2); params[3] = g_strdup_printf("%d", d->origin.s3);
    params[4] = g_strdup_printf("%d", d->oshape.s0); params[5] = g_strdup_printf("%d", d->oshape.s1);
    params[6] = g_strdup_printf("%d", d->oshape.s2); params[7] = g_strdup_printf("%d", d->oshape.s3);
    *numVariables = 0;
    return "Slice";
}

dR_Node *dR_slice_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape4 origin, shape;
    (void)variables;
    if (numINodes != 1) { g_print("Parsing Error: Slice Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 8 || numVariables != 0) { g_print("Parsing Error: Slice Node needs 8 Parameters and 0 Variables!\n"); return NULL; }
    origin.s0 = atoi(params[0]); origin.s1 = atoi(params[1]); origin.s2 = atoi(params[2]); origin.s3 = atoi(params[3]);
    shape.s0 = atoi(params[4]); shape.s1 = atoi(params[5]); shape.s2 = atoi(params[6]); shape.s3 = atoi(params[7]);
    return dR_Slice(net, iNodes[0], &origin, &shape);
}

gboolean dR_slice_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

/* reference src/dR_nodes_transform.c:155-174; the slice must lie inside the input (the reference reads out of range otherwise) */
gboolean dR_slice_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_Slice_Data *d = (dR_Slice_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("Extract Slice Node with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    d->ishape = dR_firstInput(layer)->oshape;
    if (d->origin.s0 < 0 || d->origin.s1 < 0 || d->origin.s2 < 0 || d->oshape.s0 <= 0 || d->oshape.s1 <= 0 || d->oshape.s2 <= 0 ||
        d->origin.s0 + d->oshape.s0 > d->ishape.s0 || d->origin.s1 + d->oshape.s1 > d->ishape.s1 || d->origin.s2 + d->oshape.s2 > d->ishape.s2) {
        g_print("Slice Node %d: slice [%d,%d,%d]+[%d,%d,%d] leaves the input %dx%dx%d\n", layer->layerID, d->origin.s0, d->origin.s1, d->origin.s2,
                d->oshape.s0, d->oshape.s1, d->oshape.s2, d->ishape.s0, d->ishape.s1, d->ishape.s2);
        return FALSE;
    }
    layer->oshape.s0 = d->oshape.s0; layer->oshape.s1 = d->oshape.s1; layer->oshape.s2 = d->oshape.s2;
    return TRUE;
}

gint32 dR_slice_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_slice_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_slice_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_slice_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_slice_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_slice_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

/* reference src/dR_nodes_transform.c:123-153 */
gboolean dR_slice_compute(dR_Graph *net, dR_Node *layer)
{
    dR_Slice_Data *d = (dR_Slice_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_slice(net->clConfig->clCommandQueue, dR_actPtr(in) + in->act_coffset, dR_actPtr(layer), net->config->batchSize,
                                       d->ishape.s0, d->ishape.s1, d->ishape.s2, d->origin.s0, d->origin.s1, d->origin.s2,
                                       d->oshape.s0, d->oshape.s1, d->oshape.s2, in->act_cstride);
    return dR_finishCLKernel(net, "deepRACIN:extractSlice");
}

gchar *dR_slice_printLayer(dR_Node *layer)
{
    dR_Slice_Data *d = (dR_Slice_Data *)layer->layer;
    return g_strdup_printf("Extract Slice Node: %d\n Origin: [%d, %d, %d, %d]\n Size: [%d, %d, %d, %d]\n", layer->layerID,
                           d->origin.s0, d->origin.s1, d->origin.s2, d->origin.s3, d->oshape.s0, d->oshape.s1, d->oshape.s2, d->oshape.s3);
}

/* ------------------------------------------------------------------- concat */
/* reference src/dR_nodes_transform.c:238-281; n in 1..3 */
dR_Node *dR_Concat(dR_Graph *net, dR_Node **inputNodes, gint n, gint concatDim)
{
    if (!inputNodes || n < 1 || n > 3 || concatDim < 0 || concatDim > 2) {
        g_print("Error: Concat node needs 1 to 3 input nodes and a dimension 0..2 \n");
        return NULL;
    }
    for (gint i = 0; i < n; i++) if (!inputNodes[i]) { g_print("Error: Concat node got a NULL input\n"); return NULL; }
    dR_Concat_Data *d = (dR_Concat_Data *)calloc(1, sizeof(dR_Concat_Data));
    d->n = n;
    d->concatDim = concatDim;
    dR_Node *l = dR_newNode(tConcat, d);
    l->compute = dR_concat_compute;
    l->schedule = dR_concat_schedule;
    l->propagateShape = dR_concat_propagateShape;
    l->getRequiredOutputBufferSize = dR_concat_getRequiredOutputBufferSize;
    l->createKernel = dR_concat_createKernel;
    l->allocateBuffers = dR_concat_allocateBuffers;
    l->fillBuffers = dR_concat_fillBuffers;
    l->cleanupBuffers = dR_concat_cleanupBuffers;
    l->cleanupLayer = dR_concat_cleanupLayer;
    l->serializeNode = dR_concat_serializeNode;
    l->parseAppendNode = dR_concat_parseAppendNode;
    l->printLayer = dR_concat_printLayer;
    for (gint i = 0; i < n; i++) dR_linkNodes(inputNodes[i], l);
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_concat_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 2) { g_print("SerializeNode needs space for 2 parameters and 0 variables!\n"); return NULL; }
    *numParams = 2;
    params[0] = g_strdup_printf("%d", d->n);
    params[1] = g_strdup_printf("%d", d->concatDim);
    *numVariables = 0;
    return "Concat";
}

dR_Node *dR_concat_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    (void)variables;
    if (numParams != 2 || numVariables != 0) { g_print("Parsing Error: Concat Node needs 2 Parameters and 0 Variables!\n"); return NULL; }
    gint n = atoi(params[0]);
    if (n != numINodes) { g_print("Parsing Error: Concat Node declares %d inputs but lists %d!\n", n, numINodes); return NULL; }
    return dR_Concat(net, iNodes, n, atoi(params[1]));
}

gboolean dR_concat_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

/* reference src/dR_nodes_transform.c:377-401: first input's shape, concat dim summed; the other dims must agree */
gboolean dR_concat_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    if (layer->previous_layers->length != d->n) {
        if (!net->config->silent) g_print("Concat Layer Error: Parameter n does not match number of given inputnodes!\n");
        return FALSE;
    }
    dR_Node *first = dR_firstInput(layer);
    layer->oshape = first->oshape;
    d->maxInputSizeInConcatDim = 0;
    for (gint i = 0; i < d->n; i++) {
        gint *sh = (gint *)&dR_nthInput(layer, i)->oshape;
        gint *fs = (gint *)&first->oshape;
        for (gint k = 0; k < 3; k++)
            if (k != d->concatDim && sh[k] != fs[k]) { g_print("Concat Layer %d: inputs disagree in dimension %d\n", layer->layerID, k); return FALSE; }
        d->inputSizesInConcatDim[i] = sh[d->concatDim];
        if (sh[d->concatDim] > d->maxInputSizeInConcatDim) d->maxInputSizeInConcatDim = sh[d->concatDim];
        if (i > 0) ((gint *)&layer->oshape)[d->concatDim] += sh[d->concatDim];
    }
    return TRUE;
}

gint32 dR_concat_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_concat_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_concat_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_concat_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_concat_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_concat_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

/* Walks one Concat input back through single-consumer scalar element-wise nodes to a full-frame Slice.
 * Returns the slice node (ops filled source-to-sink) or NULL if the chain has any other shape. */
static dR_Node *gatherChain(dR_Node *in, gint ops[4], gfloat scalars[4], gint *nops)
{
    gint rev[4]; gfloat rs[4]; gint n = 0;
    dR_Node *nd = in;
    while (nd->type == tElemWise1Op) {
        dR_ElemWise1Op_Data *e = (dR_ElemWise1Op_Data *)nd->layer;
        if (n == 4 || nd->output || nd->next_layers->length != 1 || e->op > tDivS) return NULL;
        rev[n] = e->op; rs[n] = e->scalar; n++;
        nd = dR_firstInput(nd);
    }
    if (nd->type != tSlice || nd->output || nd->next_layers->length != 1) return NULL;
    dR_Slice_Data *sl = (dR_Slice_Data *)nd->layer;
    if (sl->origin.s0 != 0 || sl->origin.s1 != 0 || sl->oshape.s0 != sl->ishape.s0 || sl->oshape.s1 != sl->ishape.s1) return NULL;
    for (gint k = 0; k < n; k++) { ops[k] = rev[n - 1 - k]; scalars[k] = rs[n - 1 - k]; }
    *nops = n;
    return nd;
}

gboolean dR_concat_planGather(dR_Node *layer)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    gint ops[4], nops; gfloat sc[4];
    if (d->concatDim != 2 || layer->oshape.s2 > DRK_CHANNEL_MAP_MAX) return FALSE;
    for (gint i = 0; i < d->n; i++)
        if (!gatherChain(dR_nthInput(layer, i), ops, sc, &nops)) return FALSE;
    for (gint i = 0; i < d->n; i++) {       /* the chain nodes compute nothing on their own any more */
        dR_Node *nd = dR_nthInput(layer, i);
        while (nd->type == tElemWise1Op) { nd->fusedAway = TRUE; nd = dR_firstInput(nd); }
        nd->fusedAway = TRUE;
    }
    d->fusedGather = TRUE;
    return TRUE;
}

/* The source node of every Slice chain of a fused Concat, one entry per Concat input (a source feeding several
 * chains appears once per chain, as it does in the Slices' dependency counts).  Returns the number of entries. */
gint dR_concat_gatherSources(dR_Node *layer, dR_Node **srcs, gint maxSrcs)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    gint n = 0;
    for (gint i = 0; i < d->n && n < maxSrcs; i++) {
        gint ops[4], nops; gfloat sc[4];
        dR_Node *sl = gatherChain(dR_nthInput(layer, i), ops, sc, &nops);
        if (sl) srcs[n++] = dR_firstInput(sl);
    }
    return n;
}

/* The gather of a fused Concat as an affine per-channel map of ONE source tensor, if it is that simple: at most four
 * channels, every chain from the same source, at most one scalar op per chain and that op exact as one FMA
 * (AddS, SubS, MulS).  A few-channel first convolution can then evaluate it while it reads its input. */
gboolean dR_concat_gatherAsInputMap(dR_Node *layer, dR_Node **srcOut, gint ch[4], gfloat scale[4], gfloat shift[4])
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    dR_Node *src0 = NULL;
    gint j = 0;
    if (layer->type != tConcat || !d->fusedGather || layer->oshape.s2 > 4) return FALSE;
    for (gint i = 0; i < d->n; i++) {
        gint ops[4], nops; gfloat sc[4];
        dR_Node *sl = gatherChain(dR_nthInput(layer, i), ops, sc, &nops);
        if (!sl || nops > 1) return FALSE;
        if (nops == 1 && ops[0] != tAddS && ops[0] != tSubS && ops[0] != tMulS) return FALSE;
        dR_Node *src = dR_firstInput(sl);
        if (src0 && src != src0) return FALSE;
        src0 = src;
        dR_Slice_Data *sd = (dR_Slice_Data *)sl->layer;
        for (gint c = 0; c < sd->oshape.s2; c++, j++) {
            if (j >= 4) return FALSE;
            ch[j] = sd->origin.s2 + c;
            scale[j] = (nops == 1 && ops[0] == tMulS) ? sc[0] : 1.0f;
            shift[j] = nops == 0 ? 0.0f : ops[0] == tAddS ? sc[0] : ops[0] == tSubS ? -sc[0] : 0.0f;
        }
    }
    if (!src0 || j != layer->oshape.s2) return FALSE;
    *srcOut = src0;
    return TRUE;
}

static gboolean concatGather(dR_Graph *net, dR_Node *layer)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    drk_ChannelMap m;
    gint j = 0;
    memset(&m, 0, sizeof m);
    for (gint i = 0; i < d->n; i++) {
        gint ops[4], nops; gfloat sc[4];
        dR_Node *sl = gatherChain(dR_nthInput(layer, i), ops, sc, &nops);
        if (!sl) return FALSE;
        dR_Slice_Data *sd = (dR_Slice_Data *)sl->layer;
        dR_Node *src = dR_firstInput(sl);
        for (gint c = 0; c < sd->oshape.s2; c++, j++) {
            m.src[j] = dR_actPtr(src) + src->act_coffset;
            m.ld[j] = src->act_cstride;
            m.ch[j] = sd->origin.s2 + c;
            m.nops[j] = nops;
            for (gint k = 0; k < nops; k++) { m.op[j][k] = ops[k]; m.scalar[j][k] = sc[k]; }
        }
    }
    m.cout = j;
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_channel_map(net->clConfig->clCommandQueue, &m, dR_actPtr(layer),
                                             (size_t)net->config->batchSize * layer->oshape.s0 * layer->oshape.s1);
    return dR_finishCLKernel(net, "deepRACIN:concatGather");
}

/* reference src/dR_nodes_transform.c:346-375; nothing to launch when the producers already wrote in place */
gboolean dR_concat_compute(dR_Graph *net, dR_Node *layer)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    if (d->elidedCopy) return TRUE;
    if (d->fusedGather) return concatGather(net, layer);
    gint off = 0;
    dR_beginCLKernel(net);
    for (gint i = 0; i < d->n; i++) {
        dR_Node *in = dR_nthInput(layer, i);
        net->clConfig->clError = dRk_concat_place(net->clConfig->clCommandQueue, dR_actPtr(in) + in->act_coffset, dR_actPtr(layer), net->config->batchSize,
                                                  in->oshape.s0, in->oshape.s1, in->oshape.s2, d->concatDim, off,
                                                  layer->oshape.s0, layer->oshape.s1, layer->oshape.s2, in->act_cstride);
        if (net->clConfig->clError) break;
        off += d->inputSizesInConcatDim[i];
    }
    return dR_finishCLKernel(net, "deepRACIN:concat");
}

gchar *dR_concat_printLayer(dR_Node *layer)
{
    dR_Concat_Data *d = (dR_Concat_Data *)layer->layer;
    return g_strdup_printf("Concat Node: %d\n Number of inputs: %d\n Concat dimension: %d\n", layer->layerID, d->n, d->concatDim);
}

/* -------------------------------------------------------------- crop or pad */
/* reference src/dR_nodes_transform.c:576-615 (which leaves the target depth unset; it is taken from the argument here) */
dR_Node *dR_CropOrPad(dR_Graph *net, dR_Node *inputLayer, dR_Shape3 *shape)
{
    dR_CropOrPad_Data *d = (dR_CropOrPad_Data *)calloc(1, sizeof(dR_CropOrPad_Data));
    d->oshape = *shape;
    dR_Node *l = dR_newNode(tCropOrPad, d);
    l->compute = dR_croporpad_compute;
    l->schedule = dR_croporpad_schedule;
    l->propagateShape = dR_croporpad_propagateShape;
    l->getRequiredOutputBufferSize = dR_croporpad_getRequiredOutputBufferSize;
    l->createKernel = dR_croporpad_createKernel;
    l->allocateBuffers = dR_croporpad_allocateBuffers;
    l->fillBuffers = dR_croporpad_fillBuffers;
    l->cleanupBuffers = dR_croporpad_cleanupBuffers;
    l->cleanupLayer = dR_croporpad_cleanupLayer;
    l->serializeNode = dR_croporpad_serializeNode;
    l->parseAppendNode = dR_croporpad_parseAppendNode;
    l->printLayer = dR_croporpad_printLayer;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: CropOrPad Node needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_croporpad_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_CropOrPad_Data *d = (dR_CropOrPad_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 3) { g_print("SerializeNode needs space for 3 parameters and 0 variables!\n"); return NULL; }
    *numParams = 3;
    params[0] = g_strdup_printf("%d", d->oshape.s0);
    params[1] = g_strdup_printf("%d", d->oshape.s1);
    params[2] = g_strdup_printf("%d", d->oshape.s2);
    *numVariables = 0;
    return "CropOrPad";
}

dR_Node *dR_croporpad_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape3 shape;
    (void)variables;
    if (numINodes != 1) { g_print("Parsing Error: CropOrPad Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 3 || numVariables != 0) { g_print("Parsing Error: CropOrPad Node needs 3 Parameters and 0 Variables!\n"); return NULL; }
    shape.s0 = atoi(params[0]); shape.s1 = atoi(params[1]); shape.s2 = atoi(params[2]);
    return dR_CropOrPad(net, iNodes[0], &shape);
}

gboolean dR_croporpad_schedule(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }

gboolean dR_croporpad_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_CropOrPad_Data *d = (dR_CropOrPad_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("CropOrPad Node with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    d->ishape = dR_firstInput(layer)->oshape;
    if (d->oshape.s2 <= 0) d->oshape.s2 = d->ishape.s2;
    if (d->oshape.s0 <= 0 || d->oshape.s1 <= 0) { g_print("CropOrPad Node %d: target size must be positive\n", layer->layerID); return FALSE; }
    layer->oshape = d->oshape;
    return TRUE;
}

gint32 dR_croporpad_getRequiredOutputBufferSize(dR_Node *layer) { return denseSize(layer); }
gboolean dR_croporpad_createKernel(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_croporpad_allocateBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_croporpad_fillBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_croporpad_cleanupBuffers(dR_Graph *net, dR_Node *layer) { return noop(net, layer); }
gboolean dR_croporpad_cleanupLayer(dR_Graph *net, dR_Node *layer) { return freeData(net, layer); }

gboolean dR_croporpad_compute(dR_Graph *net, dR_Node *layer)
{
    dR_CropOrPad_Data *d = (dR_CropOrPad_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_croporpad(net->clConfig->clCommandQueue, dR_actPtr(in) + in->act_coffset, dR_actPtr(layer), net->config->batchSize,
                                           d->ishape.s0, d->ishape.s1, d->ishape.s2, d->oshape.s0, d->oshape.s1, d->oshape.s2, in->act_cstride);
    return dR_finishCLKernel(net, "deepRACIN:cropOrPad");
}

gchar *dR_croporpad_printLayer(dR_Node *layer)
{
    dR_CropOrPad_Data *d = (dR_CropOrPad_Data *)layer->layer;
    return g_strdup_printf("CropOrPad Node: %d\n Target size: [%d, %d, %d]\n", layer->layerID, d->oshape.s0, d->oshape.s1, d->oshape.s2);
}
