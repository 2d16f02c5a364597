/*
 * Graph core of the CUDA build: node registration, feed nodes, scheduling, the
 * liveness-based activation-buffer planner, kernel-variant selection and cleanup.
 * Same roles and entry points as the reference's src/dR_core.c; the device work behind
 * them is CUDA.
 *
 * Layouts.  Every node keeps its activations in N-HWC (`node->act`).  Buffers the API
 * exposes -- a feed node's buffer and an output node's buffer, both `node->outputBuf` --
 * hold the reference's [C][H][W] layout (include/deepRACIN.h:61) unless the graph was
 * switched to DR_LAYOUT_HWC.  Where both layouts describe the same bytes (W*H == 1,
 * C == 1 or HWC interface) `act` and `outputBuf` are one handler and no conversion runs.
 */
#include "dR_core.h"
#include "dR_b200.h"
#include "dR_kernels.h"
#include "dR_parser.h"

dR_Node *dR_newNode(dR_LayerType type, void *data)
{
    dR_Node *l = (dR_Node *)calloc(1, sizeof(dR_Node));
    l->type = type;
    l->layer = data;
    l->previous_layers = dR_list_createEmptyList();
    l->next_layers = dR_list_createEmptyList();
    return l;
}

void dR_linkNodes(dR_Node *input, dR_Node *l)
{
    dR_list_append(l->previous_layers, input);
    dR_list_append(input->next_layers, l);
}

dR_Node *dR_nthInput(dR_Node *l, gint n)
{
    dR_ListElement *e = l->previous_layers->first;
    while (e && n-- > 0) e = e->next;
    return e ? (dR_Node *)e->element : NULL;
}

dR_Node *dR_firstInput(dR_Node *l) { return dR_nthInput(l, 0); }

float *dR_actPtr(dR_Node *l)
{
    if (!l || !l->act || !l->act->bufptr) return NULL;
    return (float *)(*l->act->bufptr);
}

/* reference src/dR_core.c:6-16 */
dR_Graph *dR_appendLayer(dR_Graph *net, dR_Node *l)
{
    l->propagated = FALSE;
    l->output = FALSE;
    l->queued = FALSE;
    l->layerID = net->number_of_layers;
    if (l->type != tDataFeedNode) l->outputBuf = NULL;
    dR_list_append(net->allNodes, l);
    net->number_of_layers++;
    return net;
}

static gboolean layoutsCoincide(dR_Graph *net, dR_Shape3 s)
{
    return net->config->interfaceLayout == DR_LAYOUT_HWC || s.s0 * s.s1 == 1 || s.s2 == 1;
}

/* ------------------------------------------------------------- feed node */
/* reference src/dR_core.c:18-42 */
dR_Node *dR_Datafeednode(dR_Graph *net, dR_Shape3 *shape)
{
    dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)calloc(1, sizeof(dR_DataFeedNode_Data));
    d->shape = *shape;
    dR_Node *l = dR_newNode(tDataFeedNode, d);
    dR_list_append(net->feed_layers, l);
    l->printLayer = dR_datafeednode_printLayer;
    l->allocateBuffers = dR_datafeednode_allocateBuffers;
    l->getRequiredOutputBufferSize = dR_datafeednode_getRequiredOutputBufferSize;
    l->cleanupLayer = dR_datafeednode_cleanupLayer;
    l->serializeNode = dR_datafeednode_serializeNode;
    l->parseAppendNode = dR_datafeednode_parseAppendNode;
    l->compute = dR_datafeednode_compute;
    dR_appendLayer(net, l);
    return l;
}

gchar *dR_datafeednode_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],
                                     gint variableSizes[], gint *numVariables)
{
    dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)layer->layer;
    (void)variables; (void)variableSizes;
    if (*numParams < 3) { g_print("DataFeedNode needs space for 3 parameters and 0 variables!\n"); return NULL; }
    *numParams = 3;
    params[0] = g_strdup_printf("%d", d->shape.s0);
    params[1] = g_strdup_printf("%d", d->shape.s1);
    params[2] = g_strdup_printf("%d", d->shape.s2);
    *numVariables = 0;
    return "DataFeedNode";
}

dR_Node *dR_datafeednode_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params,
                                         gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape3 shape;
    (void)iNodes; (void)variables;
    if (numINodes != 0) { g_print("Parsing Error: DataFeedNode Node needs 0 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 3 || numVariables != 0) { g_print("Parsing Error: DataFeedNode Node needs 3 Parameters and 0 Variables!\n"); return NULL; }
    shape.s0 = atoi(params[0]); shape.s1 = atoi(params[1]); shape.s2 = atoi(params[2]);
    return dR_Datafeednode(net, &shape);
}

gchar *dR_datafeednode_printLayer(dR_Node *layer)
{
    dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)layer->layer;
    return g_strdup_printf("DataFeedNode: %d\n Data dimensions: %dx%dx%d\n", layer->layerID, d->shape.s0, d->shape.s1, d->shape.s2);
}

gboolean dR_datafeednode_allocateBuffers(dR_Graph *net, dR_Node *layer)
{
    /* the interface buffer; user-supplied buffers (dR_setDataFeedNodeBuffer) are left alone */
    if (layer->outputBuf->outputBuf) return TRUE;
    if (!dR_createFloatBufferL(net, &layer->outputBuf->buf, (size_t)layer->outputBuf->size * net->config->batchSize)) return FALSE;
    if (net->config->feedOverlap && !net->config->useCudaGraph) return dR_feedOverlapInit(net, layer);
    return TRUE;
}

gint32 dR_datafeednode_getRequiredOutputBufferSize(dR_Node *layer)
{
    dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)layer->layer;
    return d->shape.s0 * d->shape.s1 * d->shape.s2;
}

gboolean dR_datafeednode_cleanupLayer(dR_Graph *net, dR_Node *layer)
{
    (void)net;
    g_free(layer->layer);
    return TRUE;
}

/* interface layout -> N-HWC, once per apply */
gboolean dR_datafeednode_compute(dR_Graph *net, dR_Node *layer)
{
    if (layer->act == layer->outputBuf) return TRUE;
    dR_beginCLKernel(net);
    net->clConfig->clError = dRk_chw_to_hwc(net->clConfig->clCommandQueue, (const float *)*layer->outputBuf->bufptr,
                                            dR_actPtr(layer), net->config->batchSize, layer->oshape.s0, layer->oshape.s1, layer->oshape.s2);
    return dR_finishCLKernel(net, "deepRACIN:feedLayout");
}

/* ------------------------------------------------------------- scheduling */
/*
 * Breadth-first walk from the feed nodes; a node is processed once every predecessor has
 * a shape, otherwise it goes back to the end of the queue.  The resulting queue order is
 * the execution order (reference src/dR_core.c:121-211).
 */
gboolean dR_propagateShapesAndSchedule(dR_Graph *net)
{
    if (net->feed_layers->length == 0) {
        g_print("A minimum of one data feed node is required to prepare the net application!\n");
        return FALSE;
    }
    gint total = net->allNodes->length;
    dR_Node **queue = (dR_Node **)calloc((size_t)total + 1, sizeof(dR_Node *));
    gint qlen = 0;
    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next) {
        dR_Node *f = (dR_Node *)e->element;
        dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)f->layer;
        f->oshape = d->shape;
        f->propagated = TRUE;
        for (dR_ListElement *n = f->next_layers->first; n; n = n->next) {
            dR_Node *nx = (dR_Node *)n->element;
            if (!nx->queued) { queue[qlen++] = nx; nx->queued = TRUE; }
        }
    }
    dR_List *order = dR_list_createEmptyList();
    gint head = 0, stalled = 0;
    /* ring of pending nodes: [head, qlen) in a growing array is enough because every node enters once;
       deferred nodes are rotated by swapping to the back */
    while (head < qlen) {
        dR_Node *l = queue[head];
        gboolean ready = TRUE;
        for (dR_ListElement *p = l->previous_layers->first; p; p = p->next)
            if (!((dR_Node *)p->element)->propagated) ready = FALSE;
        if (!ready) {
            for (gint i = head; i + 1 < qlen; i++) queue[i] = queue[i + 1];
            queue[qlen - 1] = l;
            if (++stalled > qlen - head) {
                g_print("Scheduling failed: node %d waits for an input that is never produced\n", l->layerID);
                free(queue); dR_list_cleanup(order);
                return FALSE;
            }
            continue;
        }
        stalled = 0;
        head++;
        if (!l->propagateShape(net, l)) { g_print("Propagate Shapes failed for Layer %d!\n", l->layerID); free(queue); dR_list_cleanup(order); return FALSE; }
        if (net->config->debugInfo && !net->config->silent)
            g_print("Propagated layer %d: %dx%dx%d\n", l->layerID, l->oshape.s0, l->oshape.s1, l->oshape.s2);
        if (!l->schedule(net, l)) { g_print("Scheduling failed for Layer %d! \n", l->layerID); free(queue); dR_list_cleanup(order); return FALSE; }
        l->propagated = TRUE;
        dR_list_append(order, l);
        for (dR_ListElement *n = l->next_layers->first; n; n = n->next) {
            dR_Node *nx = (dR_Node *)n->element;
            if (!nx->queued) { queue[qlen++] = nx; nx->queued = TRUE; }
        }
    }
    free(queue);
    net->scheduledLayers = order;
    if (net->config->debugInfo && !net->config->silent) dR_printSchedule(net);
    return TRUE;
}

/* ------------------------------------------------------------- fusion plan */
/*
 * A Concat along channels whose inputs are all convolutions with no other consumer needs
 * no copy: each convolution stores straight into the Concat's buffer at its channel offset.
 */
gboolean dR_planFusion(dR_Graph *net)
{
    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next) {
        dR_Node *f = (dR_Node *)e->element;
        f->elided = FALSE; f->act_coffset = 0; f->act_cstride = f->oshape.s2;
    }
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        l->elided = FALSE; l->fusedAway = FALSE; l->act_coffset = 0; l->act_cstride = l->oshape.s2;
    }
    if (!net->config->fuseGraph) return TRUE;
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (l->type != tConcat) continue;
        dR_Concat_Data *c = (dR_Concat_Data *)l->layer;
        c->elidedCopy = FALSE;
        c->fusedGather = FALSE;
        if (c->concatDim != 2) continue;
        if (dR_concat_planGather(l)) continue;
        gboolean ok = TRUE;
        for (dR_ListElement *p = l->previous_layers->first; p; p = p->next) {
            dR_Node *in = (dR_Node *)p->element;
            if (in->type != tConv2d || in->next_layers->length != 1 || in->output) ok = FALSE;
            for (dR_ListElement *q = p->next; q; q = q->next) if (q->element == in) ok = FALSE;
        }
        if (!ok) continue;
        c->elidedCopy = TRUE;
        gint off = 0;
        for (dR_ListElement *p = l->previous_layers->first; p; p = p->next) {
            dR_Node *in = (dR_Node *)p->element;
            in->elided = TRUE;
            in->act_cstride = l->oshape.s2;
            in->act_coffset = off;
            off += in->oshape.s2;
        }
    }
    return TRUE;
}

/* ------------------------------------------------------------- buffer planner */
dR_MemoryHandler *dR_newMemoryHandler(gboolean cust)
{
    dR_MemoryHandler *h = (dR_MemoryHandler *)calloc(1, sizeof(dR_MemoryHandler));
    h->outputFor = dR_list_createEmptyList();
    h->outputBuf = cust;
    h->bufptr = &h->buf;
    return h;
}

void dR_cleanupMemoryHandler(dR_Graph *net, dR_MemoryHandler *h)
{
    if (!h) return;
    if (!h->outputBuf && h->buf) dR_clMemoryBufferCleanup(net, h->buf);
    dR_list_cleanup(h->outputFor);
    g_free(h);
}

static dR_MemoryHandler *takeStreamBuffer(dR_List *all, dR_List *freeList)
{
    if (freeList->length == 0) {
        dR_MemoryHandler *h = dR_newMemoryHandler(FALSE);
        dR_list_append(all, h);
        return h;
    }
    return (dR_MemoryHandler *)dR_list_pop(freeList);
}

static dR_Node *elisionTarget(dR_Node *l)
{
    return l->elided ? (dR_Node *)l->next_layers->first->element : NULL;
}

/* A caller-owned output buffer (dR_setPreexistingOutputBuffer) whose layout is the node's own N-HWC layout is written by the
 * node's kernels directly: no stream buffer, no conversion kernel. */
static gboolean writesIntoCallersBuffer(dR_Graph *net, dR_Node *l)
{
    return l->output && l->outputBuf && l->outputBuf->outputBuf && !l->elided && layoutsCoincide(net, l->oshape);
}

/*
 * Walks the schedule; every node takes a free stream buffer (or a new one), grows it to
 * its need, and releases the buffers of predecessors whose last consumer it was.  Buffers of
 * feed and output nodes are never recycled (reference src/dR_core.c:213-325).
 */
gboolean dR_estimateAndAllocateBuffers(dR_Graph *net)
{
    dR_List *all = dR_list_createEmptyList();
    dR_List *freeList = dR_list_createEmptyList();
    gboolean ret = TRUE;
    size_t scratch = 0;

    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next) {
        dR_Node *f = (dR_Node *)e->element;
        gint req = f->getRequiredOutputBufferSize(f);
        if (f->outputBuf == NULL) f->outputBuf = dR_newMemoryHandler(FALSE);
        dR_list_append(all, f->outputBuf);
        f->outputBuf->size = req;
        f->outputBuf->numberOfDependencies = f->next_layers->length;
        dR_list_append(f->outputBuf->outputFor, f);
        if (layoutsCoincide(net, f->oshape)) f->act = f->outputBuf;
        else {
            f->act = dR_newMemoryHandler(FALSE);
            f->act->size = req;
            dR_list_append(all, f->act);
        }
        f->act_cstride = f->oshape.s2; f->act_coffset = 0;
        if (!f->allocateBuffers(net, f)) { g_print("Buffer allocation failed for feed node %d! \n", f->layerID); return FALSE; }
    }

    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        dR_Node *target = elisionTarget(l);
        gint req = l->getRequiredOutputBufferSize(l);
        if (target) {
            if (!target->act) {
                target->act = writesIntoCallersBuffer(net, target) ? target->outputBuf : takeStreamBuffer(all, freeList);
                target->act->numberOfDependencies = target->next_layers->length;
                gint treq = target->getRequiredOutputBufferSize(target);
                if (target->act->size < treq) target->act->size = treq;
            }
            l->act = target->act;
        } else if (!l->act) {
            l->act = writesIntoCallersBuffer(net, l) ? l->outputBuf : takeStreamBuffer(all, freeList);
            l->act->numberOfDependencies = l->next_layers->length;
            if (l->act->size < req) l->act->size = req;
        }
        dR_list_append(l->act->outputFor, l);
        if (l->scratchFloats > scratch) scratch = l->scratchFloats;

        if (l->output) {
            /* interface buffer of an output node */
            if (l->outputBuf == NULL) {
                if (layoutsCoincide(net, l->oshape) && !l->elided) l->outputBuf = l->act;
                else {
                    l->outputBuf = dR_newMemoryHandler(FALSE);
                    l->outputBuf->size = req;
                    dR_list_append(all, l->outputBuf);
                }
            } else {
                l->outputBuf->size = req;
                dR_list_append(all, l->outputBuf);
            }
        } else {
            l->outputBuf = l->act;
        }

        /* A Slice that a fused Concat evaluates keeps its source alive: the gather kernel reads the source when the
           Concat runs, so the source is released by the Concat (below), after the Concat has taken its own buffer. */
        gboolean deferRelease = l->fusedAway && l->type == tSlice;
        for (dR_ListElement *p = l->previous_layers->first; p && !deferRelease; p = p->next) {
            dR_Node *prev = (dR_Node *)p->element;
            if (prev->type == tDataFeedNode || prev->output || prev->act == l->act) continue;
            if (--prev->act->numberOfDependencies == 0) dR_list_append(freeList, prev->act);
        }
        if (l->type == tConcat && ((dR_Concat_Data *)l->layer)->fusedGather) {
            dR_Node *srcs[DRK_CHANNEL_MAP_MAX];
            gint ns = dR_concat_gatherSources(l, srcs, DRK_CHANNEL_MAP_MAX);
            for (gint i = 0; i < ns; i++) {
                dR_Node *prev = srcs[i];
                if (prev->type == tDataFeedNode || prev->output || prev->act == l->act) continue;
                if (--prev->act->numberOfDependencies == 0) dR_list_append(freeList, prev->act);
            }
        }
        if (!l->allocateBuffers(net, l)) { g_print("Buffer allocation failed for Layer %d! \n", l->layerID); return FALSE; }
    }
    if (!net->config->silent && net->config->debugInfo)
        g_print("Number of required stream buffers: %d, Allocating...\n", all->length);
    net->streamBufferHandlers = all;

    gint maxSize = 0;
    for (dR_ListElement *e = all->first; e; e = e->next) {
        dR_MemoryHandler *h = (dR_MemoryHandler *)e->element;
        if (h->size > maxSize) maxSize = h->size;
        if (h->outputBuf) continue;                 /* user supplied */
        if (h->buf) continue;                       /* feed interface buffer already created */
        h->bufptr = &h->buf;
        ret &= dR_createFloatBufferL(net, &h->buf, (size_t)h->size * net->config->batchSize);
        if (!net->config->silent && net->config->debugInfo) g_print("Stream buffer with size %d created!\n", h->size);
    }
    net->maxBufferSize = maxSize;
    net->scratchFloats = scratch;
    if (scratch) ret &= dR_createFloatBufferL(net, &net->scratch, scratch);
    ret &= dR_createFloatBufferL(net, &net->statusWord, 4);
    if (ret) ret &= dR_zeroBuffer(net, net->statusWord, 4);
    net->hostDebugBuffer = (cl_float *)g_malloc((size_t)(maxSize > 0 ? maxSize : 1) * 4);
    dR_list_cleanup(freeList);
    return ret;
}

/* reference src/dR_core.c:328-341 */
gboolean dR_fillBuffers(dR_Graph *net)
{
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (!l->fillBuffers(net, l)) { g_print("Device buffer filling failed for Layer %d! \n", l->layerID); return FALSE; }
    }
    return TRUE;
}

/*
 * The reference generates OpenCL source per node and builds one program here
 * (src/dR_core.c:371-418).  All CUDA kernels are compiled ahead of time, so this phase only
 * lets every node pick its kernel variant (createKernel); timing-based selection among the
 * legal variants happens after the buffers exist (dR_conv2d_autotune, called by dR_prepare).
 */
gboolean dR_generateAndCompileKernels(dR_Graph *net)
{
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (l->generateKernel && !l->generateKernel(net, l)) { g_print("Kernel Generation failed for Layer %d! \n", l->layerID); return FALSE; }
        if (!l->createKernel(net, l)) { g_print("Kernel selection failed for Layer %d! \n", l->layerID); return FALSE; }
    }
    return TRUE;
}

/* reference src/dR_core.c:421-459 */
void dR_cleanupBuffers(dR_Graph *net)
{
    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next) dR_feedOverlapCleanup(net, (dR_Node *)e->element);
    for (dR_ListElement *e = net->streamBufferHandlers->first; e; e = e->next) {
        dR_MemoryHandler *h = (dR_MemoryHandler *)e->element;
        if (!h->outputBuf && h->buf) { dR_clMemoryBufferCleanup(net, h->buf); h->buf = NULL; }
    }
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (!l->cleanupBuffers(net, l)) g_print("Device buffer cleanup failed for Layer %d! \n", l->layerID);
    }
    if (net->scratch) { dR_clMemoryBufferCleanup(net, net->scratch); net->scratch = NULL; }
    if (net->statusWord) { dR_clMemoryBufferCleanup(net, net->statusWord); net->statusWord = NULL; }
    dR_captureDestroy(net);
}

/* reference src/dR_core.c:461-500 */
void dR_cleanupNet(dR_Graph *net)
{
    if (net->prepared) {
        for (dR_ListElement *e = net->streamBufferHandlers->first; e; e = e->next) {
            dR_MemoryHandler *h = (dR_MemoryHandler *)e->element;
            dR_list_cleanup(h->outputFor);
            g_free(h);
        }
    }
    for (dR_ListElement *e = net->allNodes->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (!l->cleanupLayer(net, l)) g_print("Layer cleanup failed for layer %d! \n", l->layerID);
        dR_list_cleanup(l->previous_layers);
        dR_list_cleanup(l->next_layers);
        g_free(l);
    }
    if (net->prepared) {
        dR_list_cleanup(net->scheduledLayers);
        dR_list_cleanup(net->streamBufferHandlers);
        g_free(net->hostDebugBuffer);
    }
    dR_list_cleanup(net->allNodes);
    dR_list_cleanup(net->output_layers);
    dR_list_cleanup(net->feed_layers);
    g_free(net->clConfig);
    g_free(net->config);
    g_free(net);
}
