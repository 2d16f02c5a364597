/*
 * Public API of the CUDA build: graph lifetime, configuration, prepare / apply, feeding
 * and fetching.  Entry points, argument meaning and error behaviour (TRUE/FALSE or NULL
 * plus a message on stdout, never an abort) follow the reference's src/deepRACIN.c.
 */
#include <sys/time.h>
#include "deepRACIN.h"
#include "dR_kernels.h"
#include "dR_parser.h"

static double wallMs(void)
{
    struct timeval tv;
    gettimeofday(&tv, NULL);
    return tv.tv_sec * 1000.0 + tv.tv_usec / 1000.0;
}

static int envInt(const char *name, int dflt)
{
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

/* reference src/deepRACIN.c:6-47 */
dR_Graph *dR_NewGraph(void)
{
    dR_Graph *a = (dR_Graph *)calloc(1, sizeof(dR_Graph));
    a->clConfig = (dR_ClConfig *)calloc(1, sizeof(dR_ClConfig));
    a->config = (dR_Config *)calloc(1, sizeof(dR_Config));
    a->clConfig->clEvent = &a->clConfig->clEventObject;
    a->clConfig->clDeviceType = CL_DEVICE_TYPE_GPU;
    a->clConfig->clDeviceNumber = 0;
    a->clConfig->clInfo = TRUE;
    a->clConfig->clKernelPath = "";
    a->clConfig->clPlatformName = " ";
    a->clConfig->fastRelaxedMath = TRUE;
    a->clConfig->forceRecompile = TRUE;
    a->config->silent = TRUE;
    a->config->batchSize = 1;
    a->config->mathMode = envInt("DR_MATH", DR_MATH_FP32);
    a->config->interfaceLayout = DR_LAYOUT_CHW;
    a->config->convAlgo = envInt("DR_CONV_ALGO", DR_CONV_AUTO);
    a->config->autotune = envInt("DR_AUTOTUNE", 0);
    a->config->fuseGraph = envInt("DR_FUSE", 1);
    a->config->useCudaGraph = envInt("DR_CUDA_GRAPH", 0);
    a->feed_layers = dR_list_createEmptyList();
    a->output_layers = dR_list_createEmptyList();
    a->allNodes = dR_list_createEmptyList();
    a->debugLayer = -1;
    return a;
}

/* reference src/deepRACIN.c:51-72 */
gint dR_getOutputBuffers(dR_Graph *net, cl_mem **outptr)
{
    int i = 0;
    if (!net->prepared) {
        g_print("dR_Graph must be prepared before having output buffers. Call dR_prepare first! \n");
        return 0;
    }
    for (dR_ListElement *e = net->output_layers->first; e && i < 10; e = e->next)
        outptr[i++] = ((dR_Node *)e->element)->outputBuf->bufptr;
    return i;
}

/* reference src/deepRACIN.c:74-77 */
void dR_feedData(dR_Graph *net, dR_Node *feednode, gfloat *data, gint offset, gint numfloats)
{
    if (!net->prepared || !feednode || !feednode->outputBuf) {
        g_print("dR_feedData: graph must be prepared and the node must be a data feed node.\n");
        return;
    }
    dR_uploadArray(net, "", data, (size_t)offset * sizeof(cl_float), (size_t)numfloats * sizeof(cl_float),
                   *feednode->outputBuf->bufptr);
}

/* reference src/deepRACIN.c:79-99 */
gboolean dR_setDataFeedNodeBuffer(dR_Graph *net, dR_Node *node, cl_mem *buf)
{
    if (node->type != tDataFeedNode) {
        if (!net->config->silent) g_print("dR_setDataFeedNodeBuffer Error: Data Feed Buffer can only be set to a DataFeedNode!\n");
        return FALSE;
    }
    if (net->prepared) {
        /* same handler, new pointer: allowed between applies.  A captured CUDA graph holds the old address in its
           kernel arguments and tensor maps, so it is dropped here and captured again by the next dR_apply. */
        node->outputBuf->bufptr = buf;
        dR_captureDestroy(net);
        return TRUE;
    }
    dR_DataFeedNode_Data *d = (dR_DataFeedNode_Data *)node->layer;
    node->outputBuf = dR_newMemoryHandler(TRUE);
    node->outputBuf->bufptr = buf;
    node->outputBuf->size = d->shape.s0 * d->shape.s1 * d->shape.s2;
    return TRUE;
}

/* reference src/deepRACIN.c:102-120; ResolveRoI is not part of this build, the values are only stored. */
gboolean dR_setNodeRoI(dR_Node *node, dR_Shape3 origin)
{
    if (!node || !node->outputBuf) return FALSE;
    node->outputBuf->regionOfInterest = TRUE;
    node->outputBuf->useIndexBufferForRoI = FALSE;
    node->outputBuf->roiOrigin = origin;
    return TRUE;
}

gboolean dR_setNodeRoIBufferAndIndex(dR_Node *node, cl_mem *buf, gint index)
{
    if (!node || !node->outputBuf) return FALSE;
    node->outputBuf->regionOfInterest = TRUE;
    node->outputBuf->useIndexBufferForRoI = TRUE;
    node->outputBuf->index = index;
    node->outputBuf->indexBuffer = buf;
    return TRUE;
}

/* reference src/deepRACIN.c:122-131 */
gboolean dR_setPreexistingOutputBuffer(dR_Graph *net, dR_Node *node, cl_mem *buf)
{
    if (net->prepared) { g_print("dR_setPreexistingOutputBuffer must be called before dR_prepare.\n"); return FALSE; }
    node->outputBuf = dR_newMemoryHandler(TRUE);
    node->outputBuf->bufptr = buf;
    if (!node->output) dR_setAsOutput(net, node);
    return TRUE;
}

/* reference src/deepRACIN.c:133-141 */
gboolean dR_setAsOutput(dR_Graph *net, dR_Node *node)
{
    if (!node) return FALSE;
    if (!node->output) {
        node->output = TRUE;
        dR_list_append(net->output_layers, node);
    }
    return TRUE;
}

/* reference src/deepRACIN.c:144-146 */
gboolean dR_initCL(dR_Graph *net) { return dR_clInit(net); }

gboolean dR_conv2d_autotune(dR_Graph *net);

/* reference src/deepRACIN.c:148-202 */
gboolean dR_prepare(dR_Graph *net)
{
    if (net->prepared) { g_print("dR_prepare: graph is already prepared\n"); return FALSE; }
    if (!net->config->dryRun && !net->clConfig->clCommandQueue && !dR_clInit(net)) { g_print("dR_prepare: no CUDA device/stream (call dR_initCL)\n"); return FALSE; }
    if (!net->config->silent) g_print("Propagate shapes and schedule...\n");
    if (!dR_propagateShapesAndSchedule(net)) { g_print("dR_propagateShapesAndSchedule Failed \n"); return FALSE; }
    if (!dR_planFusion(net)) return FALSE;
    if (!net->config->silent) g_print("Done.\nSelect kernel variants...\n");
    if (!dR_generateAndCompileKernels(net)) { g_print("\ndR_generateAndCompileKernels Failed \n"); return FALSE; }
    if (!net->config->silent) g_print("Done.\nEstimate and allocate buffers...\n");
    if (!dR_estimateAndAllocateBuffers(net)) { g_print("dR_estimateAndAllocateBuffers Failed \n"); return FALSE; }
    if (!net->config->silent) g_print("Done. \nFill buffers...\n");
    if (!dR_fillBuffers(net)) { g_print("dR_fillBuffers Failed \n"); return FALSE; }
    if (!net->config->silent) g_print("Done.\n\n");
    net->prepared = TRUE;
    if (net->config->autotune && !net->config->dryRun && !dR_conv2d_autotune(net)) { g_print("variant autotuning failed\n"); return FALSE; }
    if (!dR_finish(net)) return FALSE;
    if (net->config->profilingGPU) {
        g_print("\nGPU Profiling: Whole graph GPU memory consumption: %4.6f MB \n\n", (double)net->clConfig->memConsumptionGPU / 1048576.0);
        net->clConfig->totalKernelGPUTime = 0;
    }
    return TRUE;
}

/* The device addresses a captured schedule has baked in: every feed and output interface buffer.  A caller may replace
 * the pointer behind a handler between applies (its own cl_mem variable); a replay must then not use the old capture. */
static size_t interfaceKey(dR_Graph *net)
{
    size_t key = 1469598103934665603ull;
    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next)
        key = (key ^ (size_t)*((dR_Node *)e->element)->outputBuf->bufptr) * 1099511628211ull;
    for (dR_ListElement *e = net->output_layers->first; e; e = e->next)
        key = (key ^ (size_t)*((dR_Node *)e->element)->outputBuf->bufptr) * 1099511628211ull;
    return key;
}

static gboolean launchSchedule(dR_Graph *net, gboolean capturing)
{
    for (dR_ListElement *e = net->feed_layers->first; e; e = e->next) {
        dR_Node *f = (dR_Node *)e->element;
        if (!f->compute(net, f)) { g_print("Execution of feed layer %d failed \n", f->layerID); return FALSE; }
    }
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *l = (dR_Node *)e->element;
        if (l->fusedAway) continue;                 /* evaluated inside a consumer's kernel */
        const gdouble before = net->clConfig->totalKernelGPUTime;
        if (!l->compute(net, l)) { g_print("Execution of layer %d failed \n", l->layerID); return FALSE; }
        if (net->config->profilingGPU) l->lastGpuMs = net->clConfig->totalKernelGPUTime - before;
        if (l->output && l->outputBuf != l->act) {
            dR_beginCLKernel(net);
            net->clConfig->clError = dRk_hwc_to_chw(net->clConfig->clCommandQueue, dR_actPtr(l), (float *)*l->outputBuf->bufptr,
                                                    net->config->batchSize, l->oshape.s0, l->oshape.s1, l->oshape.s2);
            if (!dR_finishCLKernel(net, "deepRACIN:outputLayout")) return FALSE;
        }
        if (l->layerID == net->debugLayer && net->config->batchSize == 1 && !capturing)     /* a blocking download would end the capture */
            dR_downloadArray(net, "", l->outputBuf->bufptr, 0, (size_t)l->oshape.s0 * l->oshape.s1 * sizeof(cl_float), net->hostDebugBuffer);
    }
    return TRUE;
}

/* reference src/deepRACIN.c:204-270 */
gboolean dR_apply(dR_Graph *net)
{
    double t0 = 0;
    if (!net->prepared) { g_print("dR_apply: call dR_prepare first!\n"); return FALSE; }
    if (net->config->dryRun) { g_print("dR_apply: graph was prepared as a dry run (no device); nothing can be computed\n"); return FALSE; }
    if (net->config->debugInfo) g_print("Applying graph...\n");
    if (net->config->profilingCPU) { t0 = wallMs(); net->config->totalNodeCPUTime = 0.0; }
    if (net->config->useCudaGraph && !net->config->profilingGPU) {
        const size_t key = interfaceKey(net);
        if (net->graphExec && net->captureKey != key) dR_captureDestroy(net);
        if (!net->graphExec) {
            if (!dR_captureBegin(net)) return FALSE;
            gboolean ok = launchSchedule(net, TRUE);
            if (!dR_captureEnd(net) || !ok) return FALSE;
            net->captureKey = key;
        }
        if (!dR_captureLaunch(net)) return FALSE;
    } else {
        if (net->config->feedOverlap && !dR_feedOverlapBeforeApply(net)) return FALSE;
        if (!launchSchedule(net, FALSE)) return FALSE;
        if (net->config->feedOverlap && !dR_feedOverlapAfterApply(net)) return FALSE;
    }
    if (net->config->profilingGPU) {
        g_print("GPU Profiling: Sum of all kernel run times: %2.3fms \n", net->clConfig->totalKernelGPUTime);
        net->clConfig->sumTotalKernelGPUTime += net->clConfig->totalKernelGPUTime;
        if (net->clConfig->totalKernelGPUTime > net->clConfig->maxTotalKernelGPUTime)
            net->clConfig->maxTotalKernelGPUTime = net->clConfig->totalKernelGPUTime;
        net->clConfig->totalKernelGPUTime = 0;
    }
    if (net->config->profilingCPU) {
        dR_finish(net);
        g_print("CPU Profiling: Whole graph took: %2.3fms, Sum of all nodes: %2.3fms \n", wallMs() - t0, net->config->totalNodeCPUTime);
    }
    if (net->config->debugInfo) g_print("Done.\n\n");
    return TRUE;
}

/* reference src/deepRACIN.c:272-283 */
void dR_cleanup(dR_Graph *net, gboolean cleanupcl)
{
    if (!net->config->silent) g_print("Cleaning up deepRACIN...\n");
    if (net->prepared) { dR_finish(net); dR_cleanupBuffers(net); }
    if (cleanupcl) dR_cleanupCL(net);
    else if (!net->clConfig->ownsStream) dR_cleanupCL(net);     /* a borrowed stream is never destroyed here; only this graph's events go */
    dR_cleanupNet(net);
}

gboolean dR_saveGraph(dR_Graph *net, gchar *path) { return dR_serializeGraph(net, path); }

dR_Node *dR_loadGraph(dR_Graph *net, gchar *path, dR_Node ***nodelist, gint *numnodes, dR_Node ***feednodes, gint *numfeednodes)
{
    return dR_parseGraph(net, path, nodelist, numnodes, feednodes, numfeednodes);
}

void dR_printNetObject(dR_Graph *net, char *path) { dR_printNet(net, path); }

/* reference src/deepRACIN.c:309-319 */
void dR_setClEnvironment(dR_Graph *net, cl_context clcontext, cl_platform_id clplatformid,
                         cl_command_queue clcommandqueue, cl_device_id cldeviceid)
{
    net->clConfig->clCommandQueue = clcommandqueue;
    net->clConfig->clContext = clcontext;
    net->clConfig->clDeviceId = cldeviceid;
    net->clConfig->clDeviceNumber = (cl_uint)cldeviceid;
    net->clConfig->clPlatformId = clplatformid;
    net->clConfig->ownsStream = FALSE;
    dR_clInit(net);
}

void dR_getClEnvironmentFrom(dR_Graph *net, dR_Graph *from)
{
    dR_setClEnvironment(net, from->clConfig->clContext, from->clConfig->clPlatformId, from->clConfig->clCommandQueue,
                        from->clConfig->clDeviceId);
}

/* reference src/deepRACIN.c:321-335 */
void dR_config(dR_Graph *net, gchar *platformname, gboolean silent, gboolean debuginfo, gboolean profileGPU,
               gboolean profileCPU, gchar *temppath)
{
    net->clConfig->clPlatformName = platformname ? g_strdup(platformname) : NULL;
    net->config->silent = silent;
    net->config->debugInfo = debuginfo;
    net->config->profilingCPU = profileCPU;
    net->config->profilingGPU = profileGPU;
    net->config->modelPath = temppath ? g_strdup(temppath) : NULL;
}

dR_Shape3 *dR_getOutputShape(dR_Node *node) { return &node->oshape; }

dR_Shape3 *dR_getFeedNodeInputShape(dR_Node *node)
{
    if (node->type != tDataFeedNode) { g_print("Error: dR_getFeedNodeInputShape only works on feed nodes!\n"); return NULL; }
    return &((dR_DataFeedNode_Data *)node->layer)->shape;
}

/* ------------------------------------------------------------ b200 additions */
static gboolean beforePrepare(dR_Graph *net, const char *what)
{
    if (net->prepared) { g_print("%s must be called before dR_prepare\n", what); return FALSE; }
    return TRUE;
}

gboolean dR_setBatchSize(dR_Graph *net, gint n)
{
    if (!beforePrepare(net, "dR_setBatchSize")) return FALSE;
    if (n < 1) { g_print("dR_setBatchSize: batch must be >= 1\n"); return FALSE; }
    net->config->batchSize = n;
    return TRUE;
}

gboolean dR_setMathMode(dR_Graph *net, gint mode)
{
    if (!beforePrepare(net, "dR_setMathMode")) return FALSE;
    if (mode != DR_MATH_FP32 && mode != DR_MATH_TF32 && mode != DR_MATH_FP32_TENSOR) return FALSE;
    net->config->mathMode = mode;
    return TRUE;
}

gboolean dR_setInterfaceLayout(dR_Graph *net, gint layout)
{
    if (!beforePrepare(net, "dR_setInterfaceLayout")) return FALSE;
    if (layout != DR_LAYOUT_CHW && layout != DR_LAYOUT_HWC) return FALSE;
    net->config->interfaceLayout = layout;
    return TRUE;
}

gboolean dR_setConvAlgo(dR_Node *node, gint algo)
{
    if (!node || node->type != tConv2d || algo < DR_CONV_AUTO || algo >= DR_CONV_ALGOS) return FALSE;
    ((dR_Conv2d_Data *)node->layer)->algo = algo;
    return TRUE;
}

gboolean dR_setGraphConvAlgo(dR_Graph *net, gint algo)
{
    if (!beforePrepare(net, "dR_setGraphConvAlgo")) return FALSE;
    if (algo < DR_CONV_AUTO || algo >= DR_CONV_ALGOS) return FALSE;
    net->config->convAlgo = algo;
    return TRUE;
}

gboolean dR_setAutotune(dR_Graph *net, gboolean on) { if (!beforePrepare(net, "dR_setAutotune")) return FALSE; net->config->autotune = on; return TRUE; }
gboolean dR_setFusion(dR_Graph *net, gboolean on) { if (!beforePrepare(net, "dR_setFusion")) return FALSE; net->config->fuseGraph = on; return TRUE; }
gboolean dR_setFeedOverlap(dR_Graph *net, gboolean on) { if (!beforePrepare(net, "dR_setFeedOverlap")) return FALSE; net->config->feedOverlap = on; return TRUE; }
gboolean dR_setCudaGraph(dR_Graph *net, gboolean on) { if (!beforePrepare(net, "dR_setCudaGraph")) return FALSE; net->config->useCudaGraph = on; return TRUE; }

gboolean dR_setDevice(dR_Graph *net, gint ordinal)
{
    if (!beforePrepare(net, "dR_setDevice") || ordinal < 0) return FALSE;
    net->clConfig->clDeviceNumber = (cl_uint)ordinal;
    net->clConfig->clDeviceId = ordinal;
    return TRUE;
}

gboolean dR_synchronize(dR_Graph *net) { return dR_finish(net); }

gdouble dR_applyTimed(dR_Graph *net, gint iterations)
{
    if (!net->prepared || iterations < 1) return -1.0;
    gboolean prof = net->config->profilingGPU;
    net->config->profilingGPU = FALSE;      /* the per-kernel event pair would serialise the stream */
    dR_timerStart(net);
    for (gint i = 0; i < iterations; i++)
        if (!dR_apply(net)) { net->config->profilingGPU = prof; return -1.0; }
    gdouble ms = dR_timerStopMs(net);
    net->config->profilingGPU = prof;
    return ms;
}

gint dR_getConvAlgo(dR_Node *node) { return node && node->type == tConv2d ? ((dR_Conv2d_Data *)node->layer)->chosenAlgo : -1; }
gint dR_getConvTensor(dR_Node *node) { return node && node->type == tConv2d ? ((dR_Conv2d_Data *)node->layer)->chosenTensor : -1; }
gdouble dR_getNodeGpuMs(dR_Node *node) { return node ? node->lastGpuMs : 0.0; }

gint dR_getLaunchCount(dR_Graph *net)
{
    if (!net->prepared) return 0;
    gboolean cg = net->config->useCudaGraph;
    net->config->useCudaGraph = FALSE;
    dRk_launch_count_reset();
    dR_apply(net);
    dR_finish(net);
    net->config->useCudaGraph = cg;
    return (gint)dRk_launch_count();
}

gboolean dR_feedDataAsync(dR_Graph *net, dR_Node *feednode, gfloat *pinned, size_t numfloats)
{
    if (!net->prepared || !feednode || feednode->type != tDataFeedNode) return FALSE;
    if (net->config->feedOverlap && ((dR_DataFeedNode_Data *)feednode->layer)->evReady[0])
        return dR_feedOverlapCopy(net, feednode, pinned, numfloats * sizeof(cl_float));
    return dR_uploadArrayAsync(net, pinned, numfloats * sizeof(cl_float), *feednode->outputBuf->bufptr);
}

gboolean dR_feedDataU8Async(dR_Graph *net, dR_Node *feednode, const unsigned char *pinned, size_t numbytes)
{
    if (!net->prepared || net->config->dryRun || !feednode || feednode->type != tDataFeedNode || !pinned) return FALSE;
    if (numbytes != (size_t)feednode->outputBuf->size * net->config->batchSize) {
        g_print("dR_feedDataU8Async: %zu bytes given, the feed node holds %zu samples\n", numbytes, (size_t)feednode->outputBuf->size * net->config->batchSize);
        return FALSE;
    }
    return dR_feedU8(net, feednode, pinned, numbytes);
}

gboolean dR_fetchOutputAsync(dR_Graph *net, gint outputIndex, gfloat *pinned, size_t numfloats)
{
    if (!net->prepared) return FALSE;
    dR_ListElement *e = net->output_layers->first;
    while (e && outputIndex-- > 0) e = e->next;
    if (!e) return FALSE;
    return dR_downloadArrayAsync(net, *((dR_Node *)e->element)->outputBuf->bufptr, numfloats * sizeof(cl_float), pinned);
}

void *dR_allocPinned(size_t bytes) { return dR_hostAllocPinned(bytes); }
void dR_freePinned(void *p) { dR_hostFreePinned(p); }

gboolean dR_setDryRun(dR_Graph *net, gboolean on) { if (!beforePrepare(net, "dR_setDryRun")) return FALSE; net->config->dryRun = on; return TRUE; }
gint dR_getScheduleLength(dR_Graph *net) { return net->prepared ? net->scheduledLayers->length : 0; }
gint dR_getScheduledNodeId(dR_Graph *net, gint position)
{
    if (!net->prepared) return -1;
    dR_ListElement *e = net->scheduledLayers->first;
    while (e && position-- > 0) e = e->next;
    return e ? ((dR_Node *)e->element)->layerID : -1;
}
size_t dR_getNodeActAddress(dR_Node *node) { return (size_t)(uintptr_t)dR_actPtr(node); }
gint dR_getNodeActFloats(dR_Node *node) { return node && node->act ? node->act->size : 0; }
gint dR_getNodeChannelStride(dR_Node *node) { return node ? node->act_cstride : 0; }
gint dR_getNodeChannelOffset(dR_Node *node) { return node ? node->act_coffset : 0; }
gint dR_getStreamBufferCount(dR_Graph *net) { return net->prepared ? net->streamBufferHandlers->length : 0; }
size_t dR_getScratchFloats(dR_Graph *net) { return net->scratchFloats; }
