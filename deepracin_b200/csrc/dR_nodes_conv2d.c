/*
 * Conv2d node of the CUDA build.  One node type with four kernel families
 * (dR_ConvAlgo) instead of the reference's three sets of function slots
 * (src/dR_nodes_conv2d.c:36-81): the constructor, shape rule, serialisation and
 * setVariables keep the reference's behaviour; schedule/createKernel pick a family, the
 * weights are re-packed on the host for that family (the reference does the same for its
 * Winograd and 1x1 paths, :1162-1240 and :1696-1716) and compute launches it.
 */
#include "dR_nodes_conv2d.h"
#include "dR_b200.h"
#include "dR_core.h"
#include "dR_kernels.h"
#include "dR_nodes_pooling.h"

typedef struct {
    cl_mem wbuf[DR_CONV_ALGOS];     /* packed weights per dR_ConvAlgo */
    dRk_TensorWinogradPlan *wplan;  /* tensor-core Winograd: the batched GEMM's TMA descriptors for this layer's buffers */
    const float *wplanSrc;
    float *wplanDst, *wplanScratch;
    dRk_TensorConvPlan *plan;       /* tensor path: TMA descriptors for this layer's buffers */
    gint fusedPool;                 /* 1 / 2: the following 2x2/2 max / average pooling is evaluated in this node's epilogue */
    dR_Node *mapSrc;                /* few-channel first layer: the Slice/scalar-op/Concat preamble in front of it is evaluated by its gather; */
    gint mapCh[4];                  /* the convolution then reads this node's tensor through an affine channel map */
    gfloat mapScale[4], mapShift[4];
    const float *planSrc;           /* buffers the plan's tensor maps were encoded for */
    float *planDst;
    dR_Node *mergeWith;             /* Fire-module expand pair: this 3x3 node also evaluates that 1x1 sibling (same input, neighbouring channels of one Concat) */
    cl_mem mergedBias;              /* the sibling's bias followed by this node's */
    dRk_TensorConvPlan *planAlt;    /* the plan for the other buffer pair when the input alternates (double-buffered feeding) */
    const float *planAltSrc;
    float *planAltDst;
} dR_ConvDevice;

static dR_ConvDevice *dev(dR_Conv2d_Data *c) { return (dR_ConvDevice *)c->tmaDescs; }

/* reference src/dR_nodes_conv2d.c:12-97 */
dR_Node *dR_Conv2d(dR_Graph *net, dR_Node *inputLayer, dR_Shape4 *sh, dR_Shape4 *st, dR_ActivationType acttype, gboolean useB)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)calloc(1, sizeof(dR_Conv2d_Data));
    c->shape = *sh;
    c->stride = *st;
    c->activation = acttype;
    c->useBias = useB;
    c->algo = DR_CONV_AUTO;
    c->tmaDescs = calloc(1, sizeof(dR_ConvDevice));
    dR_Node *l = dR_newNode(tConv2d, c);
    l->compute = dR_conv2d_compute;
    l->schedule = dR_conv2d_schedule;
    l->propagateShape = dR_conv2d_propagateShape;
    l->getRequiredOutputBufferSize = dR_conv2d_getRequiredOutputBufferSize;
    l->createKernel = dR_conv2d_createKernel;
    l->allocateBuffers = dR_conv2d_allocateBuffers;
    l->fillBuffers = dR_conv2d_fillBuffers;
    l->cleanupBuffers = dR_conv2d_cleanupBuffers;
    l->cleanupLayer = dR_conv2d_cleanupLayer;
    l->printLayer = dR_conv2d_printLayer;
    l->setVariables = dR_Conv2d_setVariables;
    l->serializeNode = dR_conv2d_serializeNode;
    l->parseAppendNode = dR_conv2d_parseAppendNode;
    if (inputLayer) dR_linkNodes(inputLayer, l);
    else g_print("Error: Conv2d needs an appropriate Inputnode\n");
    dR_appendLayer(net, l);
    return l;
}

/* reference src/dR_nodes_conv2d.c:100-125: out = (W/sx, H/sy, Cout), integer division */
gboolean dR_conv2d_propagateShape(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    if (layer->previous_layers->length != 1) {
        if (!net->config->silent) g_print("Conv2d Layer with id %d has %d inputs but needs 1!\n", layer->layerID, layer->previous_layers->length);
        return FALSE;
    }
    c->ishape = dR_firstInput(layer)->oshape;
    if (c->stride.s1 <= 0 || c->stride.s2 <= 0 || c->shape.s0 <= 0 || c->shape.s1 <= 0) { g_print("Conv2d: filter size and stride must be positive\n"); return FALSE; }
    if (c->ishape.s2 != c->shape.s2) {
        g_print("Conv2d Layer %d: filter expects %d input channels but the input has %d\n", layer->layerID, c->shape.s2, c->ishape.s2);
        return FALSE;
    }
    layer->oshape.s0 = c->ishape.s0 / c->stride.s1;
    layer->oshape.s1 = c->ishape.s1 / c->stride.s2;
    layer->oshape.s2 = c->shape.s3;
    if (layer->oshape.s0 <= 0 || layer->oshape.s1 <= 0 || layer->oshape.s2 <= 0) {
        g_print("Conv2d shape propagates to Zero. False shape parameters! \n");
        return FALSE;
    }
    return TRUE;
}

gint32 dR_conv2d_getRequiredOutputBufferSize(dR_Node *layer) { return layer->oshape.s0 * layer->oshape.s1 * layer->oshape.s2; }

/* reference src/dR_nodes_conv2d.c:133-173 */
gchar *dR_conv2d_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[], gint variableSizes[], gint *numVariables)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    gint nv = c->useBias ? 2 : 1;
    if (*numParams < 10 || *numVariables < nv) { g_print("SerializeNode needs space for 10 parameters and %d variables!\n", nv); return NULL; }
    if (!c->hasVariables) { g_print("Conv2d node %d has no weights to serialize\n", layer->layerID); return NULL; }
    *numParams = 10;
    params[0] = g_strdup_printf("%d", c->activation);
    params[1] = g_strdup_printf("%d", c->useBias ? 1 : 0);
    params[2] = g_strdup_printf("%d", c->shape.s0);
    params[3] = g_strdup_printf("%d", c->shape.s1);
    params[4] = g_strdup_printf("%d", c->shape.s2);
    params[5] = g_strdup_printf("%d", c->shape.s3);
    params[6] = g_strdup_printf("%d", c->stride.s0);
    params[7] = g_strdup_printf("%d", c->stride.s1);
    params[8] = g_strdup_printf("%d", c->stride.s2);
    params[9] = g_strdup_printf("%d", c->stride.s3);
    *numVariables = nv;
    variableSizes[0] = c->shape.s0 * c->shape.s1 * c->shape.s2 * c->shape.s3;
    variables[0] = c->weights;
    if (c->useBias) { variableSizes[1] = c->shape.s3; variables[1] = c->biases; }
    return "Conv2D";
}

/* reference src/dR_nodes_conv2d.c:175-208 */
dR_Node *dR_conv2d_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params, gint numParams, gfloat **variables, gint numVariables)
{
    dR_Shape4 shape, stride;
    if (numINodes != 1) { g_print("Parsing Error: Conv2d Node needs 1 InputNodes but got %d!\n", numINodes); return NULL; }
    if (numParams != 10 || numVariables < 1 || numVariables > 2) { g_print("Parsing Error: Conv2d Node needs 10 Parameters and 1 or 2 Variables!\n"); return NULL; }
    gint useB = atoi(params[1]);
    if (useB && numVariables < 2) { g_print("Parsing Error: Conv2d Node with bias needs 2 Variables!\n"); return NULL; }
    shape.s0 = atoi(params[2]); shape.s1 = atoi(params[3]); shape.s2 = atoi(params[4]); shape.s3 = atoi(params[5]);
    stride.s0 = atoi(params[6]); stride.s1 = atoi(params[7]); stride.s2 = atoi(params[8]); stride.s3 = atoi(params[9]);
    dR_Node *out = dR_Conv2d(net, iNodes[0], &shape, &stride, (dR_ActivationType)atoi(params[0]), useB);
    dR_Conv2d_setVariables(out, variables[0], useB ? variables[1] : NULL);
    return out;
}

gchar *dR_conv2d_printLayer(dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    static const char *acts[] = {"Linear", "ReLU", "Sigmoid", "Tan"};
    static const char *algos[DR_CONV_ALGOS] = {"auto", "direct (FP32 implicit GEMM)", "Winograd F(2x2,3x3)", "1x1 GEMM", "tcgen05 TF32 implicit GEMM",
                                               "Winograd, tcgen05 products (F(2x2,3x3) TF32 / F(4x4,3x3) three-pass)", "Winograd F(4x4,3x3)"};
    return g_strdup_printf("Conv2d Layer: %d\n Filter dimensions: %dx%d\n Input channels: %d\n Output channels: %d\n Activation: %s\n"
                           " Stride: %d, %d, %d, %d\n Use bias: %s\n Kernel family: %s\n",
                           layer->layerID, c->shape.s0, c->shape.s1, c->shape.s2, c->shape.s3, acts[c->activation & 3],
                           c->stride.s0, c->stride.s1, c->stride.s2, c->stride.s3, c->useBias ? "Yes" : "No", algos[c->chosenAlgo % DR_CONV_ALGOS]);
}

/* reference src/dR_nodes_conv2d.c:238-256: the node keeps its own copies */
void dR_Conv2d_setVariables(dR_Node *layer, gfloat *weights, gfloat *biases)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    size_t n = (size_t)c->shape.s0 * c->shape.s1 * c->shape.s2 * c->shape.s3;
    g_free(c->weights);
    c->weights = (gfloat *)g_malloc(n * sizeof(gfloat));
    memcpy(c->weights, weights, n * sizeof(gfloat));
    if (c->useBias && biases) {
        g_free(c->biases);
        c->biases = (gfloat *)g_malloc((size_t)c->shape.s3 * sizeof(gfloat));
        memcpy(c->biases, biases, (size_t)c->shape.s3 * sizeof(gfloat));
    }
    c->hasVariables = TRUE;
}

/* --------------------------------------------------------------- variants */
static gboolean is3x3s1(dR_Conv2d_Data *c) { return c->shape.s0 == 3 && c->shape.s1 == 3 && c->stride.s1 == 1 && c->stride.s2 == 1; }
static gboolean is1x1s1(dR_Conv2d_Data *c) { return c->shape.s0 == 1 && c->shape.s1 == 1 && c->stride.s1 == 1 && c->stride.s2 == 1; }

/* the tensor path wants stride 1, odd square 1x1/3x3 filters and channel counts TMA can address */
static gboolean x3Mode(dR_Graph *net) { return net->config->mathMode == DR_MATH_FP32_TENSOR; }

static gboolean tensorLegal(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    dR_Node *in = dR_firstInput(layer);
    if (!(is3x3s1(c) || is1x1s1(c))) return FALSE;
    if (x3Mode(net)) {      /* the FP32-accurate three-pass tensor kernel exists for 3x3 layers only */
        if (!is3x3s1(c) || !dRk_tensor_conv_x3_supported(c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3)) return FALSE;
    } else if (!dRk_tensor_conv_supported(c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3, c->shape.s0, c->shape.s1)) return FALSE;
    if (in->act_cstride != in->oshape.s2) return FALSE;     /* input must be dense N-HWC */
    return TRUE;
}

static gboolean algoLegal(dR_Graph *net, dR_Node *layer, gint algo)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    switch (algo) {
    case DR_CONV_DIRECT: return TRUE;
    case DR_CONV_WINOGRAD: return is3x3s1(c);
    case DR_CONV_WINOGRAD4: return is3x3s1(c);
    case DR_CONV_ONEBYONE: return is1x1s1(c);
    case DR_CONV_TENSOR: return tensorLegal(net, layer);
    case DR_CONV_TENSOR_WINOGRAD:
        if (x3Mode(net))        /* FP32-accurate mode: F(4x4,3x3) with three-pass products */
            return is3x3s1(c) && dR_firstInput(layer)->act_cstride == dR_firstInput(layer)->oshape.s2 &&
                   dRk_tensor_winograd4_x3_supported(c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3);
        return is3x3s1(c) && tensorLegal(net, layer) && dRk_tensor_winograd_supported(c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3);
    }
    return FALSE;
}

/* The reference's static rule (src/dR_nodes_conv2d.c:36-81): 3x3 stride 1 -> Winograd,
 * 1x1 stride 1 -> 1x1 kernel, otherwise direct.  In TF32 mode dense layers go to the tensor cores.
 * Winograd layers with at least 16 channels on both sides take the F(4x4,3x3) form (fewer products AND fewer
 * transform-domain values per output than the reference's F(2x2,3x3); error about 1e-5 of max|ref|, inside the FP32
 * class bound); narrower layers keep F(2x2,3x3).  dR_setConvAlgo / dR_setGraphConvAlgo(DR_CONV_WINOGRAD) restores
 * the reference's transform everywhere. */
static gint staticRule(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    /* FP32-accurate tensor mode: Winograd F(4x4,3x3) with three-pass products (0.75 MMA per direct multiplication) beats the direct
       three-pass kernel (3 MMAs) where a tile's product outweighs moving its operands through memory, Cin*Cout against 2*Cin + Cout
       floats per tile and transform position: measured on the VGG-16 shapes at batch 64, 128->256 and deeper win (1.2-2.2x),
       128->128 and shallower lose */
    if (x3Mode(net) && (glong)c->shape.s2 * c->shape.s3 >= 56 * (2 * (glong)c->shape.s2 + c->shape.s3) &&
        algoLegal(net, layer, DR_CONV_TENSOR_WINOGRAD)) return DR_CONV_TENSOR_WINOGRAD;
    if (net->config->mathMode != DR_MATH_FP32 && tensorLegal(net, layer)) return DR_CONV_TENSOR;
    /* a handful of input channels (RGB first layer): bound by writing the output, a direct kernel wins */
    if (is3x3s1(c) && c->shape.s2 <= 4) return DR_CONV_DIRECT;
    if (is3x3s1(c)) return (c->shape.s2 >= 16 && c->shape.s3 >= 16) ? DR_CONV_WINOGRAD4 : DR_CONV_WINOGRAD;
    if (is1x1s1(c)) return DR_CONV_ONEBYONE;
    return DR_CONV_DIRECT;
}

gboolean dR_conv2d_schedule(dR_Graph *net, dR_Node *layer)
{
    (void)net; (void)layer;         /* launch shapes are derived inside the kernel launchers */
    return TRUE;
}

gboolean dR_conv2d_createKernel(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    gint want = c->algo != DR_CONV_AUTO ? c->algo : net->config->convAlgo;
    if (want != DR_CONV_AUTO && !algoLegal(net, layer, want)) {
        if (c->algo != DR_CONV_AUTO) { g_print("Conv2d Layer %d: requested kernel family %d cannot evaluate this filter/stride\n", layer->layerID, want); return FALSE; }
        want = DR_CONV_AUTO;    /* a graph-wide wish only applies where it is legal */
    }
    c->chosenAlgo = want != DR_CONV_AUTO ? want : staticRule(net, layer);
    c->chosenTensor = (c->chosenAlgo == DR_CONV_TENSOR || c->chosenAlgo == DR_CONV_TENSOR_WINOGRAD) ? (x3Mode(net) ? 2 : 1) : 0;
    /* conv -> 2x2/2 max pool with no other reader: the tensor kernel's epilogue (or the F(4x4,3x3) output transform) stores the
       pooled tensor directly into the pooling node's buffer and the pooling node launches nothing */
    dev(c)->fusedPool = 0;
    if ((c->chosenAlgo == DR_CONV_TENSOR || c->chosenAlgo == DR_CONV_WINOGRAD4 || (c->chosenAlgo == DR_CONV_TENSOR_WINOGRAD && x3Mode(net))) &&
        net->config->fuseGraph && is3x3s1(c) && !layer->output && !layer->elided && layer->next_layers->length == 1 &&
        layer->oshape.s0 % 2 == 0 && layer->oshape.s1 % 2 == 0) {
        dR_Node *nx = (dR_Node *)layer->next_layers->first->element;
        if (nx->type == tPooling && nx->previous_layers->length == 1) {
            dR_Pooling_Data *pl = (dR_Pooling_Data *)nx->layer;
            const gint ptype = pl->poolingType == tMax ? 1 : pl->poolingType == tAverage ? 2 : 0;
            if (ptype && pl->shape.s1 == 2 && pl->shape.s2 == 2 && pl->shape.s3 == 1 &&
                pl->stride.s1 == 2 && pl->stride.s2 == 2 && pl->stride.s3 == 1 &&
                (c->chosenAlgo == DR_CONV_WINOGRAD4 || x3Mode(net)     /* the F(4x4,3x3) output transform and the three-pass kernel: max only */
                     ? ptype == 1
                     : dRk_tensor_conv_can_fuse_pool(c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3, c->shape.s0, c->shape.s1, ptype))) {
                dev(c)->fusedPool = ptype;
                pl->useLMEM = TRUE;                 /* marks "computed by the producer" for dR_pooling_compute */
                layer->elided = TRUE;
                layer->act_cstride = layer->oshape.s2;
                layer->act_coffset = 0;
            }
        }
    }
    /* Slice -> scalar op -> Concat preamble in front of a few-channel tensor layer: read the source through a channel map */
    dev(c)->mapSrc = NULL;
    {
        dR_Node *in = dR_firstInput(layer);
        dR_Node *src = NULL;
        if (c->chosenAlgo == DR_CONV_TENSOR && !x3Mode(net) && net->config->fuseGraph && !dRk_debug_switches()->no_input_map && is3x3s1(c) && c->shape.s2 <= 4 && in->type == tConcat && !in->output &&
            in->next_layers->length == 1 && dR_concat_gatherAsInputMap(in, &src, dev(c)->mapCh, dev(c)->mapScale, dev(c)->mapShift) &&
            src->type == tDataFeedNode /* feed buffers are never recycled by the buffer planner, so the source outlives the skipped nodes */) {
            guint seen = 0;                             /* the kernel wants a permutation of the source's first Cin channels */
            for (gint j = 0; j < c->shape.s2; j++)
                if (dev(c)->mapCh[j] < c->shape.s2) seen |= 1u << dev(c)->mapCh[j];
            if (seen == (1u << c->shape.s2) - 1u) {
                dev(c)->mapSrc = src;
                in->fusedAway = TRUE;
            }
        }
    }
    /* Fire-module expand pair (SqueezeNet: 1x1 and 3x3 convolutions of the same squeezed tensor, concatenated along channels,
       examples/squeezenet-v1.1/squeezenet_whole/graph.dr): a 1x1 filter is a 3x3 filter whose eight outer taps are zero, so both are
       ONE 3x3 layer with O1 + O3 output channels written at the 1x1 node's channel offset.  On the transposed kernel the extra
       channels fill MMA rows that a 64-channel layer leaves idle anyway, and the graph launches one kernel less per module. */
    dev(c)->mergeWith = NULL;
    if (c->chosenAlgo == DR_CONV_TENSOR && !x3Mode(net) && net->config->fuseGraph && !net->config->autotune && is3x3s1(c) && layer->elided &&
        !dev(c)->fusedPool && c->algo == DR_CONV_AUTO && net->config->convAlgo == DR_CONV_AUTO && !layer->output) {
        dR_Node *in = dR_firstInput(layer);
        dR_Node *cat = (dR_Node *)layer->next_layers->first->element;
        for (dR_ListElement *e = in->next_layers->first; e; e = e->next) {
            dR_Node *sib = (dR_Node *)e->element;
            if (sib == layer || sib->type != tConv2d) continue;
            dR_Conv2d_Data *sc = (dR_Conv2d_Data *)sib->layer;
            if (!is1x1s1(sc) || sc->chosenAlgo != DR_CONV_TENSOR || sc->algo != DR_CONV_AUTO || !sib->elided || sib->output || sib->fusedAway) continue;
            if (sib->next_layers->length != 1 || sib->next_layers->first->element != cat || cat->type != tConcat) continue;
            if (sc->activation != c->activation || sc->useBias != c->useBias || sc->shape.s2 != c->shape.s2) continue;
            if (sib->act_cstride != layer->act_cstride || sib->act_coffset + sc->shape.s3 != layer->act_coffset) continue;
            if (!dRk_tensor_conv_supported(c->ishape.s0, c->ishape.s1, c->shape.s2, sc->shape.s3 + c->shape.s3, 3, 3)) continue;
            dev(c)->mergeWith = sib;
            sib->fusedAway = TRUE;
            break;
        }
    }
    /* scratch for every variant the autotuner may try */
    layer->scratchFloats = 0;
    if (c->chosenAlgo == DR_CONV_WINOGRAD || (net->config->autotune && is3x3s1(c)))
        layer->scratchFloats = dRk_winograd_scratch_floats(net->config->batchSize, c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3);
    if (c->chosenAlgo == DR_CONV_WINOGRAD4 || (net->config->autotune && is3x3s1(c))) {
        const size_t s = dRk_winograd4_scratch_floats(net->config->batchSize, c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3);
        if (s > layer->scratchFloats) layer->scratchFloats = s;
    }
    if (c->chosenAlgo == DR_CONV_TENSOR_WINOGRAD ||
        (net->config->autotune && net->config->mathMode != DR_MATH_FP32 && algoLegal(net, layer, DR_CONV_TENSOR_WINOGRAD))) {
        const size_t s = x3Mode(net) ? dRk_tensor_winograd4_x3_scratch_floats(net->config->batchSize, c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3)
                                     : dRk_tensor_winograd_scratch_floats(net->config->batchSize, c->ishape.s0, c->ishape.s1, c->shape.s2, c->shape.s3);
        if (s > layer->scratchFloats) layer->scratchFloats = s;
    }
    return TRUE;
}

gboolean dR_conv2d_allocateBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    if (!c->hasVariables) { g_print("Conv2d Layer %d has no weights (call dR_Conv2d_setVariables)\n", layer->layerID); return FALSE; }
    if (c->useBias) return dR_createFloatBuffer(net, &c->biasBuf, c->shape.s3, CL_MEM_READ_ONLY);
    return TRUE;
}

/* Host-side packing of [Cin][Cout][kh][kw] weights for one kernel family + upload. */
static gboolean ensurePacked(dR_Graph *net, dR_Node *layer, gint algo)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    dR_ConvDevice *d = dev(c);
    const gint kw = c->shape.s0, kh = c->shape.s1, I = c->shape.s2, O = c->shape.s3;
    if (algo == DR_CONV_ONEBYONE) algo = DR_CONV_DIRECT;        /* same [K][Cout] packing */
    if (d->wbuf[algo]) return TRUE;
    if (algo == DR_CONV_TENSOR && d->mergeWith) {
        /* [Cin][O1 + O][3][3]: the sibling's 1x1 filters on the centre tap of the first O1 channels, then this node's filters */
        dR_Conv2d_Data *sc = (dR_Conv2d_Data *)d->mergeWith->layer;
        const gint O1 = sc->shape.s3, Om = O1 + O;
        if (!sc->hasVariables) { g_print("Conv2d Layer %d has no weights (call dR_Conv2d_setVariables)\n", d->mergeWith->layerID); return FALSE; }
        const size_t nm = dRk_tensor_conv_packed_floats(c->ishape.s0, c->ishape.s1, I, Om, 3, 3);
        gfloat *wm = (gfloat *)g_malloc0((size_t)I * Om * 9 * sizeof(gfloat));
        gfloat *pm = nm ? (gfloat *)g_malloc0(nm * sizeof(gfloat)) : NULL;
        gboolean okm = pm != NULL;
        for (gint i = 0; i < I && okm; i++) {
            for (gint o = 0; o < O1; o++) wm[((size_t)i * Om + o) * 9 + 4] = sc->weights[(size_t)i * O1 + o];
            memcpy(wm + ((size_t)i * Om + O1) * 9, c->weights + (size_t)i * O * 9, (size_t)O * 9 * sizeof(gfloat));
        }
        okm = okm && dRk_tensor_conv_pack_weights(wm, pm, c->ishape.s0, c->ishape.s1, I, Om, 3, 3) == 0 &&
              dR_createFloatBufferL(net, &d->wbuf[algo], nm) && dR_uploadArray(net, "", pm, 0, nm * sizeof(gfloat), d->wbuf[algo]);
        g_free(wm); g_free(pm);
        return okm;
    }
    size_t n = (size_t)kw * kh * I * O;
    if (algo == DR_CONV_WINOGRAD) n = (size_t)16 * I * O;
    if (algo == DR_CONV_WINOGRAD4) n = (size_t)36 * I * O;
    if (algo == DR_CONV_TENSOR) n = x3Mode(net) ? dRk_tensor_conv_x3_packed_floats(c->ishape.s0, c->ishape.s1, I, O) : dRk_tensor_conv_packed_floats(c->ishape.s0, c->ishape.s1, I, O, kw, kh);
    if (algo == DR_CONV_TENSOR_WINOGRAD) n = x3Mode(net) ? dRk_tensor_winograd4_x3_packed_floats(I, O) : dRk_tensor_winograd_packed_floats(I, O);
    if (n == 0) return FALSE;
    gfloat *p = (gfloat *)g_malloc0(n * sizeof(gfloat));
    if (algo == DR_CONV_DIRECT) {
        /* [ (ky*kw+kx)*Cin + i ][ o ] */
        for (gint i = 0; i < I; i++)
            for (gint o = 0; o < O; o++)
                for (gint t = 0; t < kh * kw; t++)
                    p[((size_t)t * I + i) * O + o] = c->weights[((size_t)i * O + o) * kh * kw + t];
    } else if (algo == DR_CONV_TENSOR) {
        /* K-major rows per output channel; the exact layout belongs to the tensor kernel picked for this shape */
        if ((x3Mode(net) ? dRk_tensor_conv_x3_pack_weights(c->weights, p, c->ishape.s0, c->ishape.s1, I, O)
                         : dRk_tensor_conv_pack_weights(c->weights, p, c->ishape.s0, c->ishape.s1, I, O, kw, kh)) != 0) { g_free(p); return FALSE; }
    } else if (algo == DR_CONV_TENSOR_WINOGRAD) {
        if ((x3Mode(net) ? dRk_tensor_winograd4_x3_pack_weights(c->weights, p, I, O) : dRk_tensor_winograd_pack_weights(c->weights, p, I, O)) != 0) { g_free(p); return FALSE; }
    } else if (algo == DR_CONV_WINOGRAD4) {
        if (dRk_winograd4_pack_weights(c->weights, p, I, O) != 0) { g_free(p); return FALSE; }
    } else {
        /* U = G g G^T with G = [[1,0,0],[.5,.5,.5],[.5,-.5,.5],[0,0,1]] (reference :1162-1240),
           stored [16][Cin][Cout] so that each of the 16 positions is one K x N matrix */
        gfloat G[12] = {1.f, 0.f, 0.f, .5f, .5f, .5f, .5f, -.5f, .5f, 0.f, 0.f, 1.f};
        gfloat tmp[12], u[16];
        for (gint i = 0; i < I; i++)
            for (gint o = 0; o < O; o++) {
                dR_matmul(G, 4, 3, c->weights + ((size_t)i * O + o) * 9, 3, 3, tmp);
                dR_matmulT(tmp, 4, 3, G, 4, 3, u);
                for (gint k = 0; k < 16; k++) p[((size_t)k * I + i) * O + o] = u[k];
            }
    }
    gboolean ok = dR_createFloatBufferL(net, &d->wbuf[algo], n) && dR_uploadArray(net, "", p, 0, n * sizeof(gfloat), d->wbuf[algo]);
    g_free(p);
    return ok;
}

gboolean dR_conv2d_fillBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    if (c->useBias && !dR_uploadArray(net, "", c->biases, 0, (size_t)c->shape.s3 * sizeof(cl_float), c->biasBuf)) return FALSE;
    if (dev(c)->mergeWith && c->useBias) {
        dR_Conv2d_Data *sc = (dR_Conv2d_Data *)dev(c)->mergeWith->layer;
        const size_t o1 = (size_t)sc->shape.s3, o3 = (size_t)c->shape.s3;
        if (!dR_createFloatBufferL(net, &dev(c)->mergedBias, o1 + o3) ||
            !dR_uploadArray(net, "", sc->biases, 0, o1 * sizeof(cl_float), dev(c)->mergedBias) ||
            !dR_uploadArray(net, "", c->biases, o1 * sizeof(cl_float), o3 * sizeof(cl_float), dev(c)->mergedBias)) return FALSE;
    }
    if (!ensurePacked(net, layer, c->chosenAlgo)) return FALSE;
    c->weightsBuf = dev(c)->wbuf[c->chosenAlgo == DR_CONV_ONEBYONE ? DR_CONV_DIRECT : c->chosenAlgo];
    return TRUE;
}

gboolean dR_conv2d_runVariant(dR_Graph *net, dR_Node *layer, gint algo, gint tensor)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    dR_ConvDevice *d = dev(c);
    dR_Node *in = dR_firstInput(layer);
    const float *src = dR_actPtr(in) + in->act_coffset;
    if (algo == DR_CONV_TENSOR && d->mapSrc) src = dR_actPtr(d->mapSrc) + d->mapSrc->act_coffset;
    float *dst = dR_actPtr(layer);
    const float *bias = c->useBias ? (const float *)c->biasBuf : NULL;
    const gint n = net->config->batchSize, W = c->ishape.s0, H = c->ishape.s1;
    const gint act = c->activation == tReLU ? 1 : 0;
    dRk_stream s = net->clConfig->clCommandQueue;
    (void)tensor;
    if (!ensurePacked(net, layer, algo)) return FALSE;
    switch (algo) {
    case DR_CONV_DIRECT:
    case DR_CONV_ONEBYONE:
        net->clConfig->clError = dRk_conv2d_f32(s, src, (const float *)d->wbuf[DR_CONV_DIRECT], bias, dst, n, W, H, c->shape.s2, c->shape.s3,
                                                c->shape.s0, c->shape.s1, c->stride.s1, c->stride.s2, act, in->act_cstride,
                                                layer->act_cstride, layer->act_coffset);
        break;
    case DR_CONV_WINOGRAD:
        net->clConfig->clError = dRk_conv2d_winograd_f32(s, src, (const float *)d->wbuf[DR_CONV_WINOGRAD], bias, dst, (float *)net->scratch, n, W, H,
                                                         c->shape.s2, c->shape.s3, act, in->act_cstride, layer->act_cstride, layer->act_coffset);
        break;
    case DR_CONV_WINOGRAD4:
        net->clConfig->clError = dRk_conv2d_winograd4_f32(s, src, (const float *)d->wbuf[DR_CONV_WINOGRAD4], bias, dst, (float *)net->scratch, n, W, H,
                                                          c->shape.s2, c->shape.s3, act, in->act_cstride, layer->act_cstride, layer->act_coffset, d->fusedPool);
        break;
    case DR_CONV_TENSOR:
        if (d->plan && (d->planSrc != src || d->planDst != dst)) {
            /* buffers moved (alternating feed buffers, a caller's new feed buffer): keep this plan aside and take the one built
               for these buffers if there is one; a third pair replaces the older of the two */
            dRk_TensorConvPlan *tp = d->plan; const float *ts = d->planSrc; float *td = d->planDst;
            d->plan = d->planAlt; d->planSrc = d->planAltSrc; d->planDst = d->planAltDst;
            d->planAlt = tp; d->planAltSrc = ts; d->planAltDst = td;
            if (d->plan && (d->planSrc != src || d->planDst != dst)) { dRk_tensor_conv_free(d->plan); d->plan = NULL; }
        }
        if (!d->plan) {
            d->planSrc = src; d->planDst = dst;
            if (d->mergeWith) {
                dR_Conv2d_Data *sc = (dR_Conv2d_Data *)d->mergeWith->layer;
                d->plan = dRk_tensor_conv_plan(src, (const float *)d->wbuf[DR_CONV_TENSOR], c->useBias ? (const float *)d->mergedBias : NULL, dst, n, W, H,
                                               c->shape.s2, sc->shape.s3 + c->shape.s3, 3, 3, act, layer->act_cstride, d->mergeWith->act_coffset, 0,
                                               (int *)net->statusWord);
            } else
            d->plan = x3Mode(net)
                ? dRk_tensor_conv_x3_plan(src, (const float *)d->wbuf[DR_CONV_TENSOR], bias, dst, n, W, H, c->shape.s2, c->shape.s3, act,
                                          layer->act_cstride, layer->act_coffset, d->fusedPool, (int *)net->statusWord)
                : dRk_tensor_conv_plan(src, (const float *)d->wbuf[DR_CONV_TENSOR], bias, dst, n, W, H, c->shape.s2, c->shape.s3,
                                       c->shape.s0, c->shape.s1, act, layer->act_cstride, layer->act_coffset, d->fusedPool, (int *)net->statusWord);
            if (!d->plan) { g_print("Conv2d Layer %d: tensor-core plan could not be built\n", layer->layerID); return FALSE; }
            if (d->mapSrc && dRk_tensor_conv_set_input_map(d->plan, d->mapSrc->act_cstride, d->mapCh, d->mapScale, d->mapShift) != 0) {
                g_print("Conv2d Layer %d: input channel map rejected\n", layer->layerID);
                return FALSE;
            }
        }
        net->clConfig->clError = dRk_tensor_conv_run(s, d->plan);
        break;
    case DR_CONV_TENSOR_WINOGRAD:
        if (d->wplan && (d->wplanSrc != src || d->wplanDst != dst || d->wplanScratch != (float *)net->scratch)) { dRk_tensor_winograd_free(d->wplan); d->wplan = NULL; }
        if (!d->wplan) {
            d->wplanSrc = src; d->wplanDst = dst; d->wplanScratch = (float *)net->scratch;
            d->wplan = x3Mode(net)
                ? dRk_tensor_winograd4_x3_plan(src, (const float *)d->wbuf[DR_CONV_TENSOR_WINOGRAD], bias, dst, (float *)net->scratch, n, W, H,
                                               c->shape.s2, c->shape.s3, act, in->act_cstride, layer->act_cstride, layer->act_coffset, d->fusedPool,
                                               (int *)net->statusWord)
                : dRk_tensor_winograd_plan(src, (const float *)d->wbuf[DR_CONV_TENSOR_WINOGRAD], bias, dst, (float *)net->scratch, n, W, H,
                                           c->shape.s2, c->shape.s3, act, in->act_cstride, layer->act_cstride, layer->act_coffset, (int *)net->statusWord);
            if (!d->wplan) { g_print("Conv2d Layer %d: tensor-core Winograd plan could not be built\n", layer->layerID); return FALSE; }
        }
        net->clConfig->clError = dRk_tensor_winograd_run(s, d->wplan);
        break;
    default:
        return FALSE;
    }
    return TRUE;
}

gboolean dR_conv2d_compute(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    dR_beginCLKernel(net);
    if (!dR_conv2d_runVariant(net, layer, c->chosenAlgo, c->chosenTensor)) return FALSE;
    return dR_finishCLKernel(net, "deepRACIN:conv2d");
}

/*
 * Resource-aware variant choice from measured timings: every convolution runs each family
 * that can evaluate it (3 warm-up + 5 timed launches on the graph's stream, on the real
 * buffers) and keeps the fastest.  The reference's scheduler only sizes work-groups from
 * device limits (src/dR_nodes_conv2d.c:263-362, 809-1006, 1526-1603); it never times.
 * FP32 mode only considers FP32 families, so the choice cannot change the arithmetic class.
 */
gboolean dR_conv2d_autotune(dR_Graph *net)
{
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) {
        dR_Node *layer = (dR_Node *)e->element;
        if (layer->type != tConv2d) continue;
        dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
        if (c->algo != DR_CONV_AUTO || net->config->convAlgo != DR_CONV_AUTO) continue;
        if (dev(c)->fusedPool || dev(c)->mapSrc) continue;     /* only the tensor kernel can store the pooled tensor / read through the channel map */
        gint best = c->chosenAlgo;
        gdouble bestMs = 1e30;
        for (gint algo = DR_CONV_DIRECT; algo < DR_CONV_ALGOS; algo++) {
            if (!algoLegal(net, layer, algo)) continue;
            if ((algo == DR_CONV_TENSOR || algo == DR_CONV_TENSOR_WINOGRAD) && net->config->mathMode == DR_MATH_FP32) continue;
            if (algo == DR_CONV_ONEBYONE) continue;             /* same kernel as DIRECT for 1x1 */
            for (gint i = 0; i < 3; i++) if (!dR_conv2d_runVariant(net, layer, algo, 0)) return FALSE;
            dR_timerStart(net);
            for (gint i = 0; i < 5; i++) if (!dR_conv2d_runVariant(net, layer, algo, 0)) return FALSE;
            gdouble ms = dR_timerStopMs(net) / 5.0;
            if (net->clConfig->clError) { dR_openCLError(net, "autotune launch failed", "dR_conv2d_autotune"); return FALSE; }
            c->tunedMs[algo] = ms;
            if (!net->config->silent && net->config->debugInfo) g_print("Layer %d family %d: %.4f ms\n", layer->layerID, algo, ms);
            if (ms < bestMs) { bestMs = ms; best = algo; }
        }
        if (best == DR_CONV_DIRECT && is1x1s1(c)) best = DR_CONV_ONEBYONE;
        c->chosenAlgo = best;
        c->chosenTensor = (best == DR_CONV_TENSOR || best == DR_CONV_TENSOR_WINOGRAD) ? (x3Mode(net) ? 2 : 1) : 0;
        c->weightsBuf = dev(c)->wbuf[best == DR_CONV_ONEBYONE ? DR_CONV_DIRECT : best];
        /* drop the packings of the losers */
        for (gint a = 1; a < DR_CONV_ALGOS; a++) {
            if (dev(c)->wbuf[a] && dev(c)->wbuf[a] != c->weightsBuf) { dR_finish(net); dR_clMemoryBufferCleanup(net, dev(c)->wbuf[a]); dev(c)->wbuf[a] = NULL; }
        }
    }
    return TRUE;
}

gint dR_getConvTensorKernel(dR_Node *node, gint geom[4])
{
    geom[0] = geom[1] = geom[2] = geom[3] = 0;
    if (!node || node->type != tConv2d) return -1;
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)node->layer;
    if (!c->chosenTensor || !dev(c)) return 0;
    return dRk_tensor_conv_plan_describe(dev(c)->plan, &geom[0], &geom[1], &geom[2], &geom[3]);
}

gboolean dR_conv2d_cleanupBuffers(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    dR_ConvDevice *d = dev(c);
    gboolean ret = TRUE;
    for (gint a = 0; a < DR_CONV_ALGOS; a++) if (d->wbuf[a]) { ret &= dR_clMemoryBufferCleanup(net, d->wbuf[a]); d->wbuf[a] = NULL; }
    if (c->biasBuf) { ret &= dR_clMemoryBufferCleanup(net, c->biasBuf); c->biasBuf = NULL; }
    if (d->plan) { dRk_tensor_conv_free(d->plan); d->plan = NULL; }
    if (d->planAlt) { dRk_tensor_conv_free(d->planAlt); d->planAlt = NULL; }
    if (d->wplan) { dRk_tensor_winograd_free(d->wplan); d->wplan = NULL; }
    if (d->mergedBias) { ret &= dR_clMemoryBufferCleanup(net, d->mergedBias); d->mergedBias = NULL; }
    c->weightsBuf = NULL;
    return ret;
}

gboolean dR_conv2d_cleanupLayer(dR_Graph *net, dR_Node *layer)
{
    dR_Conv2d_Data *c = (dR_Conv2d_Data *)layer->layer;
    (void)net;
    g_free(c->weights);
    g_free(c->biases);
    g_free(c->tmaDescs);
    g_free(c);
    return TRUE;
}
