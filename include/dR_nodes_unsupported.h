/*
 * Constructors of node types outside the CNN-layer hot path.  The reference's Python
 * module resolves every one of these symbols when it is imported
 * (python/deepracin/__init__.py.in:125-213), so they are exported; each prints
 * "not supported in the CUDA build" and returns NULL without touching the graph.
 */
#ifndef DR_LAYERS_UNSUPPORTED_H
#define DR_LAYERS_UNSUPPORTED_H
#include "dR_types.h"
#ifdef __cplusplus
extern "C" {
#endif
dR_Node *dR_Conv2dTransposed(dR_Graph *net, dR_Node *inputnode, dR_Shape4 filtershape, dR_Shape4 stride,
                             dR_ActivationType activation, gboolean useBias);
void dR_Conv2dtransposed_setVariables(dR_Node *layer, gfloat *weights, gfloat *biases);
dR_Node *dR_BatchNormalization(dR_Graph *net, dR_Node *inputLayer);
dR_Node *dR_MaskDependentFilter(dR_Graph *net, dR_Node *inputImage, dR_Node *inputFilterMask, dR_Shape3 *shape);
void dR_MaskDependentFilter_setVariables(dR_Node *layer, gfloat *weights, gfloat *bias);
dR_Node *dR_PerPixelFilter(dR_Graph *net, dR_Node *inputImage, dR_Node *inputFilter, dR_Shape4 *shape, dR_Shape4 *stride);
dR_Node *dR_ResolveRoI(dR_Graph *net, dR_Node *inputNode, dR_Shape3 *shape);
dR_Node *dR_RGB2gray(dR_Graph *net, dR_Node *inputNode);
dR_Node *dR_Upscaling(dR_Graph *net, dR_Node *inputLayer, gint type, gint scaleFactorX, gint scaleFactorY);
dR_Node *dR_LabelCreation(dR_Graph *net, dR_Node *inputLayer, gint type, gfloat class0offset, gfloat class1offset, gfloat class2offset);
dR_Node *dR_Normalization(dR_Graph *net, dR_Node *inputLayer, gint type, gfloat targetMean, gfloat targetDev);
dR_Node *dR_FFT(dR_Graph *net, dR_Node *inputNode1);
#ifdef __cplusplus
}
#endif
#endif
