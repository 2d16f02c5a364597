/*
 * Slice / Concat / CropOrPad nodes (reference include/dR_nodes_transform.h,
 * src/dR_nodes_transform.c, Kernels/dR_transform.cl).  Coordinates are (x, y, z, .).
 */
#ifndef DR_LAYERS_TRANSFORM_H
#define DR_LAYERS_TRANSFORM_H
#include "dR_types.h"
#include "dR_nodes_math.h"

typedef struct dR_Slice_Data dR_Slice_Data;
struct dR_Slice_Data { dR_Shape3 ishape; dR_Shape4 origin; dR_Shape4 oshape; };

typedef struct dR_Concat_Data dR_Concat_Data;
struct dR_Concat_Data {
    gint n; gint concatDim;
    gint inputSizesInConcatDim[3];
    gint maxInputSizeInConcatDim;
    gboolean elidedCopy;        /* producers write straight into this node's buffer */
    gboolean fusedGather;       /* inputs are Slice -> scalar-op chains: one gather kernel evaluates them all */
};

typedef struct dR_CropOrPad_Data dR_CropOrPad_Data;
struct dR_CropOrPad_Data { dR_Shape3 ishape; dR_Shape3 oshape; };

#ifdef __cplusplus
extern "C" {
#endif
/* reference src/dR_nodes_transform.c:8 */
dR_Node *dR_Slice(dR_Graph *net, dR_Node *inputLayer, dR_Shape4 *origin, dR_Shape4 *shape);
/* reference src/dR_nodes_transform.c:238 -- n in 1..3, concatDim 0=x 1=y 2=z */
dR_Node *dR_Concat(dR_Graph *net, dR_Node **inputNodes, gint n, gint concatDim);
/* reference src/dR_nodes_transform.c:576 */
dR_Node *dR_CropOrPad(dR_Graph *net, dR_Node *inputLayer, dR_Shape3 *targetshape);
#ifdef __cplusplus
}
#endif
DR_DECL_NODE_SLOTS(dR_slice)
DR_DECL_NODE_SLOTS(dR_concat)
DR_DECL_NODE_SLOTS(dR_croporpad)
#endif
