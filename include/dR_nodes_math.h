/*
 * Element-wise and softmax nodes (reference include/dR_nodes_math.h, src/dR_nodes_math.c,
 * Kernels/dR_math.cl).  Softmax normalises over the whole per-image tensor.
 */
#ifndef DR_LAYERS_MATH_H
#define DR_LAYERS_MATH_H
#include "dR_types.h"

enum dR_ElemWise2OperationType { tAdd, tSub, tMul, tDiv, tPow };
typedef enum dR_ElemWise2OperationType dR_ElemWise2OperationType;
typedef struct dR_ElemWise2Op_Data dR_ElemWise2Op_Data;
struct dR_ElemWise2Op_Data { dR_Shape3 ishape; dR_ElemWise2OperationType op; };

enum dR_ElemWise1OperationType { tAddS, tSubS, tMulS, tDivS, tLog, tExp, tSqrt, tFill, tPowS };
typedef enum dR_ElemWise1OperationType dR_ElemWise1OperationType;
typedef struct dR_ElemWise1Op_Data dR_ElemWise1Op_Data;
struct dR_ElemWise1Op_Data { dR_Shape3 ishape; dR_ElemWise1OperationType op; gfloat scalar; };

typedef struct dR_Softmax_Data dR_Softmax_Data;
struct dR_Softmax_Data { dR_Shape3 ishape; cl_kernel clKernelComputeExp; gfloat *expsHost; };

#ifdef __cplusplus
extern "C" {
#endif
dR_Node *dR_ElemWise2Operation(dR_Graph *net, dR_Node *inputNode1, dR_Node *inputNode2, dR_ElemWise2OperationType op);
dR_Node *dR_ElemWise1Operation(dR_Graph *net, dR_Node *inputNode, dR_ElemWise1OperationType op, gfloat scalar);
dR_Node *dR_Softmax(dR_Graph *net, dR_Node *inputLayer);
#ifdef __cplusplus
}
#endif

#define DR_DECL_NODE_SLOTS(p)                                                                                  \
    gboolean p##_compute(dR_Graph *net, dR_Node *layer);                                                       \
    gboolean p##_schedule(dR_Graph *net, dR_Node *layer);                                                      \
    gboolean p##_propagateShape(dR_Graph *net, dR_Node *layer);                                                \
    gint32 p##_getRequiredOutputBufferSize(dR_Node *layer);                                                    \
    gboolean p##_createKernel(dR_Graph *net, dR_Node *layer);                                                  \
    gboolean p##_allocateBuffers(dR_Graph *net, dR_Node *layer);                                               \
    gboolean p##_fillBuffers(dR_Graph *net, dR_Node *layer);                                                   \
    gboolean p##_cleanupBuffers(dR_Graph *net, dR_Node *layer);                                                \
    gboolean p##_cleanupLayer(dR_Graph *net, dR_Node *layer);                                                  \
    gchar *p##_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],            \
                             gint variableSizes[], gint *numVariables);                                        \
    dR_Node *p##_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params,              \
                                 gint numParams, gfloat **variables, gint numVariables);                       \
    gchar *p##_printLayer(dR_Node *layer);

DR_DECL_NODE_SLOTS(dR_elemwise2op)
DR_DECL_NODE_SLOTS(dR_elemwise1op)
DR_DECL_NODE_SLOTS(dR_softmax)
#endif
