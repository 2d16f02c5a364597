/*
 * Graph core: node registration, scheduling (topological order + shape propagation),
 * liveness-based activation-buffer planning, variant selection and weight upload
 * (reference include/dR_core.h, src/dR_core.c).
 */
#ifndef DR_CORE_H
#define DR_CORE_H
#include "dR_clwrap.h"
#include "dR_base.h"
#ifdef __cplusplus
extern "C" {
#endif
/* reference include/dR_core.h:39 */
dR_Node *dR_Datafeednode(dR_Graph *graph, dR_Shape3 *shape);
#ifdef __cplusplus
}
#endif

dR_Graph *dR_appendLayer(dR_Graph *net, dR_Node *l);
/* allocates a node with empty neighbour lists and the b200 fields cleared */
dR_Node *dR_newNode(dR_LayerType type, void *data);
/* links `l` behind `input` (appends to both neighbour lists) */
void dR_linkNodes(dR_Node *input, dR_Node *l);
dR_Node *dR_firstInput(dR_Node *l);
dR_Node *dR_nthInput(dR_Node *l, gint n);
/* device pointer of a node's activations (internal N-HWC layout) */
float *dR_actPtr(dR_Node *l);

gboolean dR_generateAndCompileKernels(dR_Graph *net);   /* here: select (and autotune) kernel variants */
gboolean dR_propagateShapesAndSchedule(dR_Graph *net);
gboolean dR_estimateAndAllocateBuffers(dR_Graph *net);
gboolean dR_fillBuffers(dR_Graph *net);
gboolean dR_planFusion(dR_Graph *net);
/* TRUE if every input of this channel-wise Concat is a Slice -> scalar-op chain that one gather kernel can evaluate */
gboolean dR_concat_planGather(dR_Node *concat);
gint dR_concat_gatherSources(dR_Node *concat, dR_Node **srcs, gint maxSrcs);
gboolean dR_concat_gatherAsInputMap(dR_Node *concat, dR_Node **src, gint ch[4], gfloat scale[4], gfloat shift[4]);
void dR_cleanupBuffers(dR_Graph *net);
void dR_cleanupNet(dR_Graph *net);
dR_MemoryHandler *dR_newMemoryHandler(gboolean custom);
void dR_cleanupMemoryHandler(dR_Graph *net, dR_MemoryHandler *handler);

gchar *dR_datafeednode_serializeNode(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],
                                     gint variableSizes[], gint *numVariables);
dR_Node *dR_datafeednode_parseAppendNode(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params,
                                         gint numParams, gfloat **variables, gint numVariables);
gchar *dR_datafeednode_printLayer(dR_Node *layer);
gboolean dR_datafeednode_allocateBuffers(dR_Graph *net, dR_Node *layer);
gint32 dR_datafeednode_getRequiredOutputBufferSize(dR_Node *layer);
gboolean dR_datafeednode_cleanupLayer(dR_Graph *net, dR_Node *layer);
gboolean dR_datafeednode_compute(dR_Graph *net, dR_Node *layer);

/* intrusive list with an embedded iterator (reference src/dR_core.c:504-665) */
dR_List *dR_list_createEmptyList(void);
void dR_list_append(dR_List *list, void *elem);
gboolean dR_list_removeFirstOcc(dR_List *list, void *elem);
void *dR_list_pop(dR_List *list);
void *dR_list_next(dR_List *list);
void dR_list_resetIt(dR_List *list);
void dR_list_cleanup(dR_List *list);

gchar *concat_and_free_old(gchar *string1, gchar *string2);
/* naive row-major matmuls used by host-side weight transforms (reference src/dR_core.c:677-723):
 * result = mat1 * mat2, and result = mat1 * mat2^T */
gboolean dR_matmul(gfloat *mat1, int mat1rows, int mat1cols, gfloat *mat2, int mat2rows, int mat2cols, gfloat *result);
gboolean dR_matmulT(gfloat *mat1, int mat1rows, int mat1cols, gfloat *mat2, int mat2rows, int mat2cols, gfloat *result);
#endif
