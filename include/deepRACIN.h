/*
 * Public C API of deepRacin, served by the CUDA (sm_100a) library.  Names, argument
 * meaning and return conventions follow the reference's include/deepRACIN.h (line
 * numbers cited per function); the OpenCL handle types are CUDA handles here (see
 * dR_types.h).  Buffers the API hands out or accepts (feed buffers, output buffers) hold
 * tensors "z major, x minor" ([C][H][W], include/deepRACIN.h:61), batchSize images back
 * to back; dR_setInterfaceLayout switches them to [H][W][C].
 */
#ifndef DR_H
#define DR_H
#include "dR_core.h"
#include "dR_b200.h"
#ifdef __cplusplus
extern "C" {
#endif
/* include/deepRACIN.h:18 */
dR_Graph *dR_NewGraph(void);
/* include/deepRACIN.h:32 -- fills outptr with pointers to the output nodes' buffer handles (max 10);
 * returns the count, 0 before dR_prepare. */
gint dR_getOutputBuffers(dR_Graph *graph, cl_mem **outptr);
/* include/deepRACIN.h:47 -- blocking upload of numfloats floats at float offset `offset`. */
void dR_feedData(dR_Graph *graph, dR_Node *feednode, gfloat *data, gint offset, gint numfloats);
/* include/deepRACIN.h:57 */
dR_Shape3 *dR_getFeedNodeInputShape(dR_Node *node);
/* include/deepRACIN.h:72 -- the feed node reads a caller-owned device buffer instead of its own. */
gboolean dR_setDataFeedNodeBuffer(dR_Graph *graph, dR_Node *feednode, cl_mem *clbuf);
/* include/deepRACIN.h:86,100 -- region-of-interest hooks; ResolveRoI is outside this build, kept as inert setters. */
gboolean dR_setNodeRoI(dR_Node *node, dR_Shape3 origin);
gboolean dR_setNodeRoIBufferAndIndex(dR_Node *node, cl_mem *buf, gint index);
/* include/deepRACIN.h:126 -- the node writes its (interface-layout) output into a caller-owned buffer. */
gboolean dR_setPreexistingOutputBuffer(dR_Graph *graph, dR_Node *node, cl_mem *buf);
/* include/deepRACIN.h:142 */
gboolean dR_setAsOutput(dR_Graph *graph, dR_Node *node);
/* include/deepRACIN.h:155 -- CUDA-context equivalent of the OpenCL initialisation.  Declared void in the
 * reference; returns TRUE/FALSE here because the reference's own Python module reads a bool from it
 * (python/deepracin/__init__.py.in:56-58). */
gboolean dR_initCL(dR_Graph *graph);
/* include/deepRACIN.h:169 -- launches every scheduled node on the stream; asynchronous. */
gboolean dR_apply(dR_Graph *graph);
/* include/deepRACIN.h:182 -- schedule, select kernel variants, allocate, upload weights. */
gboolean dR_prepare(dR_Graph *net);
/* include/deepRACIN.h:194 */
void dR_cleanup(dR_Graph *net, gboolean cleanupcl);
/* include/deepRACIN.h:213 -- writes <path>/dr_graph_export/{graph.dr, N.var}. */
gboolean dR_saveGraph(dR_Graph *net, gchar *path);
/* include/deepRACIN.h:216 -- fills an empty graph from <path>/graph.dr; the two arrays are malloc'ed, caller frees. */
dR_Node *dR_loadGraph(dR_Graph *net, gchar *path, dR_Node ***nodelist, gint *numnodes, dR_Node ***feednodes, gint *numfeednodes);
/* include/deepRACIN.h:227 */
void dR_printNetObject(dR_Graph *net, char *path);
/* include/deepRACIN.h:242 -- adopt a caller's stream (clcommandqueue = cudaStream_t) and device ordinal. */
void dR_setClEnvironment(dR_Graph *net, cl_context clcontext, cl_platform_id clplatformid,
                         cl_command_queue clcommandqueue, cl_device_id cldeviceid);
/* include/deepRACIN.h:262 */
void dR_config(dR_Graph *net, gchar *platformname, gboolean silent, gboolean debuginfo, gboolean profileGPU,
               gboolean profileCPU, gchar *temppath);
/* include/deepRACIN.h:279 */
dR_Shape3 *dR_getOutputShape(dR_Node *node);
/* python/deepracin/__init__.py.in binds this to share one environment between graphs. */
void dR_getClEnvironmentFrom(dR_Graph *net, dR_Graph *from);
#ifdef __cplusplus
}
#endif
#endif
