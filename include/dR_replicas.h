/*
 * Batch-sharded replicas behind the C API: N copies of one prepared graph, one per CUDA device, each fed a contiguous
 * image-major slice of the global batch by its own host thread; outputs land in one host array in global image order.
 * Images are independent on this path (the reference itself processes one image per dR_apply and runs on one device,
 * examples/vgg16/vgg_deployed.c:141-166), so there is no exchange step between the replicas and no collective: scatter and
 * gather are host copies.  No counterpart in the reference.
 *
 * Threading: the calling thread only hands out work; everything that touches a replica's graph (build, dR_prepare, feeds,
 * dR_apply, fetches, cleanup) runs on that replica's worker thread, which binds the replica's device once.  One
 * dR_Replicas object is used by one caller thread at a time.
 */
#ifndef DR_REPLICAS_H
#define DR_REPLICAS_H
#include "deepRACIN.h"
#ifdef __cplusplus
extern "C" {
#endif
typedef struct dR_Replicas dR_Replicas;

/* Builds one replica's graph on `net` (fresh from dR_NewGraph; device and batch size already set): create or load the nodes,
 * set math mode / interface layout / fusion options, and return the one feed node and the one output node.  Called once
 * per replica on that replica's thread.  Return FALSE to abort the creation. */
typedef gboolean (*dR_ReplicaBuilder)(dR_Graph *net, gint replica, void *user, dR_Node **feed, dR_Node **output);

/* ordinals[i] = CUDA device of replica i (a device may appear more than once).  batchPerReplica images per dR_apply and
 * replica.  dryRun: plan every replica without touching a device (dR_setDryRun); such replicas cannot apply.  NULL on failure. */
dR_Replicas *dR_replicasCreate(gint numReplicas, const gint *ordinals, gint batchPerReplica, dR_ReplicaBuilder build, void *user, gboolean dryRun);
/* The same for a saved model folder (dR_loadGraph): last node = output.  mathMode: dR_MathMode, layout: dR_InterfaceLayout. */
dR_Replicas *dR_replicasLoad(gint numReplicas, const gint *ordinals, gint batchPerReplica, const gchar *modelFolder, gint mathMode, gint layout);

gint dR_replicasCount(dR_Replicas *r);
gint dR_replicasGlobalBatch(dR_Replicas *r);
size_t dR_replicasInputFloatsPerImage(dR_Replicas *r);
size_t dR_replicasOutputFloatsPerImage(dR_Replicas *r);
dR_Graph *dR_replicasGraph(dR_Replicas *r, gint replica);
/* Images [lo, hi) of the global batch belong to `replica`. */
void dR_replicasShard(dR_Replicas *r, gint replica, gint *lo, gint *hi);

/* One step over the global batch: replica i copies images [i*b, (i+1)*b) of hostIn to its device, applies its graph and
 * copies its outputs to the same rows of hostOut; returns when every replica has finished.  hostIn / hostOut hold
 * globalBatch * floatsPerImage floats in the graphs' interface layout; pinned memory (dR_allocPinned) lets the copies of
 * the replicas overlap.  `steps` repetitions are issued back to back per replica (steps > 1: for timing; the same input).
 * msMax, if given, receives the largest per-replica device time of the call in milliseconds (events on each replica's stream). */
gboolean dR_replicasApply(dR_Replicas *r, const gfloat *hostIn, gfloat *hostOut, gint steps, gdouble *msMax);

void dR_replicasDestroy(dR_Replicas *r);
#ifdef __cplusplus
}
#endif
#endif
