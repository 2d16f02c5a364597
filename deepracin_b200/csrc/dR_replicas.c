/*
 * Batch-sharded replicas: one graph per device, one worker thread per replica, host-side scatter and gather
 * (see include/dR_replicas.h).  The workers are created once and sleep on a condition variable between jobs.
 */
#include <pthread.h>
#include "dR_replicas.h"

enum { JOB_NONE = 0, JOB_BUILD, JOB_APPLY, JOB_QUIT };

typedef struct {
    dR_Replicas *owner;
    gint index, ordinal;
    pthread_t thread;
    dR_Graph *net;
    dR_Node *feed, *out;
    gboolean ok;
    gdouble ms;
    gint seen;                      /* generation of the last job this worker ran */
} dR_ReplicaWorker;

struct dR_Replicas {
    gint n, batch;
    gboolean dryRun;
    dR_ReplicaBuilder build;
    void *user;
    dR_ReplicaWorker *w;
    pthread_mutex_t lock;
    pthread_cond_t wake, done;
    gint generation, job, finished;
    const gfloat *jobIn;
    gfloat *jobOut;
    gint jobSteps;
    size_t inFloats, outFloats;     /* per image */
};

typedef struct {                    /* what dR_replicasLoad's builder needs */
    const gchar *folder;
    gint mathMode, layout;
} dR_FolderOptions;

static gboolean workerBuild(dR_ReplicaWorker *w)
{
    dR_Replicas *r = w->owner;
    w->net = dR_NewGraph();
    if (!w->net) return FALSE;
    if (r->dryRun && !dR_setDryRun(w->net, TRUE)) return FALSE;
    if (!dR_setDevice(w->net, w->ordinal) || !dR_setBatchSize(w->net, r->batch)) return FALSE;
    if (!dR_initCL(w->net)) return FALSE;                       /* binds the device to this thread */
    if (!r->build(w->net, w->index, r->user, &w->feed, &w->out) || !w->feed || !w->out) return FALSE;
    if (!dR_setAsOutput(w->net, w->out)) return FALSE;
    return dR_prepare(w->net);
}

static gboolean workerApply(dR_ReplicaWorker *w)
{
    dR_Replicas *r = w->owner;
    const size_t nin = r->inFloats * (size_t)r->batch, nout = r->outFloats * (size_t)r->batch;
    const gfloat *src = r->jobIn + (size_t)w->index * nin;
    gfloat *dst = r->jobOut + (size_t)w->index * nout;
    gboolean ok = TRUE;
    w->ms = 0.0;
    if (r->dryRun) return FALSE;
    dR_timerStart(w->net);
    for (gint s = 0; s < r->jobSteps && ok; s++)
        ok = dR_feedDataAsync(w->net, w->feed, (gfloat *)src, nin) && dR_apply(w->net) && dR_fetchOutputAsync(w->net, 0, dst, nout);
    w->ms = dR_timerStopMs(w->net);                             /* synchronises this replica's stream */
    return ok && w->ms >= 0.0 && dR_getDeviceStatus(w->net) == 0;
}

static void *workerMain(void *arg)
{
    dR_ReplicaWorker *w = (dR_ReplicaWorker *)arg;
    dR_Replicas *r = w->owner;
    for (;;) {
        pthread_mutex_lock(&r->lock);
        while (r->generation == w->seen) pthread_cond_wait(&r->wake, &r->lock);
        w->seen = r->generation;
        const gint job = r->job;
        pthread_mutex_unlock(&r->lock);
        if (job == JOB_BUILD) w->ok = workerBuild(w);
        else if (job == JOB_APPLY) w->ok = workerApply(w);
        else if (job == JOB_QUIT && w->net) { dR_cleanup(w->net, TRUE); w->net = NULL; }
        pthread_mutex_lock(&r->lock);
        if (++r->finished == r->n) pthread_cond_signal(&r->done);
        pthread_mutex_unlock(&r->lock);
        if (job == JOB_QUIT) return NULL;
    }
}

/* hands `job` to every worker and waits until all have finished it; TRUE if every worker reported success */
static gboolean runJob(dR_Replicas *r, gint job)
{
    pthread_mutex_lock(&r->lock);
    r->job = job;
    r->finished = 0;
    r->generation++;
    pthread_cond_broadcast(&r->wake);
    while (r->finished < r->n) pthread_cond_wait(&r->done, &r->lock);
    pthread_mutex_unlock(&r->lock);
    gboolean ok = TRUE;
    for (gint i = 0; i < r->n; i++) ok = ok && r->w[i].ok;
    return ok;
}

dR_Replicas *dR_replicasCreate(gint numReplicas, const gint *ordinals, gint batchPerReplica, dR_ReplicaBuilder build, void *user, gboolean dryRun)
{
    if (numReplicas < 1 || numReplicas > 64 || batchPerReplica < 1 || !build) return NULL;
    dR_Replicas *r = (dR_Replicas *)calloc(1, sizeof(dR_Replicas));
    if (!r) return NULL;
    r->n = numReplicas; r->batch = batchPerReplica; r->build = build; r->user = user; r->dryRun = dryRun;
    r->w = (dR_ReplicaWorker *)calloc((size_t)numReplicas, sizeof(dR_ReplicaWorker));
    pthread_mutex_init(&r->lock, NULL);
    pthread_cond_init(&r->wake, NULL);
    pthread_cond_init(&r->done, NULL);
    gint started = 0;
    for (gint i = 0; i < numReplicas && r->w; i++, started++) {
        r->w[i].owner = r; r->w[i].index = i; r->w[i].ordinal = ordinals ? ordinals[i] : i;
        if (pthread_create(&r->w[i].thread, NULL, workerMain, &r->w[i]) != 0) break;
    }
    if (!r->w || started < numReplicas) {
        g_print("dR_replicasCreate: could not start %d worker threads\n", numReplicas);
        r->n = started;
        dR_replicasDestroy(r);
        return NULL;
    }
    if (!runJob(r, JOB_BUILD)) {
        g_print("dR_replicasCreate: building or preparing a replica failed\n");
        dR_replicasDestroy(r);
        return NULL;
    }
    dR_Shape3 *is = dR_getFeedNodeInputShape(r->w[0].feed), *os = dR_getOutputShape(r->w[0].out);
    r->inFloats = (size_t)is->s0 * is->s1 * is->s2;
    r->outFloats = (size_t)os->s0 * os->s1 * os->s2;
    return r;
}

static gboolean folderBuilder(dR_Graph *net, gint replica, void *user, dR_Node **feed, dR_Node **output)
{
    const dR_FolderOptions *o = (const dR_FolderOptions *)user;
    dR_Node **nodes = NULL, **feeds = NULL;
    gint nn = 0, nf = 0;
    (void)replica;
    if (!dR_setMathMode(net, o->mathMode) || !dR_setInterfaceLayout(net, o->layout)) return FALSE;
    dR_Node *last = dR_loadGraph(net, (gchar *)o->folder, &nodes, &nn, &feeds, &nf);
    if (!last || nf != 1) { free(nodes); free(feeds); return FALSE; }
    *feed = feeds[0];
    *output = last;
    free(nodes); free(feeds);
    return TRUE;
}

dR_Replicas *dR_replicasLoad(gint numReplicas, const gint *ordinals, gint batchPerReplica, const gchar *modelFolder, gint mathMode, gint layout)
{
    dR_FolderOptions opts;          /* read by the builder only while dR_replicasCreate runs */
    opts.folder = modelFolder; opts.mathMode = mathMode; opts.layout = layout;
    if (!modelFolder) return NULL;
    dR_Replicas *r = dR_replicasCreate(numReplicas, ordinals, batchPerReplica, folderBuilder, &opts, FALSE);
    if (r) r->user = NULL;
    return r;
}

gint dR_replicasCount(dR_Replicas *r) { return r ? r->n : 0; }
gint dR_replicasGlobalBatch(dR_Replicas *r) { return r ? r->n * r->batch : 0; }
size_t dR_replicasInputFloatsPerImage(dR_Replicas *r) { return r ? r->inFloats : 0; }
size_t dR_replicasOutputFloatsPerImage(dR_Replicas *r) { return r ? r->outFloats : 0; }
dR_Graph *dR_replicasGraph(dR_Replicas *r, gint replica) { return r && replica >= 0 && replica < r->n ? r->w[replica].net : NULL; }

void dR_replicasShard(dR_Replicas *r, gint replica, gint *lo, gint *hi)
{
    *lo = *hi = 0;
    if (!r || replica < 0 || replica >= r->n) return;
    *lo = replica * r->batch;
    *hi = *lo + r->batch;
}

gboolean dR_replicasApply(dR_Replicas *r, const gfloat *hostIn, gfloat *hostOut, gint steps, gdouble *msMax)
{
    if (msMax) *msMax = 0.0;
    if (!r || !hostIn || !hostOut || steps < 1 || r->dryRun) return FALSE;
    r->jobIn = hostIn; r->jobOut = hostOut; r->jobSteps = steps;
    const gboolean ok = runJob(r, JOB_APPLY);
    if (msMax)
        for (gint i = 0; i < r->n; i++) if (r->w[i].ms > *msMax) *msMax = r->w[i].ms;
    return ok;
}

void dR_replicasDestroy(dR_Replicas *r)
{
    if (!r) return;
    if (r->n > 0 && r->w) {
        runJob(r, JOB_QUIT);
        for (gint i = 0; i < r->n; i++) pthread_join(r->w[i].thread, NULL);
    }
    pthread_mutex_destroy(&r->lock);
    pthread_cond_destroy(&r->wake);
    pthread_cond_destroy(&r->done);
    free(r->w);
    free(r);
}
