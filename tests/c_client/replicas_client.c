/*
 * C caller of the batch-sharded replica interface (include/dR_replicas.h): R replicas of a saved model, one host thread and
 * one CUDA device each (a device may be named more than once), one image per replica and step; the global batch is scattered
 * and the class probabilities gathered by host copies in image order.
 *
 * usage: replicas_client <model folder> <R> <device ordinal of replica 0> ... <ordinal of replica R-1> [--dry-run] [image.f32 x R]
 *   image.f32 = 224 x 224 x 3 float32 in [H][W][C] order; fed in the library's [C][H][W] interface layout
 * prints "class <argmax>" per image in global order; with --dry-run the replicas are planned without a device.
 */
#include <dR_replicas.h>

#define SIDE 224

static gboolean load_folder(dR_Graph *net, gint replica, void *user, dR_Node **feed, dR_Node **output)
{
    dR_Node **nodes = NULL, **feeds = NULL;
    gint nn = 0, nf = 0;
    dR_Node *last = dR_loadGraph(net, (gchar *)user, &nodes, &nn, &feeds, &nf);
    (void)replica;
    if (!last || nf != 1) return FALSE;
    *feed = feeds[0];
    *output = last;
    free(nodes); free(feeds);
    return TRUE;
}

int main(int argc, char **argv)
{
    gint ordinals[16], R, i, j, k, arg = 3, dry = 0;
    const int count = SIDE * SIDE * 3;
    if (argc < 3) { printf("usage: %s <model folder> <R> <ordinals...> [--dry-run] [images...]\n", argv[0]); return 2; }
    R = atoi(argv[2]);
    if (R < 1 || R > 16 || argc < 3 + R) return 2;
    for (i = 0; i < R; i++) ordinals[i] = atoi(argv[arg++]);
    if (arg < argc && strcmp(argv[arg], "--dry-run") == 0) { dry = 1; arg++; }

    dR_Replicas *r = dR_replicasCreate(R, ordinals, 1, load_folder, argv[1], dry);
    if (!r) { printf("create failed\n"); return 3; }
    if (dR_replicasCount(r) != R || dR_replicasGlobalBatch(r) != R) return 4;
    if (dR_replicasInputFloatsPerImage(r) != (size_t)count || dR_replicasOutputFloatsPerImage(r) != 1000) return 5;
    for (i = 0; i < R; i++) {
        gint lo, hi;
        dR_replicasShard(r, i, &lo, &hi);
        if (lo != i || hi != i + 1 || !dR_replicasGraph(r, i) || !dR_replicasGraph(r, i)->prepared) return 6;
    }
    printf("replicas %d global batch %d\n", dR_replicasCount(r), dR_replicasGlobalBatch(r));
    float *in = (float *)dR_allocPinned((size_t)R * count * sizeof(float));
    float *out = (float *)dR_allocPinned((size_t)R * 1000 * sizeof(float));
    if (dry) {
        float dummy_in[4] = {0}, dummy_out[4];
        if (dR_replicasApply(r, dummy_in, dummy_out, 1, NULL)) { printf("a dry run applied\n"); return 7; }
        dR_replicasDestroy(r);
        printf("dry run ok\n");
        return 0;
    }
    if (!in || !out || argc < arg + R) { printf("need %d images\n", R); return 8; }
    float *hwc = (float *)malloc(count * sizeof(float));
    for (i = 0; i < R; i++) {
        FILE *f = fopen(argv[arg + i], "rb");
        if (!f || fread(hwc, sizeof(float), count, f) != (size_t)count) { printf("cannot read %s\n", argv[arg + i]); return 9; }
        fclose(f);
        for (j = 0; j < count; j++)
            in[(size_t)i * count + j] = hwc[((j / SIDE) % SIDE) * SIDE * 3 + (j % SIDE) * 3 + j / (SIDE * SIDE)];
    }
    for (k = 0; k < 2; k++) {            /* twice: the second step must give the same answers */
        gdouble ms = 0.0;
        if (!dR_replicasApply(r, in, out, 1, &ms) || ms <= 0.0) { printf("apply failed\n"); return 10; }
        for (i = 0; i < R; i++) {
            int argmax = 0;
            for (j = 1; j < 1000; j++)
                if (out[(size_t)i * 1000 + j] > out[(size_t)i * 1000 + argmax]) argmax = j;
            printf("class %d\n", argmax);
        }
    }
    free(hwc);
    dR_freePinned(in); dR_freePinned(out);
    dR_replicasDestroy(r);
    return 0;
}
