/*
 * A C caller of the drop-in boundary, written the way the reference's deployed examples use the library
 * (examples/squeezenet-v1.1/squeezenet_deployed.c:95-207): configuration by writing struct fields of
 * net->config / net->clConfig, dR_initCL, dR_loadGraph of a saved model folder, dR_setAsOutput on the last
 * node, dR_prepare, dR_getOutputBuffers once, then per image a [C][H][W] dR_feedData, dR_apply and a blocking
 * dR_downloadArray of the 1000 class probabilities.  Compiled by the tests with a C compiler against include/
 * only, so that header / struct-layout disagreement with the library shows up as a wrong answer here.
 *
 * usage: squeezenet_client <model folder> [--dry-run] [image.f32 ...]
 *   image.f32 = 224 x 224 x 3 float32 in [H][W][C] order (what a decoded PNG row holds)
 * prints one line "class <argmax> p <probability>" per image; with --dry-run the graph is planned without a
 * device and dR_apply must refuse.
 */
#include <deepRACIN.h>

#define SIDE 224

int main(int argc, char **argv)
{
    dR_Graph *net;
    dR_Node **nodeslist, **feedlist;
    dR_Node *lastnode;
    gint numnodes = 0, numfeeds = 0, dry = 0, i, j, first_image = 2;
    cl_mem *outbuffers[1];
    float *hwc, *feed_buffer, *odata;
    const int count = SIDE * SIDE * 3;

    if (argc < 2) { printf("usage: %s <model folder> [--dry-run] [image.f32 ...]\n", argv[0]); return 2; }
    if (argc > 2 && strcmp(argv[2], "--dry-run") == 0) { dry = 1; first_image = 3; }

    net = dR_NewGraph();
    net->config->debugInfo = FALSE;
    net->config->profilingGPU = FALSE;
    net->config->profilingCPU = FALSE;
    net->config->silent = TRUE;
    net->clConfig->clPlatformName = NULL;
    if (dry && !dR_setDryRun(net, TRUE)) return 3;
    if (!dR_initCL(net)) { printf("no device\n"); return 4; }

    lastnode = dR_loadGraph(net, argv[1], &nodeslist, &numnodes, &feedlist, &numfeeds);
    if (!lastnode || numnodes < 1 || numfeeds != 1 || lastnode != nodeslist[numnodes - 1]) { printf("load failed\n"); return 5; }
    if (net->number_of_layers != numnodes || net->allNodes->length != numnodes || net->feed_layers->length != 1) { printf("graph fields disagree\n"); return 6; }
    if (!dR_setAsOutput(net, lastnode) || net->output_layers->length != 1) return 7;
    if (!dR_prepare(net) || !net->prepared) { printf("prepare failed\n"); return 8; }
    {
        dR_Shape3 *os = dR_getOutputShape(lastnode), *is = dR_getFeedNodeInputShape(feedlist[0]);
        printf("nodes %d feeds %d in %dx%dx%d out %dx%dx%d\n", numnodes, numfeeds, is->s0, is->s1, is->s2, os->s0, os->s1, os->s2);
        if (is->s0 != SIDE || is->s1 != SIDE || is->s2 != 3 || os->s0 * os->s1 * os->s2 != 1000) return 9;
    }
    if (dR_getOutputBuffers(net, outbuffers) != 1) return 10;
    if (dry) {
        if (dR_apply(net)) { printf("a dry run applied\n"); return 11; }
        dR_cleanup(net, TRUE);
        printf("dry run ok\n");
        return 0;
    }

    hwc = (float *)malloc(count * sizeof(float));
    feed_buffer = (float *)malloc(count * sizeof(float));
    odata = (float *)malloc(1000 * sizeof(float));
    for (i = first_image; i < argc; i++) {
        FILE *f = fopen(argv[i], "rb");
        int argmax = 0;
        if (!f || fread(hwc, sizeof(float), count, f) != (size_t)count) { printf("cannot read %s\n", argv[i]); return 12; }
        fclose(f);
        /* the library wants [c][h][w]; the decoded image is [h][w][c] */
        for (j = 0; j < count; j++)
            feed_buffer[j] = hwc[((j / SIDE) % SIDE) * SIDE * 3 + (j % SIDE) * 3 + j / (SIDE * SIDE)];
        dR_feedData(net, feedlist[0], (cl_float *)feed_buffer, 0, count);
        if (!dR_apply(net)) { printf("apply failed\n"); return 13; }
        dR_downloadArray(net, "", outbuffers[0], 0, 1000 * sizeof(cl_float), odata);
        for (j = 1; j < 1000; j++)
            if (odata[j] > odata[argmax]) argmax = j;
        printf("class %d p %.4f\n", argmax, odata[argmax]);
    }
    if (dR_getDeviceStatus(net) != 0) { printf("device status set\n"); return 14; }
    free(hwc); free(feed_buffer); free(odata); free(nodeslist); free(feedlist);
    dR_cleanup(net, TRUE);
    return 0;
}
