/*
 * Saved-model folder reader / writer and the text printers.
 *
 * Format (byte-compatible with the reference's src/dR_parser.c:58-523):
 *   line 1         "deepRACIN graph: <N> nodes, <F> feed nodes"
 *   per node       "Node <id>: <Type>"
 *                  "params: p0 p1 ..."
 *                  "previous_nodes: i j ..."
 *                  "next_nodes: ..."            (written, ignored on load)
 *                  "variable_files: k.var ..."  (raw little-endian float32, global counter)
 * Type strings are matched by prefix in the reference; here they are matched exactly, which
 * accepts every file the reference writes.
 */
#include "dR_parser.h"
#include "dR_core.h"

#define MAX_PARAMS 16
#define MAX_VARS 4
#define MAX_PREV 256

typedef struct {
    const char *name;
    fParseAppendNode parse;
    gint minInputs, maxInputs;
} dR_NodeKind;

static const dR_NodeKind kinds[] = {
    {"Conv2D", dR_conv2d_parseAppendNode, 1, 1},
    {"Pooling", dR_pooling_parseAppendNode, 1, 1},
    {"FullyConnected", dR_fc_parseAppendNode, 1, 1},
    {"Softmax", dR_softmax_parseAppendNode, 1, 1},
    {"Slice", dR_slice_parseAppendNode, 1, 1},
    {"Concat", dR_concat_parseAppendNode, 2, 3},
    {"CropOrPad", dR_croporpad_parseAppendNode, 1, 1},
    {"ElemWise2Op", dR_elemwise2op_parseAppendNode, 2, 2},
    {"ElemWise1Op", dR_elemwise1op_parseAppendNode, 1, 1},
    {"DataFeedNode", dR_datafeednode_parseAppendNode, 0, 0},
};

/* splits `line` in place at blanks; returns the token count */
static gint tokenize(gchar *line, gchar **tok, gint maxTok)
{
    gint n = 0;
    gchar *p = line;
    while (*p && n < maxTok) {
        while (*p == ' ' || *p == '\t' || *p == '\r') p++;
        if (!*p) break;
        tok[n++] = p;
        while (*p && *p != ' ' && *p != '\t' && *p != '\r') p++;
        if (*p) *p++ = 0;
    }
    return n;
}

static gchar *nextLine(gchar **cursor)
{
    gchar *p = *cursor;
    if (!p || !*p) return NULL;
    gchar *end = strchr(p, '\n');
    if (end) { *end = 0; *cursor = end + 1; } else { *cursor = p + strlen(p); }
    return p;
}

/* Floats that variable file `k` of a node must hold, from the node's parameters: Conv2D "act useBias kw kh Cin Cout ..."
 * (src/dR_nodes_conv2d.c:153-162) has kw*kh*Cin*Cout weights and, with a bias, Cout more; FullyConnected "act useBias Nin
 * Nout" (src/dR_nodes_fc.c:70-73) has Nin*Nout and Nout.  -1: the node type takes no variables this function knows; -2: the
 * parameters themselves are unusable (non-positive or overflowing sizes).  setVariables copies exactly this many floats out of
 * the file's buffer, so a shorter file would be read past its end. */
static long long expectedVariableFloats(const char *desc, gchar **params, gint numParams, gint k)
{
    long long dims[4];
    gint first, nd;
    if (strcmp(desc, "Conv2D") == 0) { first = 2; nd = 4; }
    else if (strcmp(desc, "FullyConnected") == 0) { first = 2; nd = 2; }
    else return -1;
    if (numParams < first + nd) return -2;
    long long prod = 1;
    for (gint i = 0; i < nd; i++) {
        dims[i] = atoll(params[first + i]);
        if (dims[i] <= 0 || dims[i] > 0x7fffffffLL) return -2;
        prod *= dims[i];
        if (prod > 0x7fffffffLL) return -2;
    }
    if (k == 0) return prod;
    if (k == 1 && atoi(params[1])) return dims[nd - 1];
    return -2;                                          /* more variable files than the node has variables */
}

dR_Node *dR_parseGraph(dR_Graph *net, gchar *path, dR_Node ***outnodes, gint *numnodes, dR_Node ***outfeednodes, gint *numfeednodes)
{
    if (net->number_of_layers != 0) {
        g_print("dR_parseGraph can only fill an empty graph! Given graph not empty!\n");
        return NULL;
    }
    net->config->modelPath = g_strdup(path);
    gchar *filepath = dR_build_filename(path, "graph.dr");
    if (!net->config->silent) g_print("Loading Model File %s ...\n", path);
    size_t length = 0;
    gchar *content = dR_file_get_contents(filepath, &length);
    g_free(filepath);
    if (!content) { g_print("Error while opening the graph file.\n"); return NULL; }

    gchar *cursor = content;
    gchar *tok[MAX_PREV + 2];
    gchar *line = nextLine(&cursor);
    gint nt = line ? tokenize(line, tok, 16) : 0;
    if (nt < 6 || strcmp(tok[0], "deepRACIN") != 0) { g_print("Parsing Error: not a deepRACIN graph file\n"); g_free(content); return NULL; }
    gint nNodes = atoi(tok[2]), nFeeds = atoi(tok[4]);
    if (nNodes <= 0 || nFeeds < 0) { g_print("Parsing Error: bad node counts\n"); g_free(content); return NULL; }

    dR_Node **graphnodes = (dR_Node **)calloc((size_t)nNodes, sizeof(dR_Node *));
    dR_Node **feednodes = (dR_Node **)calloc((size_t)(nFeeds > 0 ? nFeeds : 1), sizeof(dR_Node *));
    gint feedIt = 0;
    if (!net->config->silent) g_print("Found graph with %d nodes and %d feed nodes.\n", nNodes, nFeeds);

    for (gint i = 0; i < nNodes; i++) {
        gchar *params[MAX_PARAMS];
        gfloat *variables[MAX_VARS] = {0};
        dR_Node *inputs[MAX_PREV];
        gint numParams = 0, numVars = 0, numPrev = 0, id;
        dR_Node *node = NULL;
        gchar desc[64];

        line = nextLine(&cursor);
        nt = line ? tokenize(line, tok, 8) : 0;
        if (nt < 3) { g_print("Parsing Error: truncated graph file at node %d\n", i); goto fail; }
        id = atoi(tok[1]);
        snprintf(desc, sizeof desc, "%s", tok[2]);
        if (id < 0 || id >= nNodes) { g_print("Parsing Error: node id %d out of range\n", id); goto fail; }

        line = nextLine(&cursor);
        nt = line ? tokenize(line, tok, MAX_PARAMS + 1) : 0;
        if (nt < 1) { g_print("Parsing Error: missing params line of node %d\n", id); goto fail; }
        for (gint k = 1; k < nt; k++) params[numParams++] = tok[k];

        gchar *prevTok[MAX_PREV + 1];
        line = nextLine(&cursor);
        nt = line ? tokenize(line, prevTok, MAX_PREV + 1) : 0;
        if (nt < 1) { g_print("Parsing Error: missing previous_nodes line of node %d\n", id); goto fail; }
        for (gint k = 1; k < nt; k++) {
            gint pid = atoi(prevTok[k]);
            if (pid < 0 || pid >= nNodes || !graphnodes[pid]) { g_print("Parsing Error: node %d refers to unknown node %d\n", id, pid); goto fail; }
            inputs[numPrev++] = graphnodes[pid];
        }
        line = nextLine(&cursor);                       /* next_nodes: ignored */
        gchar *varTok[MAX_VARS + 2];
        line = nextLine(&cursor);
        nt = line ? tokenize(line, varTok, MAX_VARS + 1) : 0;
        if (nt < 1) { g_print("Parsing Error: missing variable_files line of node %d\n", id); goto fail; }
        for (gint k = 1; k < nt; k++) {
            gchar *vp = dR_build_filename(path, varTok[k]);
            size_t vlen = 0;
            variables[numVars] = (gfloat *)dR_file_get_contents(vp, &vlen);
            if (!variables[numVars]) { g_print("Error while opening variable file: %s\n", vp); g_free(vp); goto failvars; }
            numVars++;
            const long long want = expectedVariableFloats(desc, params, numParams, numVars - 1);
            if (want == -2 || (want >= 0 && (long long)vlen != want * (long long)sizeof(gfloat))) {
                g_print("Parsing Error: variable file %s holds %zu bytes, node %d (%s) needs %lld floats\n", vp, vlen, id, desc, want);
                g_free(vp);
                goto failvars;
            }
            g_free(vp);
        }
        if (!net->config->silent && net->config->debugInfo)
            g_print("Found %s with id %d, %d params and %d variables\n", desc, id, numParams, numVars);

        const dR_NodeKind *kind = NULL;
        for (size_t k = 0; k < sizeof kinds / sizeof kinds[0]; k++)
            if (strcmp(desc, kinds[k].name) == 0) kind = &kinds[k];
        if (!kind) { g_print("Parsing Error: Node could not be identified: %s!\n", desc); goto failvars; }
        if (numPrev < kind->minInputs || numPrev > kind->maxInputs) { g_print("Failed to parse %s node: wrong number of inputs (%d)\n", desc, numPrev); goto failvars; }
        node = kind->parse(net, numPrev ? inputs : NULL, numPrev, params, numParams, variables, numVars);
        if (!node) { g_print("Parsing Error: Node could not be appended!\n"); goto failvars; }
        graphnodes[id] = node;
        if (node->type == tDataFeedNode && feedIt < nFeeds) feednodes[feedIt++] = node;
        for (gint k = 0; k < numVars; k++) g_free(variables[k]);
        continue;
    failvars:
        for (gint k = 0; k < numVars; k++) g_free(variables[k]);
        goto fail;
    }
    g_free(content);
    *outnodes = graphnodes; *outfeednodes = feednodes; *numnodes = nNodes; *numfeednodes = nFeeds;
    return graphnodes[nNodes - 1];
fail:
    g_free(content); g_free(graphnodes); g_free(feednodes);
    return NULL;
}

gboolean dR_serializeGraph(dR_Graph *net, gchar *path)
{
    gchar *folder = dR_build_filename(path, "dr_graph_export");
    if (dR_mkdir_with_parents(folder) != 0) {
        g_print("Error: Could not create folder %s.\n", folder);
        g_free(folder);
        return FALSE;
    }
    gchar *gp = dR_build_filename(folder, "graph.dr");
    FILE *out = fopen(gp, "wb");
    g_free(gp);
    if (!out) { g_print("Error: cannot write graph.dr in %s\n", folder); g_free(folder); return FALSE; }
    fprintf(out, "deepRACIN graph: %d nodes, %d feed nodes", net->allNodes->length, net->feed_layers->length);
    gint counter = 0;
    gboolean ok = TRUE;
    for (dR_ListElement *e = net->allNodes->first; e && ok; e = e->next) {
        dR_Node *n = (dR_Node *)e->element;
        gchar *params[MAX_PARAMS];
        gfloat *variables[MAX_VARS];
        gint sizes[MAX_VARS];
        gint np = MAX_PARAMS, nv = MAX_VARS;
        gchar *desc = n->serializeNode(n, params, &np, variables, sizes, &nv);
        if (!desc) { ok = FALSE; break; }
        fprintf(out, "\nNode %d: %s\nparams:", n->layerID, desc);
        for (gint i = 0; i < np; i++) { fprintf(out, " %s", params[i]); g_free(params[i]); }
        fprintf(out, "\nprevious_nodes:");
        for (dR_ListElement *p = n->previous_layers->first; p; p = p->next) fprintf(out, " %d", ((dR_Node *)p->element)->layerID);
        fprintf(out, "\nnext_nodes:");
        for (dR_ListElement *p = n->next_layers->first; p; p = p->next) fprintf(out, " %d", ((dR_Node *)p->element)->layerID);
        fprintf(out, "\nvariable_files:");
        for (gint i = 0; i < nv; i++) {
            gchar *name = g_strdup_printf("%d.var", counter++);
            gchar *vp = dR_build_filename(folder, name);
            fprintf(out, " %s", name);
            FILE *vf = fopen(vp, "wb");
            if (!vf || fwrite(variables[i], sizeof(gfloat), (size_t)sizes[i], vf) != (size_t)sizes[i]) {
                g_print("Error while creating the variable file %s.\n", name);
                ok = FALSE;
            }
            if (vf) fclose(vf);
            g_free(vp); g_free(name);
        }
    }
    fprintf(out, "\n");
    fclose(out);
    g_free(folder);
    return ok;
}

/* reference src/dR_parser.c:716-730 */
void dR_printSchedule(dR_Graph *net)
{
    g_print("Execution order:");
    for (dR_ListElement *e = net->scheduledLayers->first; e; e = e->next) g_print(" %d", ((dR_Node *)e->element)->layerID);
    g_print("\n");
}

/* reference src/dR_parser.c:788-830; prints to stdout, or to `path`/net.txt when a path is given */
void dR_printNet(dR_Graph *net, char *path)
{
    FILE *out = stdout;
    if (path) {
        gchar *fp = dR_build_filename(path, "net.txt");
        out = fopen(fp, "w");
        g_free(fp);
        if (!out) { g_print("dR_printNet: cannot write to %s\n", path); return; }
    }
    fprintf(out, "deepRACIN graph with %d nodes\n", net->allNodes->length);
    for (dR_ListElement *e = net->allNodes->first; e; e = e->next) {
        dR_Node *n = (dR_Node *)e->element;
        gchar *s = n->printLayer ? n->printLayer(n) : g_strdup("(node)\n");
        fprintf(out, "%s", s);
        g_free(s);
        fprintf(out, " Inputs:");
        for (dR_ListElement *p = n->previous_layers->first; p; p = p->next) fprintf(out, " %d", ((dR_Node *)p->element)->layerID);
        if (n->propagated) fprintf(out, "\n Output shape: %dx%dx%d", n->oshape.s0, n->oshape.s1, n->oshape.s2);
        fprintf(out, "\n\n");
    }
    if (out != stdout) fclose(out); else fflush(stdout);
}
