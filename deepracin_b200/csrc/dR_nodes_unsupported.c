/*
 * Node constructors outside the CNN-layer hot path.  They exist so that every symbol the
 * reference's Python module resolves at import (python/deepracin/__init__.py.in:125-213)
 * is present; each reports that it is not part of the CUDA build and returns NULL.
 */
#include "dR_nodes_unsupported.h"

static dR_Node *unsupported(const char *what)
{
    g_print("%s is not supported in the CUDA build of deepRacin (outside the CNN-layer path)\n", what);
    return NULL;
}

dR_Node *dR_Conv2dTransposed(dR_Graph *net, dR_Node *in, dR_Shape4 f, dR_Shape4 s, dR_ActivationType a, gboolean b)
{ (void)net; (void)in; (void)f; (void)s; (void)a; (void)b; return unsupported("dR_Conv2dTransposed"); }
void dR_Conv2dtransposed_setVariables(dR_Node *l, gfloat *w, gfloat *b) { (void)l; (void)w; (void)b; unsupported("dR_Conv2dtransposed_setVariables"); }
dR_Node *dR_BatchNormalization(dR_Graph *net, dR_Node *in) { (void)net; (void)in; return unsupported("dR_BatchNormalization"); }
dR_Node *dR_MaskDependentFilter(dR_Graph *net, dR_Node *a, dR_Node *b, dR_Shape3 *s) { (void)net; (void)a; (void)b; (void)s; return unsupported("dR_MaskDependentFilter"); }
void dR_MaskDependentFilter_setVariables(dR_Node *l, gfloat *w, gfloat *b) { (void)l; (void)w; (void)b; unsupported("dR_MaskDependentFilter_setVariables"); }
dR_Node *dR_PerPixelFilter(dR_Graph *net, dR_Node *a, dR_Node *b, dR_Shape4 *s, dR_Shape4 *t) { (void)net; (void)a; (void)b; (void)s; (void)t; return unsupported("dR_PerPixelFilter"); }
dR_Node *dR_ResolveRoI(dR_Graph *net, dR_Node *in, dR_Shape3 *s) { (void)net; (void)in; (void)s; return unsupported("dR_ResolveRoI"); }
dR_Node *dR_RGB2gray(dR_Graph *net, dR_Node *in) { (void)net; (void)in; return unsupported("dR_RGB2gray"); }
dR_Node *dR_Upscaling(dR_Graph *net, dR_Node *in, gint t, gint x, gint y) { (void)net; (void)in; (void)t; (void)x; (void)y; return unsupported("dR_Upscaling"); }
dR_Node *dR_LabelCreation(dR_Graph *net, dR_Node *in, gint t, gfloat a, gfloat b, gfloat c) { (void)net; (void)in; (void)t; (void)a; (void)b; (void)c; return unsupported("dR_LabelCreation"); }
dR_Node *dR_Normalization(dR_Graph *net, dR_Node *in, gint t, gfloat m, gfloat d) { (void)net; (void)in; (void)t; (void)m; (void)d; return unsupported("dR_Normalization"); }
dR_Node *dR_FFT(dR_Graph *net, dR_Node *in) { (void)net; (void)in; return unsupported("dR_FFT"); }
