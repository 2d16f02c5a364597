/* graph.dr + N.var model folder reader / writer and the printers
 * (reference include/dR_parser.h, src/dR_parser.c:58-523, 716-830). */
#ifndef DR_PARSER_H
#define DR_PARSER_H
#include "dR_base.h"
dR_Node *dR_parseGraph(dR_Graph *net, gchar *path, dR_Node ***nodelist, gint *numnodes, dR_Node ***feednodes, gint *numfeednodes);
gboolean dR_serializeGraph(dR_Graph *net, gchar *path);
void dR_printNet(dR_Graph *net, char *path);
void dR_printSchedule(dR_Graph *net);
#endif
