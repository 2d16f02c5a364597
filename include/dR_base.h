/* Umbrella include for the node headers (reference include/dR_base.h). */
#ifndef DR_BASE_H
#define DR_BASE_H
#include "dR_types.h"
#include "dR_nodes_conv2d.h"
#include "dR_nodes_pooling.h"
#include "dR_nodes_fc.h"
#include "dR_nodes_math.h"
#include "dR_nodes_transform.h"
#include "dR_nodes_unsupported.h"
#endif
