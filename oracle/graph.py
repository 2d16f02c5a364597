"""Run a saved deepRacin graph (graph.dr + N.var) on the CPU oracle -- TEST INFRASTRUCTURE ONLY.

The file format follows the reference's reader, src/dR_parser.c:182-523: a header line
``deepRACIN graph: <N> nodes, <F> feed nodes`` and five lines per node (``Node <id>: <Type>``,
``params:``, ``previous_nodes:``, ``next_nodes:`` (ignored), ``variable_files:``); ``.var`` files
are raw little-endian float32.
"""
import os

import numpy as np

from . import (concat, conv2d, croporpad, elemwise1, elemwise2, fc, pool, ref_available, ref_conv2d_1x1,
               ref_conv2d_winograd, ref_elemwise1, ref_fc, ref_pool, ref_slice, ref_softmax, slice_, softmax)


def parse_graph(path):
    with open(os.path.join(path, "graph.dr")) as f:
        lines = [ln.rstrip("\r\n") for ln in f.read().split("\n")]
    head = lines[0].split()
    n_nodes = int(head[2])
    nodes = []
    for i in range(n_nodes):
        l = lines[1 + 5 * i: 6 + 5 * i]
        hdr = l[0].split()
        nodes.append({
            "id": int(hdr[1].rstrip(":")),
            "type": hdr[2],
            "params": l[1].split()[1:],
            "prev": [int(t) for t in l[2].split()[1:]],
            "vars": [np.fromfile(os.path.join(path, v), dtype="<f4") for v in l[4].split()[1:]],
        })
    return nodes


def run_graph(nodes, feeds, leg="restate", keep=False):
    """feeds: list of [n,C,H,W] arrays in feed-node order.  Returns the last node's output
    (or every node's output when keep=True).  leg: "restate" or "ref" (reference kernels where the
    reference ships one for the shape, the restatement elsewhere)."""
    use_ref = leg == "ref" and ref_available()
    outs = {}
    feed_it = iter(feeds)
    for nd in nodes:
        t, p = nd["type"], nd["params"]
        ins = [outs[i] for i in nd["prev"]]
        if t == "DataFeedNode":
            y = np.ascontiguousarray(next(feed_it), dtype=np.float32)
        elif t == "Slice":
            o = [int(v) for v in p[0:3]]
            s = [int(v) for v in p[4:7]]
            y = ref_slice(ins[0], o, s) if use_ref else slice_(ins[0], o, s)
        elif t == "ElemWise1Op":
            y = (ref_elemwise1 if use_ref else elemwise1)(ins[0], int(p[0]), float(p[1]))
        elif t == "ElemWise2Op":
            y = elemwise2(ins[0], ins[1], int(p[0]))
        elif t == "Concat":
            y = concat(ins, int(p[1]))
        elif t == "CropOrPad":
            y = croporpad(ins[0], [int(v) for v in p[0:3]])
        elif t == "Conv2D":
            act, use_b, kw, kh, cin, cout = (int(v) for v in p[0:6])
            sx, sy = int(p[7]), int(p[8])
            w = nd["vars"][0].reshape(cin, cout, kh, kw)
            b = nd["vars"][1] if use_b else None
            if use_ref and kw == 3 and kh == 3 and sx == 1 and sy == 1:
                y = ref_conv2d_winograd(ins[0], w, b, act)
            elif use_ref and kw == 1 and kh == 1 and sx == 1 and sy == 1:
                y = ref_conv2d_1x1(ins[0], w, b, act)
            else:
                y = conv2d(ins[0], w, b, (sx, sy), act)
        elif t == "FullyConnected":
            act, use_b, nin, nout = (int(v) for v in p[0:4])
            w = nd["vars"][0].reshape(nin, nout)
            b = nd["vars"][1] if use_b else None
            y = (ref_fc if use_ref else fc)(ins[0], w, b, act)
        elif t == "Pooling":
            kind = int(p[0])
            size = (int(p[2]), int(p[3]), int(p[4]))
            stride = (int(p[6]), int(p[7]), int(p[8]))
            key = (size[0], kind)
            if (use_ref and size[0] == size[1] and size[2] == 1 and stride[0] == stride[1] and stride[2] == 1
                    and key in ((3, 0), (2, 1), (14, 1))):
                y = ref_pool(ins[0], size[0], stride[0], kind)
            else:
                y = pool(ins[0], size, stride, kind)
        elif t == "Softmax":
            y = (ref_softmax if use_ref else softmax)(ins[0])
        else:
            raise ValueError("node type outside the hot path: " + t)
        outs[nd["id"]] = y
    return outs if keep else outs[nodes[-1]["id"]]
