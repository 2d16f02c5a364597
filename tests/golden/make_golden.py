"""Generates tests/golden/reference_kernels.npz -- outputs of the REFERENCE's own kernel sources
(compiled as C by oracle/ref_shim, launch geometry restated from the reference's host code) on the
seeded cases of tests/cases.py, plus the SqueezeNet known-answer outputs.

Run where a reference checkout is present:  python tests/golden/make_golden.py
The reference cannot travel to the GPU box; these vectors do.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from oracle import build_oracle, graph  # noqa: E402
import cases  # noqa: E402


def main():
    build_oracle.build_all()
    if not oracle.ref_available():
        raise SystemExit("reference checkout not found: cannot generate golden vectors")
    out = {}
    for name, (kind, kw) in cases.GOLDEN_CASES.items():
        ins = cases.make_inputs(name)
        if kind == "wino":
            out[name] = oracle.ref_conv2d_winograd(ins[0], ins[1], ins[2], kw["act"])
        elif kind == "c1x1":
            out[name] = oracle.ref_conv2d_1x1(ins[0], ins[1], ins[2], kw["act"])
        elif kind == "fc":
            out[name] = oracle.ref_fc(ins[0], ins[1], ins[2], kw["act"])
        elif kind == "pool":
            out[name] = oracle.ref_pool(ins[0], kw["k"], kw["stride"], kw["kind"])
        elif kind == "softmax":
            out[name] = oracle.ref_softmax(ins[0])
        elif kind == "ew1":
            for op, s in cases.EW1_OPS:
                out["%s_op%d" % (name, op)] = oracle.ref_elemwise1(ins[0], op, s)
        elif kind == "ew2":
            for op in cases.EW2_OPS:
                out["%s_op%d" % (name, op)] = oracle.ref_elemwise2(ins[0], ins[1], op)
        elif kind == "slice":
            out[name + "_slice"] = oracle.ref_slice(ins[0], (2, 1, 1), (5, 6, 3))
            out[name + "_pad"] = oracle.ref_croporpad(ins[0], (11, 12, 6))
            out[name + "_crop"] = oracle.ref_croporpad(ins[0], (5, 4, 6))
    # known-answer test: pretrained SqueezeNet on the reference's two example images
    d = oracle.staged_squeezenet_dir()
    nodes = graph.parse_graph(d)
    for img in ("tiger", "puzzle"):
        a = np.fromfile(os.path.join(d, img + "_224x224x3_rgb_hwc.f32"), dtype=np.float32).reshape(224, 224, 3)
        x = np.ascontiguousarray(a.transpose(2, 0, 1))[None]
        outs = graph.run_graph(nodes, [x], leg="ref", keep=True)
        out["kat_%s_softmax" % img] = outs[47].reshape(1000)
        out["kat_%s_logits" % img] = outs[46].reshape(1000)
        out["kat_%s_fire2_concat_sample" % img] = outs[14][0, ::8, ::7, ::7].copy()
    np.savez_compressed(os.path.join(HERE, "reference_kernels.npz"), **out)
    print("wrote %d arrays" % len(out))


if __name__ == "__main__":
    main()
