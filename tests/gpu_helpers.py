"""Helpers for the GPU parity tests: build a graph through the Python mirror of the reference's
interface (which calls the C ABI of libdeepracin.so), run it, return [n, C, H, W] arrays."""
import numpy as np

import deepracin_b200 as dr

TOL_FP32 = 1e-4   # max|err| <= 1e-4 * max|ref| per layer output (exact-FP32 kernels)
TOL_TF32 = 3e-3   # tensor-core TF32 kernels


def rel_err(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))


def hwio(w):
    """oracle conv weights [Cin, Cout, kh, kw] -> the Python interface's HWIO"""
    return np.ascontiguousarray(w.transpose(2, 3, 0, 1))


def run_graph(build, feeds, batch=None, **opts):
    """build(graph, feed_nodes) -> output node or list of nodes.  feeds: list of [n, C, H, W] arrays.
    Returns list of [n, C, H, W] outputs (always with the batch axis)."""
    n = feeds[0].shape[0] if batch is None else batch
    with dr.Environment() as env:
        for k in ("silent", "profileGPU", "debuginfo"):
            if k in opts:
                setattr(env, k, opts.pop(k))
        g = env.create_graph("CHW")
        g.batch = n
        for k, v in opts.items():
            setattr(g, k, v)
        fnodes = [dr.feed_node(g, list(f.shape[1:])) for f in feeds]
        outs = build(g, fnodes)
        outs = outs if isinstance(outs, (list, tuple)) else [outs]
        for o in outs:
            dr.mark_as_output(o)
        dr.prepare(g)
        for fn, f in zip(fnodes, feeds):
            dr.feed_data(fn, f)
        res = dr.apply(g)
        res = [r.reshape((n, o.out_shape[2], o.out_shape[1], o.out_shape[0])) for r, o in zip(res, outs)]
        return res


def conv_build(w, b, stride=1, act=1, algo=None):
    cin, cout, kh, kw = w.shape

    def build(g, f):
        return dr.Conv2d(f[0], [kh, kw, cin, cout], [1, stride, stride, 1], "relu" if act else "linear", hwio(w), b, algo=algo)
    return build
