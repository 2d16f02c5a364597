"""Single-layer microbenchmarks through the C API of libdeepracin.so (one node per graph).

  python deepracin_b200/layer_bench.py conv CIN COUT HW BATCH [--k 3] [--math tf32|fp32] [--algo auto|direct|winograd|winograd4|1x1|tensor|tensor_winograd]
  python deepracin_b200/layer_bench.py fc NIN NOUT BATCH [--math ...]
  python deepracin_b200/layer_bench.py sweep           # the conv-sweep and 1x1/FC configurations of the benchmark spec
  python deepracin_b200/layer_bench.py vgg [BATCH]     # every distinct VGG-16 3x3 layer shape: direct tensor kernel vs tensor-core Winograd (TF32), Winograd vs direct (FP32)
  python deepracin_b200/layer_bench.py membound        # pooling / element-wise / softmax / copies: GB/s of the bytes they must move

Times `--iters` launches with CUDA events on the library's stream after `--warmup` launches and prints
one JSON line per layer: ms, direct-convolution TFLOP/s (Winograd gets no discount), minimum HBM
bytes (input + output + weights once) and the GB/s they imply.  Inputs N(0,1), He-normal weights,
small biases, ReLU.  Meant to be run under `ncu -k regex:...` for kernel-level profiles as well.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import deepracin_b200 as dr  # noqa: E402


def _rng(name):
    import zlib
    return np.random.Generator(np.random.PCG64(zlib.crc32(name.encode())))


def time_graph(g, iters, warmup):
    lib = dr.lib
    for _ in range(warmup):
        lib.dR_apply(g.ptr)
    lib.dR_synchronize(g.ptr)
    # the timed loop runs inside the library (dR_applyTimed): a Python-side loop adds several microseconds of host time per launch,
    # which a layer of 10-20 us cannot hide
    ms = lib.dR_applyTimed(g.ptr, iters)
    if ms <= 0:
        raise RuntimeError("dR_applyTimed failed")
    return ms / iters


def conv_layer(cin, cout, hw, batch, k=3, math="tf32", algo="auto", iters=20, warmup=5, act="relu"):
    r = _rng("lb_conv_%d_%d_%d_%d" % (cin, cout, hw, k))
    w = (r.standard_normal((k, k, cin, cout), dtype=np.float32) * np.float32(np.sqrt(2.0 / (k * k * cin))))
    b = (r.standard_normal(cout, dtype=np.float32) * np.float32(0.1))
    x = r.standard_normal((batch, hw, hw, cin), dtype=np.float32)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = batch
        g.math = math
        f = dr.feed_node(g, [hw, hw, cin])
        o = dr.Conv2d(f, [k, k, cin, cout], [1, 1, 1, 1], act, w, b, algo=None if algo == "auto" else algo)
        dr.mark_as_output(o)
        dr.lib.dR_setInterfaceLayout(g.ptr, 1)
        dr.prepare(g)
        dr.feed_data(f, x)
        ms = time_graph(g, iters, warmup)
        chosen = dr.lib.dR_getConvAlgo(o.ptr)
        status = dr.lib.dR_getDeviceStatus(g.ptr)
    flops = 2.0 * k * k * cin * cout * hw * hw * batch
    bytes_min = 4.0 * (batch * hw * hw * (cin + cout) + k * k * cin * cout)
    return {"layer": "conv%dx%d %d->%d @%dx%d batch %d" % (k, k, cin, cout, hw, hw, batch), "math": math,
            "algo": ["auto", "direct", "winograd", "1x1", "tensor", "tensor_winograd", "winograd4"][chosen], "ms": ms, "tflops": flops / ms / 1e9,
            "min_bytes": bytes_min, "gbs_at_min_bytes": bytes_min / ms / 1e6, "flop_per_byte": flops / bytes_min, "device_status": status}


def fc_layer(nin, nout, batch, math="fp32", iters=20, warmup=5):
    r = _rng("lb_fc_%d_%d" % (nin, nout))
    w = (r.standard_normal((nin, nout), dtype=np.float32) * np.float32(np.sqrt(2.0 / nin)))
    b = (r.standard_normal(nout, dtype=np.float32) * np.float32(0.1))
    x = r.standard_normal((batch, 1, 1, nin), dtype=np.float32)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = batch
        g.math = math
        f = dr.feed_node(g, [1, 1, nin])
        o = dr.Fully_Connected(f, [nin, nout], "relu", w, b)
        dr.mark_as_output(o)
        dr.prepare(g)
        dr.feed_data(f, x)
        ms = time_graph(g, iters, warmup)
    flops = 2.0 * nin * nout * batch
    bytes_min = 4.0 * (nin * nout + batch * (nin + nout))
    return {"layer": "fc %d->%d batch %d" % (nin, nout, batch), "math": math, "ms": ms, "tflops": flops / ms / 1e9,
            "min_bytes": bytes_min, "gbs_at_min_bytes": bytes_min / ms / 1e6, "flop_per_byte": flops / bytes_min}


def single_node(build, shape_hwc, batch, bytes_moved, label, iters=20, warmup=5, feeds=1):
    """Times a graph of one memory-bound node; reports GB/s of the bytes it has to move (in + out)."""
    r = _rng(label)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = batch
        fs = [dr.feed_node(g, list(shape_hwc)) for _ in range(feeds)]
        o = build(fs)
        dr.mark_as_output(o)
        dr.lib.dR_setInterfaceLayout(g.ptr, 1)
        dr.prepare(g)
        for f in fs:
            dr.feed_data(f, r.standard_normal((batch,) + tuple(shape_hwc), dtype=np.float32))
        ms = time_graph(g, iters, warmup)
    return {"layer": label, "ms": ms, "bytes": bytes_moved, "gbs": bytes_moved / ms / 1e6}


def membound(iters, warmup):
    """Pooling, element-wise, softmax, slice/concat and layout kernels at benchmark-sized tensors (all HBM bound)."""
    out = []
    b = 64
    for hw, c in ((224, 64), (112, 128), (56, 256)):
        n = b * hw * hw * c * 4
        out.append(single_node(lambda f: dr.Pooling(f[0], "max", [1, 2, 2, 1], [1, 2, 2, 1]), (hw, hw, c), b, n * 1.25,
                               "maxpool 2x2/2 %dx%dx%d batch %d" % (hw, hw, c, b), iters, warmup))
    out.append(single_node(lambda f: dr.Pooling(f[0], "max", [1, 3, 3, 1], [1, 2, 2, 1]), (112, 112, 64), b, b * 112 * 112 * 64 * 4 * 1.25,
                           "maxpool 3x3/2 112x112x64 batch 64", iters, warmup))
    out.append(single_node(lambda f: dr.Pooling(f[0], "average", [1, 14, 14, 1], [1, 14, 14, 1]), (14, 14, 1000), b, b * 196 * 1000 * 4.0,
                           "avgpool 14x14 14x14x1000 batch 64", iters, warmup))
    n = b * 112 * 112 * 128 * 4
    out.append(single_node(lambda f: dr.Add_Scalar(f[0], 1.5), (112, 112, 128), b, 2.0 * n, "add scalar 112x112x128 batch 64", iters, warmup))
    out.append(single_node(lambda f: dr.Add(f[0], f[1]), (112, 112, 128), b, 3.0 * n, "add 112x112x128 batch 64", iters, warmup, feeds=2))
    out.append(single_node(lambda f: dr.Softmax(f[0]), (1, 1, 1000), b, 2.0 * b * 1000 * 4, "softmax 1000 batch 64", iters, warmup))
    out.append(single_node(lambda f: dr.Concat([f[0], f[1]], 2), (56, 56, 64), b, 4.0 * b * 56 * 56 * 64 * 4, "concat(z) 2 x 56x56x64 batch 64", iters, warmup, feeds=2))
    out.append(single_node(lambda f: dr.Slice(f[0], (0, 0, 16), (56, 56, 32)), (56, 56, 64), b, 2.0 * b * 56 * 56 * 32 * 4, "slice 32 of 64 channels 56x56 batch 64", iters, warmup))
    return out


def sweep(iters, warmup):
    out = []
    for cin, hw in ((64, 56), (128, 28), (256, 14)):
        for math, algo in (("fp32", "direct"), ("fp32", "winograd"), ("fp32", "winograd4"), ("tf32", "auto")):
            out.append(conv_layer(cin, cin, hw, 32, 3, math, algo, iters, warmup))
    for math in ("fp32", "tf32"):
        out.append(conv_layer(256, 512, 28, 64, 1, math, "auto", iters, warmup))
    for batch in (1, 8, 64):
        for nin, nout in ((25088, 4096), (4096, 4096), (4096, 1000)):
            out.append(fc_layer(nin, nout, batch, "fp32", iters, warmup))
    return out


def vgg_layers(batch, iters, warmup):
    out = []
    for cin, cout, hw in ((64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56), (256, 512, 28), (512, 512, 28), (512, 512, 14)):
        for math, algo in (("tf32", "tensor"), ("tf32", "tensor_winograd"), ("fp32x3", "tensor"), ("fp32x3", "tensor_winograd"), ("fp32", "winograd"), ("fp32", "winograd4"), ("fp32", "direct")):
            out.append(conv_layer(cin, cout, hw, batch, 3, math, algo, iters, warmup))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["conv", "fc", "sweep", "membound", "vgg"])
    ap.add_argument("dims", nargs="*", type=int)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--math", default="tf32")
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    if a.what == "conv":
        cin, cout, hw, batch = a.dims
        res = [conv_layer(cin, cout, hw, batch, a.k, a.math, a.algo, a.iters, a.warmup)]
    elif a.what == "fc":
        nin, nout, batch = a.dims
        res = [fc_layer(nin, nout, batch, a.math, a.iters, a.warmup)]
    elif a.what == "membound":
        res = membound(a.iters, a.warmup)
    elif a.what == "vgg":
        res = vgg_layers(a.dims[0] if a.dims else 64, a.iters, a.warmup)
    else:
        res = sweep(a.iters, a.warmup)
    for r in res:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
