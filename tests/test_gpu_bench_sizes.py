"""GPU parity tests at the benchmark's own sizes: the kernels, block geometries, batch sizes and channel depths that
``bench.py`` times (VGG-16 at batch 64 in both arithmetic classes, the conv sweep at batch 32, the 1x1 / fully connected
microbenchmark shapes at batch 64).  Every test asserts which tensor-core kernel and geometry its launches ran, so that a
planner change cannot silently move the benchmark onto an unchecked combination.

Bounds: exact-FP32 kernels max|err| <= 1e-4 * max|ref| per layer, TF32 tensor-core kernels 3e-3 * max|ref| per layer,
equal softmax top-1.  The CPU oracle evaluates single images / rows (it needs ~0.4 s per 3.7 GFLOP image)."""
import ctypes

import numpy as np
import pytest

import cases
import deepracin_b200 as dr
import nets
import oracle
from gpu_helpers import TOL_FP32, TOL_TF32, conv_build, rel_err

pytestmark = pytest.mark.gpu

FLAT, PLAIN, HALO, SWAP, PAIR, FIRST = 1, 2, 3, 4, 5, 6


def tensor_kernel(node):
    geom = (ctypes.c_int * 4)()
    v = dr.lib.dR_getConvTensorKernel(node.ptr, geom)
    return (v,) + tuple(geom)


def nchw(a, n):
    """HWC-interface output [n, H, W, C] (or squeezed) -> [n, C, H, W]"""
    a = a.reshape((n,) + a.shape[-3:]) if a.ndim >= 3 else a
    return np.ascontiguousarray(a.transpose(0, 3, 1, 2))


def max_rel(got, ref):
    """rel_err without float64 copies of GB-sized tensors"""
    assert got.shape == ref.shape
    num = den = 0.0
    for i in range(got.shape[0]):
        num = max(num, float(np.max(np.abs(got[i] - ref[i]))))
        den = max(den, float(np.max(np.abs(ref[i]))))
    return num / max(den, 1e-30)


def run_layer(x, wt, b, math, pool=False, act=1):
    """One convolution (+ optional 2x2/2 max pool) at x's batch size; returns ([n, C, H, W] result, kernel description)."""
    n, cin, h, w = x.shape
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = n
        g.math = math
        f = dr.feed_node(g, [cin, h, w])
        c = conv_build(wt, b, 1, act)(g, [f])
        o = dr.Pooling(c, "max", [1, 2, 2, 1], [1, 2, 2, 1]) if pool else c
        dr.mark_as_output(o)
        dr.prepare(g)
        dr.feed_data(f, x)
        got = dr.apply(g)[0]
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
        kern = tensor_kernel(c)
    ho, wo = (h // 2, w // 2) if pool else (h, w)
    return got.reshape(n, wt.shape[1], ho, wo), kern


DEEP_LAYERS = [
    # name, n, cin, cout, hw, pool, expected kernel of the TF32 run
    ("conv3_2_p30", 40, 256, 256, 56, False, (SWAP, 30, 28, 8, 240)),        # 8 K slabs, 2 channel blocks per pixel tile
    ("conv3_3_p30_pool", 40, 256, 256, 56, True, (SWAP, 30, 28, 8, 240)),
    ("conv4_2_14x14", 64, 512, 512, 28, False, (SWAP, 16, 14, 14, 224)),     # 16 K slabs, 4 channel blocks
    ("conv4_3_14x14_pool", 64, 512, 512, 28, True, (SWAP, 16, 14, 14, 224)),
    ("conv5_1_14x14", 64, 512, 512, 14, False, (SWAP, 16, 14, 14, 224)),     # one image per tile
    ("conv5_3_14x14_pool", 64, 512, 512, 14, True, (SWAP, 16, 14, 14, 224)),
    ("conv2_2_p30_pool", 16, 128, 128, 112, True, (SWAP, 30, 28, 8, 240)),
    ("conv1_2_pair", 8, 64, 64, 224, False, (PAIR, 30, 28, 8, 240)),         # two output rows per MMA at the 30-pixel pitch
    ("conv1_2_pair_pool", 8, 64, 64, 224, True, (PAIR, 30, 28, 8, 240)),
    ("conv4_1_14x14", 64, 256, 512, 28, False, (SWAP, 16, 14, 14, 224)),     # Cin = Cout / 2
]


@pytest.mark.parametrize("name,n,cin,cout,hw,pool,kernel", DEEP_LAYERS)
def test_deep_layers_on_the_benchmark_geometries(name, n, cin, cout, hw, pool, kernel):
    """Full-depth VGG layers at batch sizes where the planner takes the benchmark's kernel and geometry: TF32 against the
    exact-FP32 kernels over the whole batch, both against the CPU oracle on the first and last image."""
    x, wt, b = cases.conv_case("deep_" + name, n, cin, cout, hw, hw, 3, True)
    tf, kern = run_layer(x, wt, b, "tf32", pool)
    assert kern == kernel
    fp, kfp = run_layer(x, wt, b, "fp32", pool)
    assert kfp[0] == 0
    assert max_rel(tf, fp) <= TOL_TF32
    for i in (0, n - 1):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        if pool:
            ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)
        assert rel_err(fp[i:i + 1], ref) <= TOL_FP32
        assert rel_err(tf[i:i + 1], ref) <= TOL_TF32


def vgg_outputs(math, imgs, which):
    """VGG-16 at imgs' batch size with the nodes named in `which` marked as outputs (at most 10: the reference's cap of
    dR_getOutputBuffers).  Names: convI_J, poolI, fc6..8, prob.  Only nodes whose marking leaves the fusion plan of the
    benchmark untouched may be named: a convolution in front of a pool is evaluated together with it, so its own tensor
    never exists there.  Returns {name: [n, C, H, W] array}, {conv name: kernel description}."""
    n = imgs.shape[0]
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = n
        g.math = math
        x, out = nets.vgg16(g, size=224)
        names, block, idx, fc = {}, 1, 0, 6
        for node in g.nodes[1:]:
            if node.desc == "Conv2D":
                idx += 1
                names["conv%d_%d" % (block, idx)] = node
            elif node.desc == "Pooling":
                names["pool%d" % block] = node
                block, idx = block + 1, 0
            elif node.desc == "FullyConnected":
                names["fc%d" % fc] = node
                fc += 1
            else:
                names["prob"] = node
        assert len(which) <= 10
        for k in which:
            dr.mark_as_output(names[k])
        dr.prepare(g)
        dr.feed_data(x, imgs)
        res = dr.apply(g)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
        kernels = {k: tensor_kernel(v) for k, v in names.items() if k.startswith("conv")}
        launches = dr.lib.dR_getLaunchCount(g.ptr)
    outs = {}
    for k, r in zip(which, res):
        w, h, c = names[k].out_shape
        outs[k] = np.ascontiguousarray(r.reshape(n, h, w, c).transpose(0, 3, 1, 2))
    return outs, kernels, launches


VGG_KERNELS_B64 = {
    "conv1_1": (FIRST, 0, 0, 0, 0), "conv1_2": (PAIR, 30, 28, 8, 240),
    "conv2_1": (SWAP, 30, 28, 8, 240), "conv2_2": (SWAP, 30, 28, 8, 240),
    "conv3_1": (SWAP, 30, 28, 8, 240), "conv3_2": (SWAP, 30, 28, 8, 240), "conv3_3": (SWAP, 30, 28, 8, 240),
    "conv4_1": (SWAP, 16, 14, 14, 224), "conv4_2": (SWAP, 16, 14, 14, 224), "conv4_3": (SWAP, 16, 14, 14, 224),
    "conv5_1": (SWAP, 16, 14, 14, 224), "conv5_2": (SWAP, 16, 14, 14, 224), "conv5_3": (SWAP, 16, 14, 14, 224),
}
# (layer, the tensor it reads, what the oracle applies to that tensor)
VGG_ORACLE_STEPS = [
    ("pool1", "conv1_1", "conv+pool", 1), ("pool2", "conv2_1", "conv+pool", 3), ("conv3_2", "conv3_1", "conv", 5),
    ("conv4_1", "pool3", "conv", 7), ("conv5_1", "pool4", "conv", 10), ("conv5_2", "conv5_1", "conv", 11), ("fc6", "pool5", "fc", 0), ("fc7", "fc6", "fc", 1),
    ("fc8", "fc7", "fc", 2),
]


def test_vgg16_batch64_every_layer_tf32_against_fp32_and_oracle():
    """The benchmark's own run: VGG-16, batch 64.  Every layer output that exists under the benchmark's fusion plan is
    compared between the TF32 tensor-core path and the exact-FP32 path (3e-3 per layer, equal top-1 on all 64 images), and
    single layers of both paths are re-evaluated by the CPU oracle from the path's OWN input of that layer (first and
    last image), which pins each kernel at its benchmark geometry without error accumulated from the layers before it."""
    imgs = nets.synthetic_images("vgg_b64", 64, 224)
    sets = [["conv1_1", "pool1", "conv2_1", "pool2", "conv3_1", "conv3_2", "pool3", "conv4_1"],
            ["conv4_2", "pool4", "conv5_1", "conv5_2", "pool5", "fc6", "fc7", "fc8", "prob"]]
    # the weights the graph builder drew, regenerated in the same order for the oracle
    g = cases.rng("vgg16")
    conv_w, cin = [], 3
    for v in nets.VGG16_CFG:
        if v != "M":
            conv_w.append(nets.he(g, (3, 3, cin, v), 9 * cin))
            cin = v
    fc_w, nin = [], 25088
    for i, nout in enumerate((4096, 4096, 1000)):
        w = nets.he(g, (nin, nout), nin)
        fc_w.append(w * np.float32(0.05) if i == 2 else w)
        nin = nout
    worst = {}
    for which in sets:
        tf, kernels, launches_tf = vgg_outputs("tf32", imgs, which)
        assert kernels == VGG_KERNELS_B64
        fp, kfp, _ = vgg_outputs("fp32", imgs, which)
        assert all(v[0] == 0 for v in kfp.values())
        for k in which:
            worst[k] = max_rel(tf[k], fp[k])
        if "prob" in which:
            assert np.array_equal(tf["prob"].reshape(64, -1).argmax(1), fp["prob"].reshape(64, -1).argmax(1))
        for layer, src, op, wi in VGG_ORACLE_STEPS:
            if layer not in which or src not in which:
                continue
            for path, tol in ((fp, TOL_FP32), (tf, TOL_TF32)):
                for i in (0, 63):
                    xin = path[src][i:i + 1]
                    if op == "fc":
                        ref = oracle.fc(xin.reshape(1, -1, 1, 1) if xin.shape[2] == 1 else xin, fc_w[wi], np.zeros(fc_w[wi].shape[1], np.float32), 0 if wi == 2 else 1)
                        got = path[layer][i:i + 1].reshape(ref.shape)
                    else:
                        ref = oracle.conv2d(xin, np.ascontiguousarray(conv_w[wi].transpose(2, 3, 0, 1)), np.zeros(conv_w[wi].shape[3], np.float32), (1, 1), 1)
                        if op == "conv+pool":
                            ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)
                        got = path[layer][i:i + 1]
                    assert rel_err(got, ref) <= tol, (layer, i, "fp32" if path is fp else "tf32")
    # accumulated over the layers before it, every layer output still sits inside the per-layer TF32 bound; the softmax
    # exponentiates the class scores' differences, so the probabilities get the bound the whole-network tests use
    assert max(v for k, v in worst.items() if k != "prob") <= TOL_TF32, worst
    assert worst["prob"] <= 2e-2, worst


def test_first_layer_at_batch64_against_oracle():
    """conv1_1 (3 -> 64 @ 224x224) at batch 64 on the producer-gather tensor kernel, with and without the preamble."""
    imgs = nets.synthetic_images("first_b64", 64, 224)
    x = np.ascontiguousarray(imgs.transpose(0, 3, 1, 2))
    _, wt, b = cases.conv_case("first_b64_w", 1, 3, 64, 8, 8, 3, True)
    tf, kern = run_layer(x, wt, b, "tf32")
    assert kern[0] == FIRST
    for i in (0, 31, 63):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        assert rel_err(tf[i:i + 1], ref) <= TOL_TF32


@pytest.mark.parametrize("math,tol", [("fp32", TOL_FP32), ("tf32", TOL_TF32)])
def test_1x1_microbenchmark_shape_at_batch64(math, tol):
    """1x1 convolution 28x28x256 -> 512 at batch 64 (flat tensor GEMM in TF32 mode, FFMA GEMM in FP32 mode)."""
    x, wt, b = cases.conv_case("cfg3_1x1", 64, 256, 512, 28, 28, 1, True)
    got, kern = run_layer(x, wt, b, math)
    assert kern[0] == (FLAT if math == "tf32" else 0)
    for i in (0, 63):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        assert rel_err(got[i:i + 1], ref) <= tol


@pytest.mark.parametrize("math,tol", [("fp32", TOL_FP32), ("tf32", TOL_TF32)])
def test_fc_stack_at_batch64(math, tol):
    """FC 25088 -> 4096 -> 4096 -> 1000 at batch 64, ReLU except the last layer; every layer's output against the oracle on
    the first and last row, each layer fed with the path's own previous output."""
    g = cases.rng("cfg3_fc")
    dims = [(25088, 4096), (4096, 4096), (4096, 1000)]
    ws = [g.standard_normal(d, dtype=np.float32) * np.float32(np.sqrt(2.0 / d[0])) for d in dims]
    bs = [g.standard_normal(d[1], dtype=np.float32) * np.float32(0.1) for d in dims]
    x = g.standard_normal((64, 512, 7, 7), dtype=np.float32)
    with dr.Environment() as env:
        gr = env.create_graph("CHW")
        gr.batch = 64
        gr.math = math
        f = dr.feed_node(gr, [512, 7, 7])
        node, outs = f, []
        for i, (d, w, b) in enumerate(zip(dims, ws, bs)):
            node = dr.Fully_Connected(node, list(d), "linear" if i == 2 else "relu", w, b)
            dr.mark_as_output(node)
            outs.append(node)
        dr.prepare(gr)
        dr.feed_data(f, x)
        res = [r.reshape(64, -1) for r in dr.apply(gr)]
        assert dr.lib.dR_getDeviceStatus(gr.ptr) == 0
    prev = x
    for i, (w, b) in enumerate(zip(ws, bs)):
        for row in (0, 63):
            xin = prev[row:row + 1] if i == 0 else prev[row:row + 1].reshape(1, -1, 1, 1)
            ref = oracle.fc(xin, w, b, 0 if i == 2 else 1).reshape(1, -1)
            assert rel_err(res[i][row:row + 1], ref) <= tol, (i, row)
        prev = res[i]


@pytest.mark.parametrize("cin,hw", [(64, 56), (128, 28), (256, 14)])
def test_conv_sweep_at_batch32_tf32(cin, hw):
    """The conv-sweep layers (3x3, stride 1, bias + ReLU) at batch 32 on the tensor cores, against the exact-FP32 kernels over
    the whole batch and the oracle on two images."""
    x, wt, b = cases.conv_case("sweep_tf32_%d" % cin, 32, cin, cin, hw, hw, 3, True)
    tf, kern = run_layer(x, wt, b, "tf32")
    assert kern[0] in (SWAP, PAIR, HALO)
    fp, _ = run_layer(x, wt, b, "fp32")
    assert max_rel(tf, fp) <= TOL_TF32
    for i in (0, 31):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        assert rel_err(fp[i:i + 1], ref) <= TOL_FP32
        assert rel_err(tf[i:i + 1], ref) <= TOL_TF32
