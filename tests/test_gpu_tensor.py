"""GPU parity tests of the tensor-core (tcgen05, TF32) convolution path against the CPU oracle.
Bound: max|err| <= 3e-3 * max|ref| per layer output, and equal softmax top-1 on whole networks."""
import ctypes

import numpy as np
import pytest

import cases
import deepracin_b200 as dr
import nets
import oracle
from gpu_helpers import TOL_TF32, conv_build, rel_err, run_graph

pytestmark = pytest.mark.gpu

TENSOR_SHAPES = [
    # name, n, cin, cout, h, w, k
    ("t_64_56", 2, 64, 64, 56, 56, 3),
    ("t_64_224", 1, 64, 64, 224, 224, 3),
    ("t_128_112", 1, 64, 128, 112, 112, 3),
    ("t_256_28", 3, 128, 256, 28, 28, 3),
    ("t_512_14", 5, 256, 512, 14, 14, 3),
    ("t_odd_30x20", 2, 32, 64, 20, 30, 3),
    ("t_odd_13x17", 3, 64, 192, 17, 13, 3),
    ("t_1x1_256_512", 2, 256, 512, 28, 28, 1),
    ("t_1x1_odd", 3, 32, 64, 9, 7, 1),
    ("t_1x1_1000", 2, 512, 1000, 14, 14, 1),         # Cout not a multiple of the N tile: zero-filled filter rows, masked stores
    ("t_3x3_cout_72", 2, 32, 72, 28, 28, 3),
    ("t_1x1_squeeze_16", 2, 64, 16, 56, 56, 1),      # SqueezeNet squeeze layers: fewer output channels than any N tile
    ("t_1x1_squeeze_48", 3, 256, 48, 14, 14, 1),
    ("t_3x3_cout_16", 1, 32, 16, 28, 28, 3),
    ("t_3x3_cin_16", 2, 16, 64, 56, 56, 3),          # channel counts that do not fill a 32-channel slab: zero-filled tail
    ("t_3x3_cin_48", 2, 48, 192, 14, 14, 3),
    ("t_1x1_cin_16", 2, 16, 64, 56, 56, 1),
    ("t_3x3_cin_8", 1, 8, 32, 20, 28, 3),
    ("t_3x3_cin_40_swap", 1, 40, 64, 32, 28, 3),
    ("t_3x3_cout_48_swap", 1, 64, 48, 28, 32, 3),
    ("t_3x3_cout_200", 1, 64, 200, 14, 14, 3),
    ("t_pair_odd_h", 2, 32, 48, 61, 28, 3),          # Cout <= 64: two output rows per MMA; odd height, idle channel rows
    ("t_pair_cin16", 1, 16, 64, 56, 56, 3),
    ("t_pair_cout32", 3, 64, 32, 32, 42, 3),
    ("t_first_rgb", 2, 3, 64, 40, 36, 3),            # few input channels: patch operand gathered by producer warps
    ("t_first_rgb_224", 1, 3, 64, 224, 224, 3),
    ("t_first_c1", 3, 1, 32, 17, 13, 3),             # pixel count not a multiple of the 256-pixel tile
    ("t_first_c4", 2, 4, 128, 20, 24, 3),            # K = 36: two swizzle slabs
    ("t_first_c2_48", 1, 2, 48, 15, 15, 3),
    ("t_first_c4_cout64", 1, 4, 64, 10, 12, 3),      # two K slabs and only two of the four TMEM lane quarters in use
    ("t_first_c3_cout128", 1, 3, 128, 9, 9, 3),
    ("t_pair_w15", 2, 24, 40, 34, 15, 3),            # image one pixel wider than a 14-pixel block: a second, nearly empty block column
    # enough images for a tile per SM: the planner then takes the transposed kernel with the geometry that fills best
    ("t_swap_p30", 40, 8, 128, 56, 56, 3),           # 28 x 8-pixel tiles at a 30-pixel pitch, N = 240
    ("t_swap_p16_th14", 40, 8, 256, 28, 28, 3),      # 14 x 14-pixel tiles, N = 224, two channel blocks per pixel tile
    ("t_swap_14x14", 160, 8, 192, 14, 14, 3),        # one image per tile
    ("t_swap_odd", 40, 8, 136, 29, 27, 3),           # odd width and height, channel count that does not fill the last block
    ("t_pair_p30", 6, 16, 64, 56, 56, 3),            # row-pair kernel at the 30-pixel pitch
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,k", TENSOR_SHAPES)
@pytest.mark.parametrize("act,bias", [(1, True), (0, False)])
def test_tensor_conv_matches_oracle(name, n, cin, cout, h, w, k, act, bias):
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, k, bias)
    ref = oracle.conv2d(x, wt, b, (1, 1), act)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = n
        g.math = "tf32"
        f = dr.feed_node(g, [cin, h, w])
        o = conv_build(wt, b, 1, act)(g, [f])
        dr.mark_as_output(o)
        dr.prepare(g)
        assert dr.lib.dR_getConvAlgo(o.ptr) == 4 and dr.lib.dR_getConvTensor(o.ptr) == 1
        dr.feed_data(f, x)
        got = dr.apply(g)[0].reshape(ref.shape)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert rel_err(got, ref) <= TOL_TF32


def test_tensor_path_falls_back_where_it_cannot_tile():
    """Few input channels with more than 128 filters, 5x5 filters and strided layers stay on the FP32 kernels."""
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.math = "tf32"
        f = dr.feed_node(g, [3, 16, 16])
        z = np.zeros
        a = dr.Conv2d(f, [3, 3, 3, 192], [1, 1, 1, 1], "relu", z((3, 3, 3, 192), np.float32), None)
        b = dr.Conv2d(a, [3, 3, 192, 64], [1, 1, 1, 1], "relu", z((3, 3, 192, 64), np.float32), None)
        c = dr.Conv2d(b, [5, 5, 64, 64], [1, 1, 1, 1], "relu", z((5, 5, 64, 64), np.float32), None)
        d = dr.Conv2d(c, [3, 3, 64, 64], [1, 2, 2, 1], "relu", z((3, 3, 64, 64), np.float32), None)
        dr.mark_as_output(d)
        dr.prepare(g)
        assert [dr.lib.dR_getConvAlgo(n.ptr) for n in (a, b, c, d)] == [1, 4, 1, 1]


def test_tf32_network_agrees_with_fp32_on_top1():
    imgs = nets.synthetic_images("tf32_net", 4, 64)
    outs = {}
    for math in ("fp32", "tf32"):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 4
            g.math = math
            x, out = nets.vgg16(g, size=64, width_div=2, fc_dims=(1024, 1024, 200))
            dr.mark_as_output(out)
            dr.prepare(g)
            dr.feed_data(x, imgs)
            outs[math] = dr.apply(g)[0].reshape(4, -1)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert np.array_equal(outs["fp32"].argmax(1), outs["tf32"].argmax(1))
    assert rel_err(outs["tf32"], outs["fp32"]) <= 2e-2     # probabilities after 16 TF32 layers


@pytest.mark.parametrize("n,cin,cout,h,w", [(1, 64, 64, 56, 56), (2, 128, 256, 28, 28), (3, 256, 512, 14, 14), (2, 32, 64, 12, 20), (1, 64, 64, 224, 224), (2, 32, 48, 28, 30), (3, 64, 32, 64, 28), (2, 16, 16, 32, 28), (1, 128, 128, 16, 46),
                                            (40, 8, 128, 56, 56), (40, 8, 256, 28, 28), (160, 8, 192, 14, 14), (6, 16, 64, 56, 56), (40, 8, 72, 30, 26)])
def test_conv_with_fused_maxpool_matches_oracle(n, cin, cout, h, w):
    """conv3x3 + ReLU followed by 2x2/2 max pooling: the tensor kernel's epilogue stores the pooled tensor."""
    x, wt, b = cases.conv_case("fusedpool_%d_%d" % (cin, h), n, cin, cout, h, w, 3, True)
    ref = oracle.pool(oracle.conv2d(x, wt, b, (1, 1), 1), (2, 2, 1), (2, 2, 1), 0)
    res = {}
    for fuse in (True, False):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.math = "tf32"
            g.fuse = fuse
            f = dr.feed_node(g, [cin, h, w])
            c = conv_build(wt, b, 1, 1)(g, [f])
            o = dr.Pooling(c, "max", [1, 2, 2, 1], [1, 2, 2, 1])
            dr.mark_as_output(o)
            dr.prepare(g)
            dr.feed_data(f, x)
            res[fuse] = dr.apply(g)[0].reshape(ref.shape)
            assert dr.lib.dR_getLaunchCount(g.ptr) == (3 if fuse else 4)     # feed layout, conv(+pool), [pool], output layout
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert rel_err(res[True], ref) <= TOL_TF32
    assert np.array_equal(res[True], res[False])        # same accumulators, max commutes with bias + ReLU


@pytest.mark.parametrize("kind", ["max", "average"])
@pytest.mark.parametrize("n,cin,cout,h,w,act", [(2, 3, 64, 20, 24, 1), (1, 3, 64, 224, 224, 1), (3, 1, 32, 6, 10, 0), (2, 2, 48, 18, 14, 1)])
def test_first_layer_with_fused_pool_matches_oracle(kind, n, cin, cout, h, w, act):
    """Few-channel first layer followed by 2x2/2 max or average pooling (SqueezeNet reference graph: conv1 -> average pool):
    the two rows of a window sit in different TMEM lane quarters and meet through the shared-memory exchange."""
    x, wt, b = cases.conv_case("firstpool_%d_%d_%s" % (cin, h, kind), n, cin, cout, h, w, 3, True)
    ref = oracle.pool(oracle.conv2d(x, wt, b, (1, 1), act), (2, 2, 1), (2, 2, 1), 0 if kind == "max" else 1)
    res, launches = {}, {}
    for fuse in (True, False):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.math = "tf32"
            g.fuse = fuse
            f = dr.feed_node(g, [cin, h, w])
            c = conv_build(wt, b, 1, act)(g, [f])
            o = dr.Pooling(c, kind, [1, 2, 2, 1], [1, 2, 2, 1])
            dr.mark_as_output(o)
            dr.prepare(g)
            assert dr.lib.dR_getConvAlgo(c.ptr) == 4
            dr.feed_data(f, x)
            res[fuse] = dr.apply(g)[0].reshape(ref.shape)
            launches[fuse] = dr.lib.dR_getLaunchCount(g.ptr)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert launches[False] - launches[True] == 1        # the pooling node launches nothing when fused
    assert rel_err(res[True], ref) <= TOL_TF32
    assert rel_err(res[True], res[False]) <= 1e-6       # same accumulators; the average sums in a different order


@pytest.mark.parametrize("ops", [("sub", "sub", "sub"), ("add", "mul", None)])
def test_first_layer_reads_through_preamble_channel_map(ops):
    """Slice -> scalar op -> Concat in front of a few-channel first layer (mean subtraction + BGR reordering of the reference's
    example graphs): in TF32 mode the convolution's gather evaluates it and the preamble launches nothing."""
    n, h, w, cout = 2, 22, 26, 32
    x, wt, b = cases.conv_case("premap_%s" % ops[1], n, 3, cout, h, w, 3, True)
    x = x * np.float32(40.0)
    scal = (np.float32(103.9), np.float32(1.7), np.float32(123.6))
    order = (2, 0, 1)
    planes = []
    for j, c in enumerate(order):
        v = x[:, c:c + 1]
        if ops[j] == "sub": v = v - scal[j]
        elif ops[j] == "add": v = v + scal[j]
        elif ops[j] == "mul": v = v * scal[j]
        planes.append(v.astype(np.float32))
    ref = oracle.conv2d(np.concatenate(planes, axis=1), wt, b, (1, 1), 1)
    res, launches = {}, {}
    for fuse in (True, False):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.math = "tf32"
            g.fuse = fuse
            f = dr.feed_node(g, [3, h, w])
            parts = []
            for j, c in enumerate(order):
                nd = dr.Slice(f, (c, 0, 0), (1, h, w))
                if ops[j] == "sub": nd = dr.Sub_Scalar(nd, float(scal[j]))
                elif ops[j] == "add": nd = dr.Add_Scalar(nd, float(scal[j]))
                elif ops[j] == "mul": nd = dr.Mul_Scalar(nd, float(scal[j]))
                parts.append(nd)
            cat = dr.Concat(parts, 0)
            o = conv_build(wt, b, 1, 1)(g, [cat])
            dr.mark_as_output(o)
            dr.prepare(g)
            dr.feed_data(f, x)
            res[fuse] = dr.apply(g)[0].reshape(ref.shape)
            launches[fuse] = dr.lib.dR_getLaunchCount(g.ptr)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert launches[True] == 3                          # feed layout, convolution, output layout
    assert rel_err(res[True], ref) <= TOL_TF32
    assert rel_err(res[False], ref) <= TOL_TF32
    assert rel_err(res[True], res[False]) <= 1e-6


@pytest.mark.parametrize("n,c,h,w,nout,act", [(64, 64, 4, 4, 256, 1), (16, 512, 7, 7, 512, 0), (33, 32, 2, 8, 768, 1), (64, 256, 2, 2, 1000, 0), (20, 64, 2, 2, 72, 1)])
def test_tensor_fc_matches_oracle(n, c, h, w, nout, act):
    """TF32 mode, batch >= 16: fully connected layers run as a split-K GEMM on the tensor cores."""
    x, wt, b = cases.fc_case("tfc_%d_%d" % (c * h * w, nout), n, c, h, w, nout, True)
    ref = oracle.fc(x, wt, b, act)
    (got,) = run_graph(lambda g, f: dr.Fully_Connected(f[0], [c * h * w, nout], "relu" if act else "linear", wt, b), [x], math="tf32")
    assert rel_err(got, ref) <= TOL_TF32
    (exact,) = run_graph(lambda g, f: dr.Fully_Connected(f[0], [c * h * w, nout], "relu" if act else "linear", wt, b), [x], math="fp32")
    assert rel_err(exact, ref) <= 1e-4
    assert not np.array_equal(got, exact)       # the two arithmetic classes really are different kernels
    # the FP32-accurate tensor mode: the same GEMM with three-pass products, at the FP32 class's bound
    (x3,) = run_graph(lambda g, f: dr.Fully_Connected(f[0], [c * h * w, nout], "relu" if act else "linear", wt, b), [x], math="fp32x3")
    err = rel_err(x3, ref)
    print("fp32x3 fc %d->%d batch %d: %.2e" % (c * h * w, nout, n, err))
    assert err <= 2e-5
    assert not np.array_equal(x3, exact) and not np.array_equal(x3, got)


def _random_shapes(count, seed):
    r = np.random.Generator(np.random.PCG64(seed))
    out = []
    for i in range(count):
        k = 3 if r.random() < 0.7 else 1
        cin = int(r.choice([1, 2, 3, 4])) if (k == 3 and r.random() < 0.2) else 4 * int(r.integers(2, 25))
        cout = 4 * int(r.integers(4, 70))
        if cin <= 4 and cout > 128:
            cout = 4 * int(r.integers(4, 33))
        h, w = int(r.integers(3, 64)), int(r.integers(3, 64))
        n = int(r.integers(1, 4))
        pool = bool(k == 3 and r.random() < 0.4)
        if pool:
            h += h & 1
            w += w & 1
        out.append((i, n, cin, cout, h, w, k, pool))
    return out


@pytest.mark.parametrize("idx,n,cin,cout,h,w,k,pool", _random_shapes(40, 20251))
def test_random_layer_shapes_match_oracle(idx, n, cin, cout, h, w, k, pool):
    """Seeded random layer shapes across the boundaries between the tensor kernels (first layer, row pair, transposed, halo,
    plain, flat 1x1), with and without a following 2x2 max pool, bias + ReLU: every one must match the oracle."""
    x, wt, b = cases.conv_case("rnd_%d" % idx, n, cin, cout, h, w, k, True)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    if pool:
        ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = n
        g.math = "tf32"
        f = dr.feed_node(g, [cin, h, w])
        o = conv_build(wt, b, 1, 1)(g, [f])
        if pool:
            o = dr.Pooling(o, "max", [1, 2, 2, 1], [1, 2, 2, 1])
        dr.mark_as_output(o)
        dr.prepare(g)
        dr.feed_data(f, x)
        got = dr.apply(g)[0].reshape(ref.shape)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert rel_err(got, ref) <= TOL_TF32


TENSOR_WINOGRAD_SHAPES = [
    # name, n, cin, cout, h, w
    ("tw_32_64_20x30", 2, 32, 64, 20, 30),
    ("tw_odd_13x17", 3, 64, 192, 17, 13),             # odd width and height: ragged 2x2 output tiles
    ("tw_16_16", 2, 16, 16, 12, 12),                  # channel counts below one 32-channel slab
    ("tw_8_24_9x11", 1, 8, 24, 11, 9),
    ("tw_48_72", 2, 48, 72, 28, 28),
    ("tw_conv5", 64, 512, 512, 14, 14),               # the benchmark's 14x14 layers at batch 64
    ("tw_conv4", 16, 256, 512, 28, 28),
    ("tw_chunked", 23, 64, 64, 224, 224),             # more transform-domain data than the scratch cap: two full image chunks and a tail
]


@pytest.mark.parametrize("name,n,cin,cout,h,w", TENSOR_WINOGRAD_SHAPES)
def test_tensor_core_winograd_matches_oracle(name, n, cin, cout, h, w):
    """Winograd F(2x2,3x3) with the sixteen transform-domain GEMMs on the tensor cores (TF32 operands): same bound as the direct
    tensor kernels, against the CPU oracle on the first and last image and against the exact-FP32 Winograd kernels on all."""
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, 3, True)
    res = {}
    for math, algo in (("tf32", "tensor_winograd"), ("fp32", "winograd")):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.math = math
            f = dr.feed_node(g, [cin, h, w])
            o = conv_build(wt, b, 1, 1, algo=algo)(g, [f])
            dr.mark_as_output(o)
            dr.prepare(g)
            assert dr.lib.dR_getConvAlgo(o.ptr) == dr.CONV_ALGO[algo]
            dr.feed_data(f, x)
            res[math] = dr.apply(g)[0].reshape(n, cout, h, w)
            again = dr.apply(g)[0].reshape(n, cout, h, w)
            assert np.array_equal(res[math], again)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    for i in (0, n - 1):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        assert rel_err(res["tf32"][i:i + 1], ref) <= TOL_TF32
        assert rel_err(res["fp32"][i:i + 1], ref) <= 1e-4
    num = max(float(np.max(np.abs(res["tf32"][i] - res["fp32"][i]))) for i in range(n))
    assert num / float(np.max(np.abs(res["fp32"]))) <= TOL_TF32


@pytest.mark.parametrize("math,tol", [("tf32", TOL_TF32), ("fp32x3", 1e-4)])
def test_autotuner_may_choose_among_the_tensor_variants(math, tol):
    """Tensor modes with autotuning: every family that can evaluate the layer in the mode's error class is timed (TF32: the direct
    tensor kernel and tensor-core Winograd; FP32-accurate mode: the direct three-pass kernel, Winograd F(4x4,3x3) with three-pass
    products and the FFMA kernels); whichever wins, the result holds at the mode's bound."""
    x, wt, b = cases.conv_case("tw_autotune", 8, 128, 128, 28, 28, 3, True)
    ref = oracle.conv2d(x[:1], wt, b, (1, 1), 1)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = 8
        g.math = math
        g.autotune = True
        f = dr.feed_node(g, [128, 28, 28])
        o = conv_build(wt, b, 1, 1)(g, [f])
        dr.mark_as_output(o)
        dr.prepare(g)
        chosen = dr.lib.dR_getConvAlgo(o.ptr)
        if math == "tf32":
            assert chosen in (dr.CONV_ALGO["tensor"], dr.CONV_ALGO["tensor_winograd"])
        else:
            assert chosen in (dr.CONV_ALGO["tensor"], dr.CONV_ALGO["tensor_winograd"], dr.CONV_ALGO["winograd4"], dr.CONV_ALGO["winograd"], dr.CONV_ALGO["direct"])
        dr.feed_data(f, x)
        got = dr.apply(g)[0].reshape(8, 128, 28, 28)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert rel_err(got[:1], ref) <= tol


X3_SHAPES = [
    # name, n, cin, cout, h, w, pool
    ("x3_32_64_20x30", 2, 32, 64, 20, 30, False),
    ("x3_odd_13x17", 3, 64, 192, 17, 13, False),
    ("x3_swap_odd", 40, 8, 136, 29, 27, False),            # odd image, Cout ends inside a warp, one zero-filled K slab
    ("x3_16_16", 2, 16, 16, 12, 12, False),
    ("x3_48_72_pool", 2, 48, 72, 28, 30, True),
    ("x3_pool_p30", 6, 16, 64, 56, 56, True),
    ("x3_conv3_2", 40, 256, 256, 56, 56, False),           # the benchmark's geometries at full depth
    ("x3_conv5_pool", 64, 512, 512, 14, 14, True),
    ("x3_conv1_2", 4, 64, 64, 224, 224, True),
    ("x3_w15", 2, 24, 40, 34, 15, False),                   # too narrow for the row-pair blocks: transposed kernel; Cin not a multiple of 32
    ("x3_pair_odd_h", 2, 32, 48, 61, 28, False),
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,pool", X3_SHAPES)
def test_fp32_accurate_tensor_conv_matches_oracle_at_the_fp32_bound(name, n, cin, cout, h, w, pool):
    """math = 'fp32x3': 3x3 layers on the tensor cores with every product split into high and low TF32 parts (three passes).
    The bound is the exact-FP32 kernels' 1e-4 * max|ref|, thirty times tighter than the TF32 class."""
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, 3, True)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = n
        g.math = "fp32x3"
        f = dr.feed_node(g, [cin, h, w])
        c = conv_build(wt, b, 1, 1, algo="tensor")(g, [f])     # the direct three-pass kernel (from 64 channels up the rule prefers Winograd)
        o = dr.Pooling(c, "max", [1, 2, 2, 1], [1, 2, 2, 1]) if pool else c
        dr.mark_as_output(o)
        dr.prepare(g)
        assert dr.lib.dR_getConvAlgo(c.ptr) == dr.CONV_ALGO["tensor"] and dr.lib.dR_getConvTensor(c.ptr) == 2
        dr.feed_data(f, x)
        got = dr.apply(g)[0]
        launches = dr.lib.dR_getLaunchCount(g.ptr)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
        geom = (ctypes.c_int * 4)()
        kernel = dr.lib.dR_getConvTensorKernel(c.ptr, geom)
        # at most 64 output channels on an image that suits its blocks: the row-pair kernel in three-pass mode (5); else the transposed kernel (4)
        assert kernel == (5 if name in ("x3_pool_p30", "x3_conv1_2", "x3_pair_odd_h") else 4), (name, kernel, list(geom))
    ho, wo = (h // 2, w // 2) if pool else (h, w)
    got = got.reshape(n, cout, ho, wo)
    assert launches == 3                                # feed layout, convolution (+ pool in its epilogue), output layout
    worst = 0.0
    for i in sorted({0, n // 2, n - 1}):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        if pool:
            ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)
        worst = max(worst, rel_err(got[i:i + 1], ref))
    print("fp32x3 %s: max rel err %.2e" % (name, worst))
    # What is left is the tensor core's accumulator rounding (it truncates), which grows with the number of MMAs per output:
    # ~5e-6 at K = 9 * 32, ~5e-5 at K = 9 * 512.  An operand split that is off would show as ~1e-3 (the TF32 class's error).
    assert worst <= 6e-5


X3_WINOGRAD_SHAPES = [
    # name, n, cin, cout, h, w, pool, forced (None: the mode's static rule picks it)
    ("x3w_64_64_30x34", 2, 64, 64, 30, 34, False, "tensor_winograd"),        # shallower than the rule's threshold: forced
    ("x3w_64_192_13x17", 3, 64, 192, 17, 13, False, "tensor_winograd"),      # ragged 4x4 tiles
    ("x3w_128_256_pool", 2, 128, 256, 28, 28, True, None),
    ("x3w_32_48", 2, 32, 48, 20, 22, False, "tensor_winograd"),
    ("x3w_conv3_2", 40, 256, 256, 56, 56, False, None),              # the benchmark's layers at full depth
    ("x3w_conv4_pool", 16, 512, 512, 28, 28, True, None),
    ("x3w_conv5_pool", 64, 512, 512, 14, 14, True, None),
    ("x3w_conv1_2", 4, 64, 64, 224, 224, True, "tensor_winograd"),
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,pool,forced", X3_WINOGRAD_SHAPES)
def test_fp32_accurate_tensor_winograd_matches_oracle_at_the_fp32_bound(name, n, cin, cout, h, w, pool, forced):
    """math = 'fp32x3', Winograd F(4x4,3x3) with its 36 products on the tensor cores as three TF32 passes each (operands stored as
    high | low halves): a quarter of the direct multiplications, FP32-class error bound."""
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, 3, True)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = n
        g.math = "fp32x3"
        f = dr.feed_node(g, [cin, h, w])
        c = conv_build(wt, b, 1, 1, algo=forced)(g, [f])
        o = dr.Pooling(c, "max", [1, 2, 2, 1], [1, 2, 2, 1]) if pool else c
        dr.mark_as_output(o)
        dr.prepare(g)
        assert dr.lib.dR_getConvAlgo(c.ptr) == dr.CONV_ALGO["tensor_winograd"] and dr.lib.dR_getConvTensor(c.ptr) == 2
        dr.feed_data(f, x)
        got = dr.apply(g)[0]
        launches = dr.lib.dR_getLaunchCount(g.ptr)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    ho, wo = (h // 2, w // 2) if pool else (h, w)
    got = got.reshape(n, cout, ho, wo)
    assert launches % 3 == 2 and launches >= 5          # feed layout, (input transform, GEMM, output transform) per image chunk, output layout
    worst = 0.0
    for i in sorted({0, n // 2, n - 1}):
        ref = oracle.conv2d(x[i:i + 1], wt, b, (1, 1), 1)
        if pool:
            ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)
        worst = max(worst, rel_err(got[i:i + 1], ref))
    print("fp32x3 winograd %s: max rel err %.2e" % (name, worst))
    assert worst <= 1e-4


def test_fp32_accurate_tensor_mode_on_a_whole_network():
    """VGG-style network in 'fp32x3' mode: 3x3 layers with >= 8 input channels on the tensor cores, first layer / FC / pooling /
    softmax on the FP32 kernels; probabilities against the exact-FP32 run at the FP32 class's whole-network bound."""
    imgs = nets.synthetic_images("x3_net", 4, 64)
    outs, tensor_layers = {}, {}
    for math in ("fp32", "fp32x3"):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 4
            g.math = math
            x, out = nets.vgg16(g, size=64, width_div=2, fc_dims=(1024, 1024, 200))
            dr.mark_as_output(out)
            dr.prepare(g)
            dr.feed_data(x, imgs)
            outs[math] = dr.apply(g)[0].reshape(4, -1)
            tensor_layers[math] = [dr.lib.dR_getConvTensor(nd.ptr) for nd in g.nodes if nd.desc == "Conv2D"]
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert tensor_layers["fp32"] == [0] * 13
    assert tensor_layers["fp32x3"] == [0] + [2] * 12
    assert np.array_equal(outs["fp32"].argmax(1), outs["fp32x3"].argmax(1))
    assert rel_err(outs["fp32x3"], outs["fp32"]) <= 5e-4


@pytest.mark.parametrize("s,e,hw,n", [(16, 64, 28, 4), (32, 128, 14, 3), (48, 192, 14, 70), (16, 24, 11, 2)])
def test_fire_expand_pair_runs_as_one_layer(s, e, hw, n):
    """Fire module in TF32 mode: the 1x1 and 3x3 expand convolutions of one squeezed tensor, concatenated along channels, are one
    3x3 launch (the 1x1 filters sit on the centre tap): one kernel less than without fusion, same results as the oracle's two
    convolutions, and the same as the unfused graph within TF32 rounding order."""
    x, w1, b1 = cases.conv_case("fire_e1_%d" % e, n, s, e, hw, hw, 1, True)
    _, w3, b3 = cases.conv_case("fire_e3_%d" % e, 1, s, e, hw, hw, 3, True)
    ref = np.concatenate([oracle.conv2d(x[:2], w1, b1, (1, 1), 1), oracle.conv2d(x[:2], w3, b3, (1, 1), 1)], axis=1)
    res, launches = {}, {}
    for fuse in (True, False):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.math = "tf32"
            g.fuse = fuse
            f = dr.feed_node(g, [s, hw, hw])
            e1 = conv_build(w1, b1, 1, 1)(g, [f])
            e3 = conv_build(w3, b3, 1, 1)(g, [f])
            cat = dr.Concat([e1, e3], 0)
            dr.mark_as_output(cat)
            dr.prepare(g)
            dr.feed_data(f, x)
            res[fuse] = dr.apply(g)[0].reshape(n, 2 * e, hw, hw)
            launches[fuse] = dr.lib.dR_getLaunchCount(g.ptr)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert launches[True] == 3                          # feed layout, ONE convolution, output layout
    assert launches[False] == 6                         # feed layout, two convolutions, two concat placements, output layout
    assert rel_err(res[True][:2], ref) <= TOL_TF32
    assert rel_err(res[False][:2], ref) <= TOL_TF32
    assert rel_err(res[True], res[False]) <= 1e-6 * 50  # same TF32 products; the accumulation order of the centre tap differs
