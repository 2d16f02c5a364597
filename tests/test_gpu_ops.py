"""GPU parity tests, one operator per graph, through the C ABI of libdeepracin.so, against the CPU
oracle (plain-C restatement, double accumulation) and against golden vectors produced by the
reference's own kernel sources.  Bound for the exact-FP32 kernels: max|err| <= 1e-4 * max|ref|."""
import os

import numpy as np
import pytest

import cases
import deepracin_b200 as dr
import oracle
from gpu_helpers import TOL_FP32, conv_build, hwio, rel_err, run_graph

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz"))


# ------------------------------------------------------------------ convolution
CONV_SHAPES = [
    # name, n, cin, cout, h, w, k, stride
    ("c3_small", 1, 3, 8, 7, 10, 3, 1),
    ("c3_16", 2, 16, 16, 12, 12, 3, 1),
    ("c3_odd_channels", 1, 5, 6, 9, 13, 3, 1),
    ("c3_first_layer", 2, 3, 64, 17, 23, 3, 1),      # RGB first layer: the few-input-channel kernel
    ("c3_cin4", 1, 4, 32, 9, 10, 3, 1),
    ("c3_cin1", 3, 1, 16, 8, 9, 3, 1),
    ("c3_wide", 3, 32, 72, 17, 19, 3, 1),
    ("c3_deep", 1, 128, 64, 14, 14, 3, 1),
    ("c1_64to16", 2, 64, 16, 20, 20, 1, 1),
    ("c1_odd", 1, 7, 9, 5, 6, 1, 1),
    ("c5", 1, 4, 4, 12, 12, 5, 1),
    ("c7_stride2", 1, 3, 16, 32, 32, 7, 2),
    ("c3_stride2", 2, 8, 12, 15, 16, 3, 2),
    ("c1_stride2", 1, 8, 8, 10, 10, 1, 2),
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,k,stride", CONV_SHAPES)
@pytest.mark.parametrize("act,bias", [(1, True), (0, False)])
def test_conv_direct_matches_oracle(name, n, cin, cout, h, w, k, stride, act, bias):
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, k, bias)
    ref = oracle.conv2d(x, wt, b, (stride, stride), act)
    (got,) = run_graph(conv_build(wt, b, stride, act, algo="direct"), [x])
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("name,n,cin,cout,h,w,k,stride", [c for c in CONV_SHAPES if c[6] == 3 and c[7] == 1])
@pytest.mark.parametrize("act,bias", [(1, True), (0, False)])
def test_conv_winograd_matches_oracle(name, n, cin, cout, h, w, k, stride, act, bias):
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, k, bias)
    ref = oracle.conv2d(x, wt, b, (1, 1), act)
    (got,) = run_graph(conv_build(wt, b, 1, act, algo="winograd"), [x])
    assert rel_err(got, ref) <= TOL_FP32


WINO4_DEEP = [
    # name, n, cin, cout, h, w: depths and edge sizes of the VGG layers (tiles of 4x4 outputs: 14 and 30 leave ragged edges)
    ("w4_64_30", 2, 64, 64, 30, 34),
    ("w4_256_28", 2, 256, 256, 28, 28),
    ("w4_512_14", 3, 512, 512, 14, 14),
    ("w4_128to256_9", 1, 128, 256, 9, 11),
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,k,stride", [c for c in CONV_SHAPES if c[6] == 3 and c[7] == 1])
@pytest.mark.parametrize("act,bias", [(1, True), (0, False)])
def test_conv_winograd4_matches_oracle(name, n, cin, cout, h, w, k, stride, act, bias):
    """F(4x4,3x3): 6x6 tiles, 36 transform-domain GEMMs; same bound as every exact-FP32 kernel."""
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, k, bias)
    ref = oracle.conv2d(x, wt, b, (1, 1), act)
    (got,) = run_graph(conv_build(wt, b, 1, act, algo="winograd4"), [x])
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("name,n,cin,cout,h,w", WINO4_DEEP)
def test_conv_winograd4_deep_layers_stay_inside_the_fp32_bound(name, n, cin, cout, h, w):
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, 3, True)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    (got,) = run_graph(conv_build(wt, b, 1, 1, algo="winograd4"), [x])
    err = rel_err(got, ref)
    print(f"{name}: F(4x4,3x3) error {err:.2e} of max|ref|")
    assert err <= TOL_FP32


def _random_fp32_shapes(count, seed):
    r = np.random.Generator(np.random.PCG64(seed))
    out = []
    for i in range(count):
        k = int(r.choice([1, 3, 3, 3, 5]))
        stride = 2 if (k == 3 and r.random() < 0.15) else 1
        cin = int(r.integers(1, 6)) if r.random() < 0.2 else int(r.integers(8, 97))
        cout = int(r.integers(4, 97))
        h, w = int(r.integers(5, 41)), int(r.integers(5, 41))
        if r.random() < 0.5:
            h, w = h & ~1, w & ~1
        pool = bool(k == 3 and stride == 1 and h % 2 == 0 and w % 2 == 0 and r.random() < 0.4)
        out.append((i, int(r.integers(1, 4)), cin, cout, max(h, 4), max(w, 4), k, stride, pool))
    return out


@pytest.mark.parametrize("idx,n,cin,cout,h,w,k,stride,pool", _random_fp32_shapes(36, 4711))
def test_random_layer_shapes_match_oracle_in_fp32_mode(idx, n, cin, cout, h, w, k, stride, pool):
    """Seeded random layers under the FP32 mode's static rule -- F(4x4,3x3) from 16 channels up (with and without the fused 2x2 max
    pool), F(2x2,3x3) below, the few-channel kernel, the 1x1 GEMM, direct for other filters and strides; odd channel counts take
    the scalar transform paths."""
    x, wt, b = cases.conv_case("rnd32_%d" % idx, n, cin, cout, h, w, k, True)
    ref = oracle.conv2d(x, wt, b, (stride, stride), 1)
    if pool:
        ref = oracle.pool(ref, (2, 2, 1), (2, 2, 1), 0)

    def build(g, f):
        o = conv_build(wt, b, stride, 1)(g, f)
        return dr.Pooling(o, "max", [1, 2, 2, 1], [1, 2, 2, 1]) if pool else o
    (got,) = run_graph(build, [x])
    assert rel_err(got.reshape(ref.shape), ref) <= TOL_FP32


@pytest.mark.parametrize("n,cin,cout,h,w,act", [(2, 32, 32, 12, 16, 1), (3, 64, 128, 14, 14, 1), (1, 16, 48, 30, 26, 0), (2, 128, 64, 28, 28, 1)])
def test_winograd4_with_fused_maxpool_matches_oracle(n, cin, cout, h, w, act):
    """FP32 mode, conv3x3 followed by 2x2/2 max pooling: the F(4x4,3x3) output transform stores the pooled tensor (each 4x4 tile
    holds four whole pooling windows) and the pooling node launches nothing; identical to the unfused pair bit for bit."""
    x, wt, b = cases.conv_case("w4pool_%d_%d" % (cin, h), n, cin, cout, h, w, 3, True)
    ref = oracle.pool(oracle.conv2d(x, wt, b, (1, 1), act), (2, 2, 1), (2, 2, 1), 0)
    res = {}
    for fuse in (True, False):
        with dr.Environment() as env:
            g = env.create_graph("CHW")
            g.batch = n
            g.fuse = fuse
            f = dr.feed_node(g, [cin, h, w])
            c = conv_build(wt, b, 1, act)(g, [f])
            o = dr.Pooling(c, "max", [1, 2, 2, 1], [1, 2, 2, 1])
            dr.mark_as_output(o)
            dr.prepare(g)
            assert dr.lib.dR_getConvAlgo(c.ptr) == dr.CONV_ALGO["winograd4"]
            dr.feed_data(f, x)
            res[fuse] = dr.apply(g)[0].reshape(ref.shape)
            # feed layout, input transform, GEMM, output transform(+pool), [pool], output layout
            assert dr.lib.dR_getLaunchCount(g.ptr) == (5 if fuse else 6)
    assert rel_err(res[True], ref) <= TOL_FP32
    assert np.array_equal(res[True], res[False])


@pytest.mark.parametrize("name", [n for n, (k, _) in cases.GOLDEN_CASES.items() if k in ("wino", "c1x1")])
def test_conv_matches_reference_kernel_golden(name):
    kind, kw = cases.GOLDEN_CASES[name]
    x, wt, b = cases.make_inputs(name)
    algos = (None, "direct", "winograd4") if kind == "wino" else (None, "direct")
    for algo in algos:                  # None: the static rule (3x3 -> Winograd, 1x1 -> 1x1 GEMM)
        (got,) = run_graph(conv_build(wt, b, 1, kw["act"], algo=algo), [x])
        assert rel_err(got, GOLD[name]) <= TOL_FP32


def test_static_variant_rule_follows_the_reference():
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        f = dr.feed_node(g, [8, 12, 12])
        z = np.zeros
        a = dr.Conv2d(f, [3, 3, 8, 8], [1, 1, 1, 1], "relu", z((3, 3, 8, 8), np.float32), None)
        b = dr.Conv2d(a, [1, 1, 8, 8], [1, 1, 1, 1], "relu", z((1, 1, 8, 8), np.float32), None)
        c = dr.Conv2d(b, [3, 3, 8, 8], [1, 2, 2, 1], "relu", z((3, 3, 8, 8), np.float32), None)
        d = dr.Conv2d(c, [5, 5, 8, 8], [1, 1, 1, 1], "relu", z((5, 5, 8, 8), np.float32), None)
        e = dr.Conv2d(d, [3, 3, 8, 32], [1, 1, 1, 1], "relu", z((3, 3, 8, 32), np.float32), None)
        h = dr.Conv2d(e, [3, 3, 32, 16], [1, 1, 1, 1], "relu", z((3, 3, 32, 16), np.float32), None)
        dr.mark_as_output(h)
        dr.prepare(g)
        # the reference's rule; 3x3 stride-1 layers with >= 16 channels on both sides take the F(4x4,3x3) form of Winograd (6)
        assert [dr.lib.dR_getConvAlgo(n.ptr) for n in (a, b, c, d, e, h)] == [2, 3, 1, 1, 2, 6]
        assert [dr.lib.dR_getConvTensor(n.ptr) for n in (a, b, c, d, e, h)] == [0, 0, 0, 0, 0, 0]


def test_autotuned_variants_keep_parity():
    x, wt, b = cases.conv_case("tune", 4, 32, 32, 28, 28, 3)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    (got,) = run_graph(conv_build(wt, b, 1, 1), [x], autotune=True)
    assert rel_err(got, ref) <= TOL_FP32


# ------------------------------------------------------------ fully connected
@pytest.mark.parametrize("n", [1, 3, 8, 16, 40])
@pytest.mark.parametrize("c,h,w,nout,act,bias", [(8, 2, 3, 20, 1, True), (16, 4, 4, 64, 0, True), (12, 5, 5, 10, 1, False),
                                                 (32, 7, 7, 1000, 0, True), (3, 3, 3, 7, 1, True)])
def test_fc_matches_oracle(n, c, h, w, nout, act, bias):
    x, wt, b = cases.fc_case("fc%d_%d" % (c * h * w, nout), n, c, h, w, nout, bias)
    ref = oracle.fc(x, wt, b, act)

    def build(g, f):
        return dr.Fully_Connected(f[0], [c * h * w, nout], "relu" if act else "linear", wt, b)
    (got,) = run_graph(build, [x])
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("n", [2, 4, 5, 12, 16, 17, 24, 32, 33, 64])
@pytest.mark.parametrize("c,h,w,nout", [(41, 10, 10, 132), (64, 8, 9, 1000)])
def test_fc_streaming_kernels_on_ragged_shapes(n, c, h, w, nout):
    """Every batch-size class of the weight-streaming path (2, 4, 8 and 16 rows per pass, passes of 16 with a shorter last one, the
    K-sliced GEMM above 32 rows) on shapes whose K slices end inside an input stage (Nin = 4100, 4608) and whose last column block is
    partly empty (Nout = 132, 1000)."""
    x, wt, b = cases.fc_case("fcr%d_%d" % (c * h * w, nout), n, c, h, w, nout, True)
    ref = oracle.fc(x, wt, b, 1)

    def build(g, f):
        return dr.Fully_Connected(f[0], [c * h * w, nout], "relu", wt, b)
    (got,) = run_graph(build, [x])
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("name", ["fc_3x2x8_to_20", "fc_4x4x16_to_64_linear"])
def test_fc_matches_reference_kernel_golden(name):
    kind, kw = cases.GOLDEN_CASES[name]
    x, wt, b = cases.make_inputs(name)

    def build(g, f):
        return dr.Fully_Connected(f[0], list(wt.shape), "relu" if kw["act"] else "linear", wt, b)
    (got,) = run_graph(build, [x])
    assert rel_err(got, GOLD[name]) <= TOL_FP32


# ----------------------------------------------------------------------- pooling
@pytest.mark.parametrize("name", [n for n, (k, _) in cases.GOLDEN_CASES.items() if k == "pool"])
def test_pool_matches_reference_kernel_golden(name):
    kind, kw = cases.GOLDEN_CASES[name]
    (x,) = cases.make_inputs(name)
    k, s = kw["k"], kw["stride"]
    (got,) = run_graph(lambda g, f: dr.Pooling(f[0], "max" if kw["kind"] == 0 else "average", [1, k, k, 1], [1, s, s, 1]), [x])
    if kw["kind"] == 0:
        assert np.array_equal(got, GOLD[name])
    else:
        assert rel_err(got, GOLD[name]) <= 1e-6


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n,c,h,w,size,stride", [(2, 8, 14, 14, (2, 2, 1), (2, 2, 1)), (1, 5, 11, 13, (3, 3, 1), (2, 2, 1)),
                                                 (3, 64, 28, 28, (3, 3, 1), (2, 2, 1)), (1, 6, 9, 7, (3, 2, 1), (1, 2, 1)),
                                                 (1, 9, 6, 6, (2, 2, 3), (2, 2, 3)), (2, 4, 7, 7, (7, 7, 1), (7, 7, 1))])
def test_pool_matches_oracle(kind, n, c, h, w, size, stride):
    x = cases.act_case("pool%d%d%d" % (c, h, w), n, c, h, w)
    x -= 2.0        # all-negative regions make the zero padding visible in max pooling
    ref = oracle.pool(x, size, stride, kind)
    sx, sy, sz = size
    stx, sty, stz = stride
    (got,) = run_graph(lambda g, f: dr.Pooling(f[0], "max" if kind == 0 else "average", [1, sy, sx, sz], [1, sty, stx, stz]), [x])
    if kind == 0:
        assert np.array_equal(got, ref)
    else:
        assert rel_err(got, ref) <= 1e-6


# ----------------------------------------------------- softmax and element-wise
def test_softmax_matches_golden_and_oracle():
    (x,) = cases.make_inputs("softmax_1000")
    (got,) = run_graph(lambda g, f: dr.Softmax(f[0]), [x])
    assert rel_err(got, GOLD["softmax_1000"]) <= 1e-5
    xb = cases.act_case("softmax_b", 5, 10, 3, 4, 2.0)
    (got,) = run_graph(lambda g, f: dr.Softmax(f[0]), [xb])
    assert rel_err(got, oracle.softmax(xb)) <= 1e-5
    assert np.allclose(got.reshape(5, -1).sum(1), 1.0, atol=1e-5)


def test_softmax_stays_finite_where_the_reference_overflows():
    x = np.zeros((1, 6, 1, 1), np.float32)
    x[0, :, 0, 0] = [100.0, 99.0, 0.0, -5.0, 98.0, 100.0]     # exp(100) overflows fp32: the reference gives inf/inf
    (got,) = run_graph(lambda g, f: dr.Softmax(f[0]), [x])
    e = np.exp(x.astype(np.float64) - 100.0)
    assert np.all(np.isfinite(got))
    assert rel_err(got, e / e.sum()) <= 1e-5


def test_elementwise_ops_match_golden():
    (x,) = cases.make_inputs("ew1_all")
    for (op, s), fn in zip(cases.EW1_OPS, [dr.Add_Scalar, dr.Sub_Scalar, dr.Mul_Scalar, dr.Div_Scalar, None, None, None, dr.Fill, dr.Pow_Scalar]):
        if op == 4:
            build = lambda g, f: dr.Log(f[0])
        elif op == 5:
            build = lambda g, f: dr.Exp(f[0])
        elif op == 6:
            build = lambda g, f: dr.Sqrt(f[0])
        else:
            build = lambda g, f, fn=fn, s=s: fn(f[0], s)
        (got,) = run_graph(build, [x])
        assert rel_err(got, GOLD["ew1_all_op%d" % op]) <= 2e-6, op
    a, b = cases.make_inputs("ew2_all")
    for op, fn in zip(cases.EW2_OPS, [dr.Add, dr.Sub, dr.Mul, dr.Div, dr.Pow]):
        (got,) = run_graph(lambda g, f, fn=fn: fn(f[0], f[1]), [a, b])
        assert rel_err(got, GOLD["ew2_all_op%d" % op]) <= 2e-6, op


def test_elementwise_large_and_unaligned_lengths():
    x = cases.act_case("ew_big", 3, 7, 33, 31)
    (got,) = run_graph(lambda g, f: dr.Mul_Scalar(dr.Add_Scalar(f[0], 1.25), -2.0), [x])
    assert np.array_equal(got, (x + np.float32(1.25)) * np.float32(-2.0))


# --------------------------------------------------- slice / crop-or-pad / concat
def test_slice_croporpad_match_golden():
    (x,) = cases.make_inputs("slice_crop")
    (got,) = run_graph(lambda g, f: dr.Slice(f[0], (1, 1, 2), (3, 6, 5)), [x])     # CHW order: (c, y, x)
    assert np.array_equal(got, GOLD["slice_crop_slice"])
    (got,) = run_graph(lambda g, f: dr.Crop_Or_Pad(f[0], (6, 12, 11)), [x])
    assert np.array_equal(got, GOLD["slice_crop_pad"])
    (got,) = run_graph(lambda g, f: dr.Crop_Or_Pad(f[0], (6, 4, 5)), [x])
    assert np.array_equal(got, GOLD["slice_crop_crop"])


@pytest.mark.parametrize("dim", [0, 1, 2])          # CHW interface: 0 = channels, 1 = rows, 2 = columns
def test_concat_every_axis(dim):
    shapes = [[2, 4, 6, 5], [2, 4, 6, 5], [2, 4, 6, 5]]
    shapes[1][dim + 1] += 2
    shapes[2][dim + 1] += 1
    xs = [cases.act_case("cat%d%d" % (dim, i), *s) for i, s in enumerate(shapes)]
    (got,) = run_graph(lambda g, f: dr.Concat(list(f), dim), xs)
    assert np.array_equal(got, np.concatenate(xs, axis=dim + 1))


# ------------------------------------------------------------ interface details
def test_hwc_interface_layout_equals_chw():
    x, wt, b = cases.conv_case("layout", 2, 6, 10, 9, 11, 3)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = 2
        f = dr.feed_node(g, [9, 11, 6])
        o = dr.Conv2d(f, [3, 3, 6, 10], [1, 1, 1, 1], "relu", hwio(wt), b)
        dr.mark_as_output(o)
        dr.prepare(g)
        dr.feed_data(f, np.ascontiguousarray(x.transpose(0, 2, 3, 1)))
        (got,) = dr.apply(g)
    assert rel_err(got.transpose(0, 3, 1, 2), ref) <= TOL_FP32


def test_native_hwc_interface_skips_conversion():
    """dR_setInterfaceLayout(HWC): feed and output buffers are N-HWC, no layout kernels run."""
    from ctypes import c_void_p, pointer
    from deepracin_b200._lib import Shape3, Shape4
    lib = dr.lib
    x, wt, b = cases.conv_case("native", 2, 8, 8, 6, 7, 3)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    g = lib.dR_NewGraph()
    lib.dR_setBatchSize(g, 2)
    lib.dR_setInterfaceLayout(g, 1)
    assert lib.dR_initCL(g)
    f = lib.dR_Datafeednode(g, pointer(Shape3(7, 6, 8)))
    c = lib.dR_Conv2d(g, f, pointer(Shape4(3, 3, 8, 8)), pointer(Shape4(1, 1, 1, 1)), 1, 1)
    lib.dR_Conv2d_setVariables(c, wt.ctypes.data_as(dr._FP), b.ctypes.data_as(dr._FP))
    lib.dR_setAsOutput(g, c)
    assert lib.dR_prepare(g)
    xin = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    lib.dR_feedData(g, f, xin.ctypes.data_as(dr._FP), 0, xin.size)
    assert lib.dR_getLaunchCount(g) == 3            # Winograd: transform, GEMMs, inverse transform -- nothing else
    outs = (c_void_p * 1)()
    assert lib.dR_getOutputBuffers(g, outs) == 1
    got = np.empty((2, 6, 7, 8), np.float32)
    lib.dR_downloadArray(g, b"", outs[0], 0, got.nbytes, got.ctypes.data_as(c_void_p))
    lib.dR_cleanup(g, 1)
    assert rel_err(got.transpose(0, 3, 1, 2), ref) <= TOL_FP32


def test_partial_feed_with_offset_and_repeated_apply():
    x, wt, b = cases.conv_case("offset", 3, 4, 4, 6, 6, 3)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = 3
        f = dr.feed_node(g, [4, 6, 6])
        o = dr.Conv2d(f, [3, 3, 4, 4], [1, 1, 1, 1], "relu", hwio(wt), b)
        dr.mark_as_output(o)
        dr.prepare(g)
        per = 4 * 6 * 6
        for i in (2, 0, 1):     # one image at a time at its float offset, as a host loop would
            img = np.ascontiguousarray(x[i])
            dr.lib.dR_feedData(g.ptr, f.ptr, img.ctypes.data_as(dr._FP), i * per, per)
        a = dr.apply(g)[0]
        b2 = dr.apply(g)[0]
    assert np.array_equal(a, b2)
    assert rel_err(a, ref) <= TOL_FP32


def test_profiling_reports_kernel_times(capfd):
    x, wt, b = cases.conv_case("prof", 1, 8, 8, 8, 8, 3)
    run_graph(conv_build(wt, b), [x], profileGPU=True, silent=False)
    out = capfd.readouterr().out
    assert "GPU Profiling: deepRACIN:conv2d took" in out
    assert "Sum of all kernel run times" in out


def test_caller_owned_stream_and_buffers():
    """dR_setClEnvironment with the caller's CUDA stream, dR_setDataFeedNodeBuffer / dR_setPreexistingOutputBuffer with the
    caller's device buffers (reference include/deepRACIN.h:72,126,242): nothing is copied, the graph reads and writes them."""
    import ctypes
    import torch
    from ctypes import c_void_p, pointer
    from deepracin_b200._lib import Shape3, Shape4
    lib = dr.lib
    x, wt, b = cases.conv_case("caller_owned", 2, 8, 12, 6, 10, 3)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    xin = torch.from_numpy(x).to(dev)                       # [n, C, H, W]: the reference's interface layout
    yout = torch.zeros(2, 12, 6, 10, device=dev)
    g = lib.dR_NewGraph()
    lib.dR_setBatchSize(g, 2)
    lib.dR_setClEnvironment(g, None, None, stream.cuda_stream, 0)
    f = lib.dR_Datafeednode(g, pointer(Shape3(10, 6, 8)))
    c = lib.dR_Conv2d(g, f, pointer(Shape4(3, 3, 8, 12)), pointer(Shape4(1, 1, 1, 1)), 1, 1)
    lib.dR_Conv2d_setVariables(c, wt.ctypes.data_as(dr._FP), b.ctypes.data_as(dr._FP))
    in_ptr, out_ptr = c_void_p(xin.data_ptr()), c_void_p(yout.data_ptr())
    assert lib.dR_setDataFeedNodeBuffer(g, f, ctypes.byref(in_ptr))
    assert lib.dR_setPreexistingOutputBuffer(g, c, ctypes.byref(out_ptr))
    assert lib.dR_prepare(g)
    torch.cuda.synchronize(dev)
    assert lib.dR_apply(g)
    stream.synchronize()
    assert rel_err(yout.cpu().numpy(), ref) <= TOL_FP32
    # a new input buffer between applies: only the pointer changes
    xin2 = torch.from_numpy(np.ascontiguousarray(x[::-1])).to(dev)
    in_ptr2 = c_void_p(xin2.data_ptr())
    assert lib.dR_setDataFeedNodeBuffer(g, f, ctypes.byref(in_ptr2))
    assert lib.dR_apply(g)
    stream.synchronize()
    assert rel_err(yout.cpu().numpy(), ref[::-1]) <= TOL_FP32
    lib.dR_cleanup(g, 0)
    assert np.array_equal(xin.cpu().numpy(), x)             # caller's buffers survive the cleanup
