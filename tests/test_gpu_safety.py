"""GPU tests of what stands in for a memory checker and a fault injector on this path:

* guard bands -- every kernel family writes a caller-owned output buffer (dR_setPreexistingOutputBuffer) that sits inside a
  larger allocation filled with a sentinel; after dR_apply the sentinels in front of and behind the tensor must be
  untouched and the tensor itself must hold no sentinel.  Shapes are the awkward ones: odd widths and heights, channel
  counts that end inside a warp or inside an N tile, pooled outputs, channel-offset stores into a Concat buffer.
* the bounded-wait failure path -- a one-CTA probe makes the kernels' own wait function run out on a barrier that nothing
  arrives at (limit ~1 ms), the status word reports it, and the same graph computes correctly afterwards.  Nothing here
  faults, traps or hangs the device.
* replacing a feed buffer under a captured CUDA graph."""
import ctypes
from ctypes import c_void_p, pointer

import numpy as np
import pytest

import cases
import deepracin_b200 as dr
import oracle
from deepracin_b200._lib import Shape2, Shape3, Shape4
from gpu_helpers import TOL_FP32, TOL_TF32, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SENTINEL = np.float32(-7.25e30)
GUARD = 4096                                    # floats on either side


def guarded_run(build, x, out_shape, math, fuse=True):
    """Builds feed -> build(lib, graph, feed) -> node with the graph's interface in N-HWC, so that the node's own kernels
    (not a layout conversion) write the caller-owned output buffer, which sits between two sentinel-filled guard bands.
    x and the result are [n, C, H, W]; returns (result, guard in front, guard behind)."""
    lib = dr.lib
    n, c, h, w = x.shape
    no, co, ho, wo = out_shape
    out_floats = no * co * ho * wo
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    whole = torch.full((GUARD + out_floats + GUARD,), float(SENTINEL), device=dev, dtype=torch.float32)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).to(dev)
    g = lib.dR_NewGraph()
    lib.dR_setBatchSize(g, n)
    lib.dR_setMathMode(g, dr.MATH[math])
    lib.dR_setFusion(g, 1 if fuse else 0)
    lib.dR_setInterfaceLayout(g, 1)
    lib.dR_setClEnvironment(g, None, None, stream.cuda_stream, 0)
    f = lib.dR_Datafeednode(g, pointer(Shape3(w, h, c)))
    node = build(lib, g, f)
    in_ptr = c_void_p(xin.data_ptr())
    out_ptr = c_void_p(whole.data_ptr() + GUARD * 4)
    assert lib.dR_setDataFeedNodeBuffer(g, f, ctypes.byref(in_ptr))
    assert lib.dR_setPreexistingOutputBuffer(g, node, ctypes.byref(out_ptr))
    assert lib.dR_prepare(g)
    assert lib.dR_getNodeActAddress(node) == out_ptr.value      # the node's kernels store into the caller's buffer itself
    torch.cuda.synchronize(dev)
    assert lib.dR_apply(g)
    stream.synchronize()
    assert lib.dR_getDeviceStatus(g) == 0
    host = whole.cpu().numpy()
    lib.dR_cleanup(g, 0)
    out = host[GUARD:GUARD + out_floats]
    assert not np.any(out == SENTINEL), "output element never written"
    return out.reshape(no, ho, wo, co).transpose(0, 3, 1, 2), host[:GUARD], host[GUARD + out_floats:]


def conv_node(wt, b, act=1, stride=1):
    cin, cout, kh, kw = wt.shape

    def build(lib, g, f):
        c = lib.dR_Conv2d(g, f, pointer(Shape4(kw, kh, cin, cout)), pointer(Shape4(1, stride, stride, 1)), act, 1 if b is not None else 0)
        lib.dR_Conv2d_setVariables(c, wt.ctypes.data_as(dr._FP), None if b is None else b.ctypes.data_as(dr._FP))
        return c
    return build


def check_guards(out, front, back):
    assert np.all(front == SENTINEL), "write in front of the output tensor"
    assert np.all(back == SENTINEL), "write behind the output tensor"


GUARD_CONVS = [
    # name, n, cin, cout, h, w, k, math
    ("g_swap_odd", 40, 8, 136, 29, 27, 3, "tf32"),          # transposed kernel, odd image, Cout ends inside a warp
    ("g_pair_w15", 2, 24, 40, 34, 15, 3, "tf32"),           # row-pair kernel, image one pixel wider than a block
    ("g_pair_odd_h", 2, 32, 48, 61, 28, 3, "tf32"),
    ("g_1x1_1000", 2, 512, 1000, 14, 14, 1, "tf32"),        # Cout ends inside the last N tile
    ("g_1x1_odd", 3, 32, 72, 9, 7, 1, "tf32"),
    ("g_halo_13x17", 3, 64, 200, 17, 13, 3, "tf32"),
    ("g_first_c3", 3, 3, 48, 17, 13, 3, "tf32"),            # producer-gather first layer, pixel count not a multiple of its tile
    ("g_wino_odd", 2, 8, 20, 11, 9, 3, "fp32"),             # FP32 Winograd F(2x2,3x3) with ragged 2x2 output tiles
    ("g_wino4_odd", 2, 16, 20, 11, 9, 3, "fp32"),           # F(4x4,3x3): ragged 4x4 output tiles, Cout ends inside a warp
    ("g_wino4_c17", 3, 17, 19, 14, 6, 3, "fp32"),           # odd channel counts: scalar transform path
    ("g_x3w_odd", 2, 128, 264, 13, 11, 3, "fp32x3"),        # F(4x4,3x3) with three-pass tensor products: ragged tiles, padded GEMM rows
    ("g_x3_direct", 3, 32, 40, 15, 18, 3, "fp32x3"),        # the direct three-pass kernel
    ("g_direct_5x5", 2, 6, 10, 9, 13, 5, "fp32"),
    ("g_1x1_fp32", 2, 24, 52, 7, 5, 1, "fp32"),
    ("g_first_fp32", 2, 3, 20, 9, 11, 3, "fp32"),
]


@pytest.mark.parametrize("name,n,cin,cout,h,w,k,math", GUARD_CONVS)
def test_convolution_stores_stay_inside_the_output_tensor(name, n, cin, cout, h, w, k, math):
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, k, True)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    out, front, back = guarded_run(conv_node(wt, b), x, ref.shape, math)
    check_guards(out, front, back)
    assert rel_err(out, ref) <= (TOL_TF32 if math == "tf32" else TOL_FP32)


@pytest.mark.parametrize("name,n,cin,cout,h,w,math", [("gp_swap", 40, 8, 72, 30, 26, "tf32"), ("gp_pair", 6, 16, 64, 56, 56, "tf32"),
                                                       ("gp_halo", 2, 32, 136, 12, 20, "tf32"), ("gp_first", 2, 3, 64, 18, 22, "tf32"),
                                                       ("gp_wino4", 3, 16, 36, 14, 10, "fp32"), ("gp_wino4_c17", 2, 17, 21, 6, 18, "fp32"),
                                                       ("gp_x3w", 2, 128, 256, 12, 20, "fp32x3")])
def test_fused_pool_stores_stay_inside_the_output_tensor(name, n, cin, cout, h, w, math):
    """conv3x3 + 2x2/2 max pool evaluated by the convolution's epilogue (FP32 mode: by the F(4x4,3x3) output transform): the
    guarded buffer is the POOLING node's output."""
    x, wt, b = cases.conv_case(name, n, cin, cout, h, w, 3, True)
    ref = oracle.pool(oracle.conv2d(x, wt, b, (1, 1), 1), (2, 2, 1), (2, 2, 1), 0)

    def build(lib, g, f):
        c = conv_node(wt, b)(lib, g, f)
        return lib.dR_Pooling(g, c, pointer(Shape4(1, 2, 2, 1)), pointer(Shape4(1, 2, 2, 1)), 0)
    out, front, back = guarded_run(build, x, ref.shape, math)
    check_guards(out, front, back)
    assert rel_err(out, ref) <= (TOL_TF32 if math == "tf32" else TOL_FP32)


@pytest.mark.parametrize("math", ["fp32", "tf32"])
def test_channel_offset_stores_into_a_concat_buffer(math):
    """Fire-module expand layers store at their channel offsets of the Concat's buffer (no copy kernel): with 24 + 40 channels
    neither store may touch the neighbour's channels or the guards."""
    x, w1, b1 = cases.conv_case("gc_e1", 3, 16, 24, 9, 11, 1, True)
    _, w3, b3 = cases.conv_case("gc_e3", 1, 16, 40, 9, 11, 3, True)
    ref = np.concatenate([oracle.conv2d(x, w1, b1, (1, 1), 1), oracle.conv2d(x, w3, b3, (1, 1), 1)], axis=1)

    def build(lib, g, f):
        a = conv_node(w1, b1)(lib, g, f)
        c = conv_node(w3, b3)(lib, g, f)
        nodes = (c_void_p * 2)(a, c)
        return lib.dR_Concat(g, nodes, 2, 2)
    out, front, back = guarded_run(build, x, ref.shape, math)
    check_guards(out, front, back)
    assert rel_err(out, ref) <= (TOL_TF32 if math == "tf32" else TOL_FP32)


@pytest.mark.parametrize("n,c,h,w,nout,math", [(3, 5, 3, 7, 37, "fp32"), (20, 64, 2, 2, 72, "tf32"), (17, 8, 4, 4, 1000, "fp32"),
                                               (5, 33, 4, 4, 132, "fp32"), (19, 33, 4, 4, 132, "fp32"), (40, 16, 4, 4, 200, "fp32")])
def test_fully_connected_stores_stay_inside_the_output_tensor(n, c, h, w, nout, math):
    x, wt, b = cases.fc_case("gfc_%d" % nout, n, c, h, w, nout, True)
    ref = oracle.fc(x, wt, b, 1)

    def build(lib, g, f):
        node = lib.dR_FullyConnected(g, f, pointer(Shape2(c * h * w, nout)), 1, 1)
        lib.dR_FullyConnected_setVariables(node, wt.ctypes.data_as(dr._FP), b.ctypes.data_as(dr._FP))
        return node
    out, front, back = guarded_run(build, x, ref.shape, math)
    check_guards(out, front, back)
    assert rel_err(out, ref) <= (TOL_TF32 if math == "tf32" else TOL_FP32)


@pytest.mark.parametrize("k,stride,kind", [(3, 2, 0), (2, 2, 1), (2, 2, 0)])
def test_pooling_and_softmax_stores_stay_inside_the_output_tensor(k, stride, kind):
    x = cases.act_case("gpool_%d%d" % (k, kind), 3, 5, 11, 13)
    ref = oracle.pool(x, (k, k, 1), (stride, stride, 1), kind)
    out, front, back = guarded_run(lambda lib, g, f: lib.dR_Pooling(g, f, pointer(Shape4(1, k, k, 1)), pointer(Shape4(1, stride, stride, 1)), kind), x, ref.shape, "fp32")
    check_guards(out, front, back)
    assert rel_err(out, ref) <= 1e-6
    xs = cases.act_case("gsoft", 3, 37, 1, 1, 2.0)
    out, front, back = guarded_run(lambda lib, g, f: lib.dR_Softmax(g, f), xs, xs.shape, "fp32")
    check_guards(out, front, back)
    assert rel_err(out, oracle.softmax(xs)) <= 1e-5


def test_bounded_wait_runs_out_reports_and_leaves_the_context_usable():
    """The failure path of the tcgen05 kernels, without a failure: the kernels' own wait gives up after ~1 ms on a barrier nobody
    arrives at, dR_getDeviceStatus reports the code once, and the next dR_apply of the same graph is clean and correct."""
    x, wt, b = cases.conv_case("wait_probe", 4, 32, 64, 20, 28, 3, True)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    with dr.Environment() as env:
        g = env.create_graph("CHW")
        g.batch = 4
        g.math = "tf32"
        f = dr.feed_node(g, [32, 20, 28])
        o = dr.Conv2d(f, [3, 3, 32, 64], [1, 1, 1, 1], "relu", np.ascontiguousarray(wt.transpose(2, 3, 0, 1)), b)
        dr.mark_as_output(o)
        dr.prepare(g)
        dr.feed_data(f, x)
        first = dr.apply(g)[0].reshape(ref.shape)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
        res = (ctypes.c_int * 3)()
        assert dr.lib.dR_probeBoundedWait(g.ptr, 1000, res)
        assert res[0] == 0                              # the wait on the barrier nobody arrives at ran out ...
        assert res[1] == 1                              # ... the wait on the barrier that was arrived at did not
        khz = torch.cuda.get_device_properties(0).clock_rate
        limit_units = 1000 * (khz // 1000) // 1024
        assert limit_units <= res[2] <= 4 * limit_units + 64      # it gave up after the limit, not after the default second
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 9    # reported through the graph's status word ...
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0    # ... once
        again = dr.apply(g)[0].reshape(ref.shape)
        assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    assert np.array_equal(first, again)
    assert rel_err(again, ref) <= TOL_TF32


@pytest.mark.parametrize("math", ["fp32", "tf32"])
def test_feed_buffer_replaced_under_a_captured_cuda_graph(math):
    """dR_setDataFeedNodeBuffer between applies with CUDA-graph replay on: the captured graph holds the old address in its
    kernel arguments and tensor maps, so the next apply must capture again -- also when the caller only changes the pointer
    variable it handed over."""
    lib = dr.lib
    x, wt, b = cases.conv_case("swap_feed", 2, 16, 24, 10, 14, 3, True)
    ref = oracle.conv2d(x, wt, b, (1, 1), 1)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    bufs = [torch.from_numpy(np.ascontiguousarray(v)).to(dev) for v in (x, x[::-1], 2.0 * x)]
    refs = [ref, ref[::-1], oracle.conv2d(2.0 * x, wt, b, (1, 1), 1)]
    yout = torch.zeros(ref.shape, device=dev)
    g = lib.dR_NewGraph()
    lib.dR_setBatchSize(g, 2)
    lib.dR_setMathMode(g, dr.MATH[math])
    lib.dR_setCudaGraph(g, 1)
    lib.dR_setInterfaceLayout(g, 0)
    lib.dR_setClEnvironment(g, None, None, stream.cuda_stream, 0)
    f = lib.dR_Datafeednode(g, pointer(Shape3(14, 10, 16)))
    c = conv_node(wt, b)(lib, g, f)
    in_ptr, out_ptr = c_void_p(bufs[0].data_ptr()), c_void_p(yout.data_ptr())
    assert lib.dR_setDataFeedNodeBuffer(g, f, ctypes.byref(in_ptr))
    assert lib.dR_setPreexistingOutputBuffer(g, c, ctypes.byref(out_ptr))
    assert lib.dR_prepare(g)
    torch.cuda.synchronize(dev)
    tol = TOL_TF32 if math == "tf32" else TOL_FP32
    for _ in range(2):
        assert lib.dR_apply(g)
    stream.synchronize()
    assert rel_err(yout.cpu().numpy(), refs[0]) <= tol
    in_ptr2 = c_void_p(bufs[1].data_ptr())                  # a new handle through the API
    assert lib.dR_setDataFeedNodeBuffer(g, f, ctypes.byref(in_ptr2))
    for _ in range(2):
        assert lib.dR_apply(g)
    stream.synchronize()
    assert rel_err(yout.cpu().numpy(), refs[1]) <= tol
    in_ptr2.value = bufs[2].data_ptr()                      # the caller rewrites its own pointer variable behind the handle
    assert lib.dR_apply(g)
    stream.synchronize()
    assert rel_err(yout.cpu().numpy(), refs[2]) <= tol
    assert lib.dR_getDeviceStatus(g) == 0
    lib.dR_cleanup(g, 0)
