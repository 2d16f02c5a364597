"""CPU tests of the host side: exported C ABI, graph construction, scheduling, the buffer planner
(dry run, no device), fusion planning, the saved-graph format and API misuse."""
import filecmp
import glob
import os
import re

import numpy as np
import pytest

import deepracin_b200 as dr
import oracle
from deepracin_b200._lib import Shape3, Shape4
from ctypes import pointer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SLOTS = ["compute", "schedule", "propagateShape", "getRequiredOutputBufferSize", "createKernel", "allocateBuffers",
         "fillBuffers", "cleanupBuffers", "cleanupLayer", "serializeNode", "parseAppendNode", "printLayer"]


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#define[^\n]*(\\\n[^\n]*)*", "", text)
        for m in re.finditer(r"DR_DECL_NODE_SLOTS\((\w+)\)", text):
            names.update("%s_%s" % (m.group(1), s) for s in SLOTS)
        for m in re.finditer(r"\b((?:dRk?|concat_and_free_old)\w*)\s*\(", text):
            name = m.group(1)
            before = text[max(0, m.start() - 2):m.start()]
            if "(*" in text[max(0, m.start() - 3):m.start()] or before.endswith("*)"):
                continue
            names.add(name)
    return sorted(n for n in names if not n.startswith("DR_"))


def test_library_loads_and_exports_every_declared_symbol():
    missing = [n for n in declared_symbols() if not hasattr(dr.lib, n)]
    assert len(declared_symbols()) > 150
    assert missing == []


def small_net(env, batch=1, fuse=True):
    g = env.create_graph("HWC")
    g.batch = batch
    g.fuse = fuse
    r = np.random.default_rng(0)
    x = dr.feed_node(g, [16, 16, 3])
    c1 = dr.Conv2d(x, [3, 3, 3, 8], [1, 1, 1, 1], "relu", r.standard_normal((3, 3, 3, 8)).astype(np.float32), np.zeros(8, np.float32))
    p1 = dr.Pooling(c1, "max", [1, 3, 3, 1], [1, 2, 2, 1])
    sq = dr.Conv2d(p1, [1, 1, 8, 4], [1, 1, 1, 1], "relu", r.standard_normal((1, 1, 8, 4)).astype(np.float32), np.zeros(4, np.float32))
    e1 = dr.Conv2d(sq, [1, 1, 4, 8], [1, 1, 1, 1], "relu", r.standard_normal((1, 1, 4, 8)).astype(np.float32), np.zeros(8, np.float32))
    e3 = dr.Conv2d(sq, [3, 3, 4, 8], [1, 1, 1, 1], "relu", r.standard_normal((3, 3, 4, 8)).astype(np.float32), np.zeros(8, np.float32))
    cat = dr.Concat([e1, e3], 2)
    gp = dr.Pooling(cat, "average", [1, 8, 8, 1], [1, 8, 8, 1])
    fc = dr.Fully_Connected(gp, [16, 10], "linear", r.standard_normal((16, 10)).astype(np.float32), np.zeros(10, np.float32))
    sm = dr.Softmax(fc)
    dr.mark_as_output(sm)
    return g, dict(x=x, c1=c1, p1=p1, sq=sq, e1=e1, e3=e3, cat=cat, gp=gp, fc=fc, sm=sm)


def dry_prepare(g):
    assert dr.lib.dR_setDryRun(g.ptr, 1)
    dr.lib.dR_setBatchSize(g.ptr, g.batch)
    dr.lib.dR_setFusion(g.ptr, 1 if g.fuse else 0)
    assert dr.lib.dR_prepare(g.ptr)


def shape_of(node):
    s = dr.lib.dR_getOutputShape(node.ptr).contents
    return (s.s0, s.s1, s.s2)


def test_shapes_schedule_and_fusion_plan():
    with dr.Environment() as env:
        g, n = small_net(env)
        dry_prepare(g)
        assert shape_of(n["c1"]) == (16, 16, 8)
        assert shape_of(n["p1"]) == (8, 8, 8)            # ceil(16/2)
        assert shape_of(n["cat"]) == (8, 8, 16)
        assert shape_of(n["gp"]) == (1, 1, 16)
        assert shape_of(n["sm"]) == (10, 1, 1)
        order = [dr.lib.dR_getScheduledNodeId(g.ptr, i) for i in range(dr.lib.dR_getScheduleLength(g.ptr))]
        assert order == sorted(order) and len(order) == 9   # feed node is not scheduled
        # both expand convolutions write straight into the Concat's buffer at their channel offsets
        cat_addr = dr.lib.dR_getNodeActAddress(n["cat"].ptr)
        assert dr.lib.dR_getNodeActAddress(n["e1"].ptr) == cat_addr
        assert dr.lib.dR_getNodeActAddress(n["e3"].ptr) == cat_addr
        assert (dr.lib.dR_getNodeChannelStride(n["e1"].ptr), dr.lib.dR_getNodeChannelOffset(n["e1"].ptr)) == (16, 0)
        assert (dr.lib.dR_getNodeChannelStride(n["e3"].ptr), dr.lib.dR_getNodeChannelOffset(n["e3"].ptr)) == (16, 8)
        assert not dr.lib.dR_apply(g.ptr)                   # a dry run can never compute


def test_fusion_can_be_switched_off():
    with dr.Environment() as env:
        g, n = small_net(env, fuse=False)
        dry_prepare(g)
        addrs = {k: dr.lib.dR_getNodeActAddress(v.ptr) for k, v in n.items()}
        assert addrs["e1"] != addrs["cat"] and addrs["e3"] != addrs["cat"]
        assert dr.lib.dR_getNodeChannelStride(n["e1"].ptr) == 8


@pytest.mark.parametrize("fuse", [True, False])
def test_buffer_planner_never_aliases_live_tensors(fuse):
    """Walk the schedule: a node's output buffer must differ from every buffer that is still to be read."""
    with dr.Environment() as env:
        g, n = small_net(env, batch=3, fuse=fuse)
        dry_prepare(g)
        names = ["c1", "p1", "sq", "e1", "e3", "cat", "gp", "fc", "sm"]
        consumers = {"x": ["c1"], "c1": ["p1"], "p1": ["sq"], "sq": ["e1", "e3"], "e1": ["cat"], "e3": ["cat"], "cat": ["gp"],
                     "gp": ["fc"], "fc": ["sm"], "sm": []}
        addr = {k: dr.lib.dR_getNodeActAddress(v.ptr) for k, v in n.items()}
        size = {k: dr.lib.dR_getNodeActFloats(v.ptr) for k, v in n.items()}
        for k in names:
            w, h, c = shape_of(n[k])
            assert size[k] >= w * h * c
        done = set()
        for k in names:
            live = [p for p in ["x"] + names if p != k and (p in done or p == "x") and any(q not in done for q in consumers[p])]
            for p in live:
                shared_concat = fuse and {k, p} <= {"e1", "e3", "cat"}
                assert addr[k] != addr[p] or shared_concat, (k, p)
            done.add(k)
        assert dr.lib.dR_getStreamBufferCount(g.ptr) <= 8


def test_save_load_roundtrip(tmp_path):
    with dr.Environment() as env:
        g, _ = small_net(env)
        dr.save_graph(g, str(tmp_path / "a"))
        g2 = env.create_graph("HWC")
        nodes, feeds = dr.load_graph(g2, str(tmp_path / "a" / "dr_graph_export"))
        assert len(nodes) == 10 and len(feeds) == 1
        dr.save_graph(g2, str(tmp_path / "b"))
        da, db = str(tmp_path / "a" / "dr_graph_export"), str(tmp_path / "b" / "dr_graph_export")
        files = sorted(os.listdir(da))
        assert files == sorted(os.listdir(db)) and "graph.dr" in files
        match, mismatch, errors = filecmp.cmpfiles(da, db, files, shallow=False)
        assert mismatch == [] and errors == []
        text = open(os.path.join(da, "graph.dr")).read().split("\n")
        assert text[0] == "deepRACIN graph: 10 nodes, 1 feed nodes"
        assert text[1] == "Node 0: DataFeedNode" and text[2] == "params: 16 16 3"
        assert text[6] == "Node 1: Conv2D" and text[7] == "params: 1 1 3 3 3 8 1 1 1 1"
        assert text[10] == "variable_files: 0.var 1.var"


@pytest.mark.skipif(oracle.staged_squeezenet_dir() is None, reason="pretrained SqueezeNet fixture not staged")
def test_reference_model_folder_reloads_byte_identically(tmp_path):
    """graph.dr written by the reference -> our reader -> our writer gives the same bytes."""
    src = oracle.staged_squeezenet_dir()
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        nodes, feeds = dr.load_graph(g, src)
        assert len(nodes) == 48 and len(feeds) == 1
        dr.save_graph(g, str(tmp_path))
        out = str(tmp_path / "dr_graph_export")
        assert open(os.path.join(out, "graph.dr"), "rb").read() == open(os.path.join(src, "graph.dr"), "rb").read()
        for i in range(52):
            assert filecmp.cmp(os.path.join(out, "%d.var" % i), os.path.join(src, "%d.var" % i), shallow=False)
        dry_prepare(g)
        assert shape_of(nodes[47]) == (1, 1, 1000)
        assert shape_of(nodes[8]) == (224, 224, 64) and shape_of(nodes[10]) == (56, 56, 64)


def test_api_misuse_is_reported_not_fatal(tmp_path, capfd):
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        assert not dr.lib.dR_apply(g.ptr)                          # apply before prepare
        assert dr.lib.dR_getOutputBuffers(g.ptr, None) == 0
        dr.lib.dR_setDryRun(g.ptr, 1)
        assert not dr.lib.dR_prepare(g.ptr)                        # no feed node
        with pytest.raises(RuntimeError):
            dr.load_graph(env.create_graph("HWC"), str(tmp_path))    # no graph.dr there
        g3 = env.create_graph("HWC")
        x = dr.feed_node(g3, [8, 8, 4])
        w = np.zeros((3, 3, 5, 6), np.float32)
        dr.Conv2d(x, [3, 3, 5, 6], [1, 1, 1, 1], "relu", w, None)   # filter expects 5 channels, input has 4
        dr.lib.dR_setDryRun(g3.ptr, 1)
        assert not dr.lib.dR_prepare(g3.ptr)
        g4 = env.create_graph("HWC")
        x = dr.feed_node(g4, [4, 4, 2])
        dr.Fully_Connected(x, [30, 5], "relu", np.zeros((30, 5), np.float32), None)   # 4*4*2 != 30
        dr.lib.dR_setDryRun(g4.ptr, 1)
        assert not dr.lib.dR_prepare(g4.ptr)
        g5 = env.create_graph("HWC")
        x = dr.feed_node(g5, [4, 4, 2])
        c = dr.Node(dr.lib.dR_Conv2d(g5.ptr, x.ptr, pointer(Shape4(3, 3, 2, 2)), pointer(Shape4(1, 1, 1, 1)), 1, 0), g5, "Conv2D", [])
        dr.lib.dR_setDryRun(g5.ptr, 1)
        assert not dr.lib.dR_prepare(g5.ptr)                       # weights never set
        assert not dr.lib.dR_setBatchSize(g5.ptr, 0)
    out = capfd.readouterr().out
    assert "dR_prepare first" in out or "dR_prepare" in out


def test_unsupported_constructors_return_null():
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        x = dr.feed_node(g, [4, 4, 3])
        assert not dr.lib.dR_RGB2gray(g.ptr, x.ptr)
        assert not dr.lib.dR_ResolveRoI(g.ptr, x.ptr, pointer(Shape3(2, 2, 3)))


def test_truncated_model_files_fail_cleanly(tmp_path):
    with dr.Environment() as env:
        g, _ = small_net(env)
        dr.save_graph(g, str(tmp_path))
        d = str(tmp_path / "dr_graph_export")
        os.remove(os.path.join(d, "1.var"))
        with pytest.raises(RuntimeError):
            dr.load_graph(env.create_graph("HWC"), d)
        text = open(os.path.join(d, "graph.dr")).read()
        open(os.path.join(d, "graph.dr"), "w").write(text[: len(text) // 2].rsplit("\n", 2)[0])
        with pytest.raises(RuntimeError):
            dr.load_graph(env.create_graph("HWC"), d)


def test_variable_files_of_the_wrong_size_are_rejected(tmp_path):
    """A .var file shorter (or longer) than the node's shape implies, and shape parameters that are not positive, must make
    dR_loadGraph fail: setVariables copies prod(shape) floats out of the file's buffer."""
    with dr.Environment() as env:
        g, _ = small_net(env)
        dr.save_graph(g, str(tmp_path))
        d = str(tmp_path / "dr_graph_export")
        good = open(os.path.join(d, "0.var"), "rb").read()
        nodes, _ = dr.load_graph(env.create_graph("HWC"), d)
        assert len(nodes) == 10
        for bad in (good[:-4], good + b"\0\0\0\0", good[:8]):
            open(os.path.join(d, "0.var"), "wb").write(bad)
            with pytest.raises(RuntimeError):
                dr.load_graph(env.create_graph("HWC"), d)
        open(os.path.join(d, "0.var"), "wb").write(good)
        text = open(os.path.join(d, "graph.dr")).read()
        assert "params: 1 1 3 3 3 8 1 1 1 1" in text
        for params in ("1 1 3 3 -3 8 1 1 1 1", "1 1 3 3 3 0 1 1 1 1", "1 1 70000 70000 3 8 1 1 1 1"):
            open(os.path.join(d, "graph.dr"), "w").write(text.replace("params: 1 1 3 3 3 8 1 1 1 1", "params: " + params, 1))
            with pytest.raises(RuntimeError):
                dr.load_graph(env.create_graph("HWC"), d)


def test_tensor_planner_picks_the_expected_kernels_and_geometries():
    """Planner introspection (no device): the kernel and block geometry per VGG-16 / SqueezeNet layer shape on a 148-SM GPU."""
    import ctypes
    lib = dr.lib
    lib.dRk_tensor_conv_describe.restype = ctypes.c_int
    lib.dRk_tensor_conv_describe.argtypes = [ctypes.c_int] * 9 + [ctypes.POINTER(ctypes.c_int)] * 4

    def describe(n, w, h, cin, cout, k, pool):
        vals = [ctypes.c_int(0) for _ in range(4)]
        v = lib.dRk_tensor_conv_describe(n, w, h, cin, cout, k, k, pool, 148, *[ctypes.byref(x) for x in vals])
        return (v,) + tuple(x.value for x in vals)

    FLAT, PLAIN, HALO, SWAP, PAIR, FIRST = 1, 2, 3, 4, 5, 6
    assert describe(64, 224, 224, 3, 64, 3, 0)[0] == FIRST
    assert describe(64, 224, 224, 64, 64, 3, 1) == (PAIR, 30, 28, 8, 240)            # conv1_2: 28 x 16-pixel tiles, two rows per MMA
    assert describe(64, 112, 112, 128, 128, 3, 1) == (SWAP, 30, 28, 8, 240)          # conv2_2
    assert describe(64, 56, 56, 256, 256, 3, 0) == (SWAP, 30, 28, 8, 240)            # conv3_2: two channel blocks per pixel tile
    assert describe(64, 28, 28, 512, 512, 3, 1) == (SWAP, 16, 14, 14, 224)           # conv4_3: 14 x 14-pixel tiles
    assert describe(64, 14, 14, 512, 512, 3, 0) == (SWAP, 16, 14, 14, 224)           # conv5: one image per tile
    assert describe(64, 28, 28, 256, 512, 1, 0)[0] == FLAT
    assert describe(1, 14, 14, 64, 256, 3, 0)[0] == HALO                             # batch 1: fewer tiles than SMs, smaller tiles spread further
    assert describe(64, 224, 224, 3, 64, 3, 2)[0] == FIRST                           # first layer with the average pool fused
    assert describe(64, 56, 56, 256, 256, 3, 2)[0] == 0                              # average pooling is only fused into the first-layer kernel
    assert describe(2, 20, 20, 64, 64, 5, 0)[0] == 0                                 # 5x5 filters stay on the FP32 kernels


def test_static_rule_per_math_mode_on_the_vgg16_channel_plan():
    """Which kernel family the planner's static rule gives every VGG-16 convolution in the three arithmetic modes (planning only, no
    device): FP32 -> the few-channel direct kernel, then Winograd F(4x4,3x3); TF32 -> the tensor kernels; FP32-accurate tensor mode ->
    FFMA for the RGB layer, the direct three-pass kernel up to 128 -> 128, Winograd F(4x4,3x3) with three-pass products from 128 -> 256 on."""
    plan = [(3, 64), (64, 64), (64, 128), (128, 128), (128, 256), (256, 256), (256, 256), (256, 512), (512, 512), (512, 512), (512, 512), (512, 512), (512, 512)]
    expected = {"fp32": [1] + [6] * 12, "tf32": [4] * 13, "fp32x3": [1, 4, 4, 4] + [5] * 9}
    tensor = {"fp32": [0] * 13, "tf32": [1] * 13, "fp32x3": [0] + [2] * 12}
    for math in ("fp32", "tf32", "fp32x3"):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 64
            g.math = math
            node = dr.feed_node(g, [16, 16, 3])
            convs = []
            for cin, cout in plan:
                node = dr.Conv2d(node, [3, 3, cin, cout], [1, 1, 1, 1], "relu", np.zeros((3, 3, cin, cout), np.float32), np.zeros(cout, np.float32))
                convs.append(node)
            dr.mark_as_output(node)
            dr.lib.dR_setMathMode(g.ptr, dr.MATH[math])
            dry_prepare(g)
            assert [dr.lib.dR_getConvAlgo(c.ptr) for c in convs] == expected[math], math
            assert [dr.lib.dR_getConvTensor(c.ptr) for c in convs] == tensor[math], math


def test_host_side_weight_packings():
    """The host-side packers of the Winograd F(4x4,3x3) and tensor-FC kernels against their definitions in NumPy (no device)."""
    import ctypes
    lib = dr.lib
    FP = ctypes.POINTER(ctypes.c_float)
    rng = np.random.default_rng(7)
    cin, cout = 32, 12
    w = rng.standard_normal((cin, cout, 3, 3)).astype(np.float32)           # the reference's [Cin][Cout][kh][kw]
    G = np.array([[1 / 4, 0, 0], [-1 / 6, -1 / 6, -1 / 6], [-1 / 6, 1 / 6, -1 / 6], [1 / 24, 1 / 12, 1 / 6], [1 / 24, -1 / 12, 1 / 6], [0, 0, 1]])
    U = np.einsum("ij,cojk,lk->ilco", G, w.astype(np.float64), G)           # [6][6][Cin][Cout]
    # FFMA path: [36][Cin][Cout] in float
    lib.dRk_winograd4_pack_weights.argtypes = [FP, FP, ctypes.c_int, ctypes.c_int]
    out = np.zeros((36, cin, cout), np.float32)
    assert lib.dRk_winograd4_pack_weights(w.ctypes.data_as(FP), out.ctypes.data_as(FP), cin, cout) == 0
    assert np.allclose(out, U.reshape(36, cin, cout), rtol=2e-7, atol=1e-9)     # double arithmetic, rounded to float once
    # three-pass tensor path: [36][Cout][2*Cin], upper 19 bits of the float value, then the remainder of the double value
    lib.dRk_tensor_winograd4_x3_packed_floats.restype = ctypes.c_size_t
    lib.dRk_tensor_winograd4_x3_packed_floats.argtypes = [ctypes.c_int, ctypes.c_int]
    assert lib.dRk_tensor_winograd4_x3_packed_floats(cin, cout) == 36 * cout * 2 * cin
    lib.dRk_tensor_winograd4_x3_pack_weights.argtypes = [FP, FP, ctypes.c_int, ctypes.c_int]
    out2 = np.zeros((36, cout, 2 * cin), np.float32)
    assert lib.dRk_tensor_winograd4_x3_pack_weights(w.ctypes.data_as(FP), out2.ctypes.data_as(FP), cin, cout) == 0
    Ut = U.reshape(36, cin, cout).transpose(0, 2, 1)                        # [36][Cout][Cin]
    hi, lo = out2[:, :, :cin], out2[:, :, cin:]
    assert not np.any(hi.view(np.uint32) & np.uint32(0x1FFF))               # a TF32 operand: the low 13 mantissa bits are zero
    assert np.all(np.abs(lo) <= np.abs(hi) * 2.0 ** -10 + 1e-30)            # the remainder sits below the kept bits
    assert np.max(np.abs(hi.astype(np.float64) + lo - Ut)) <= 2.0 ** -30 * np.max(np.abs(Ut))   # high + low carry the double value to ~2^-34
    # tensor FC: [n tile][K slab][256][32], zeros past Nout; the three-pass packing is the high blocks followed by the low blocks
    nin, nout = 64, 300
    wf = rng.standard_normal((nin, nout)).astype(np.float32)
    lib.dRk_tensor_fc_packed_floats.restype = ctypes.c_size_t
    lib.dRk_tensor_fc_packed_floats.argtypes = [ctypes.c_int, ctypes.c_int]
    assert lib.dRk_tensor_fc_packed_floats(nin, nout) == 2 * 256 * nin
    lib.dRk_tensor_fc_pack_weights.argtypes = [FP, FP, ctypes.c_int, ctypes.c_int]
    pk = np.full((2, nin // 32, 256, 32), 7.0, np.float32)
    assert lib.dRk_tensor_fc_pack_weights(wf.ctypes.data_as(FP), pk.ctypes.data_as(FP), nin, nout) == 0
    padded = np.zeros((nin, 512), np.float32)
    padded[:, :nout] = wf
    expect = padded.reshape(nin // 32, 32, 2, 256).transpose(2, 0, 3, 1)    # [tile][slab][row][e]
    assert np.array_equal(pk, expect)
    lib.dRk_tensor_fc_x3_pack_weights.argtypes = [FP, FP, ctypes.c_int, ctypes.c_int]
    pk2 = np.full((2, 2, nin // 32, 256, 32), 7.0, np.float32)
    assert lib.dRk_tensor_fc_x3_pack_weights(wf.ctypes.data_as(FP), pk2.ctypes.data_as(FP), nin, nout) == 0
    ehi = (expect.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    assert np.array_equal(pk2[:, 0], ehi) and np.array_equal(pk2[:, 1], expect - ehi)


def test_tensor_planner_geometries_respect_the_kernels_limits():
    """Every geometry the planner can hand to the transposed and row-pair kernels stays inside what those kernels were
    written for: N a multiple of 16 and at most 256, whole 32-column epilogue chunks at the 16-pixel pitch, an even row
    count under fused pooling, the last column's taps inside the 304-pixel shared-memory slot, valid pixels at most
    pitch - 2 (the halo columns)."""
    import ctypes
    lib = dr.lib
    lib.dRk_tensor_conv_describe.restype = ctypes.c_int
    lib.dRk_tensor_conv_describe.argtypes = [ctypes.c_int] * 9 + [ctypes.POINTER(ctypes.c_int)] * 4
    SWAP, PAIR = 4, 5
    seen = set()
    sizes = list(range(2, 66)) + [96, 111, 112, 113, 127, 128, 150, 223, 224, 225, 256, 300]
    for w in sizes:
        for h in (2, 3, 7, 8, 13, 14, 15, 16, 27, 28, 29, 30, 31, 32, 56, 57, 112, 224, w):
            for cout, pool, n in ((64, 0, 64), (64, 1, 64), (128, 0, 64), (136, 1, 64), (512, 0, 64), (256, 0, 1)):
                if pool and ((w | h) & 1):
                    continue
                vals = [ctypes.c_int(0) for _ in range(4)]
                v = lib.dRk_tensor_conv_describe(n, w, h, 64, cout, 3, 3, pool, 148, *[ctypes.byref(x) for x in vals])
                P, TW, TH, ncols = (x.value for x in vals)
                if v == SWAP:
                    assert P in (16, 30, 32) and 2 <= TW <= P - 2 and TH >= 4, (w, h, cout, pool, P, TW, TH)
                    assert ncols == P * TH and ncols % 16 == 0 and ncols <= 256
                    assert P != 16 or ncols % 32 == 0
                    assert not pool or TH % 2 == 0
                    assert ncols + 2 * P + 2 <= 304
                    seen.add((SWAP, P))
                elif v == PAIR:
                    assert cout <= 64 and (P, TW, TH) in ((16, 14, 16), (30, 28, 8)) and ncols <= 256
                    seen.add((PAIR, P))
    assert {(SWAP, 16), (SWAP, 30), (SWAP, 32), (PAIR, 16), (PAIR, 30)} <= seen


def test_fused_concat_gather_keeps_its_source_alive():
    """A Slice -> Concat channel reorder in the middle of a network is evaluated by the Concat's gather kernel, which reads
    the Slices' source: the planner must not hand the source's buffer to the Concat (or to anything scheduled in between)."""
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        r = np.random.default_rng(1)
        x = dr.feed_node(g, [8, 8, 3])
        c1 = dr.Conv2d(x, [3, 3, 3, 4], [1, 1, 1, 1], "relu", r.standard_normal((3, 3, 3, 4)).astype(np.float32), np.zeros(4, np.float32))
        s1 = dr.Slice(c1, (0, 0, 2), (8, 8, 2))
        s0 = dr.Slice(c1, (0, 0, 0), (8, 8, 2))
        cat = dr.Concat([s1, s0], 2)
        c2 = dr.Conv2d(cat, [3, 3, 4, 4], [1, 1, 1, 1], "relu", r.standard_normal((3, 3, 4, 4)).astype(np.float32), np.zeros(4, np.float32))
        dr.mark_as_output(c2)
        dry_prepare(g)
        a = {k: dr.lib.dR_getNodeActAddress(v.ptr) for k, v in dict(c1=c1, s1=s1, s0=s0, cat=cat, c2=c2).items()}
        assert a["cat"] != a["c1"]
        assert a["s1"] != a["c1"] and a["s0"] != a["c1"]
        assert a["c2"] != a["cat"]
