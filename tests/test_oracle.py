"""CPU tests that pin the oracle: the plain-C restatement against (a) golden vectors produced by the
reference's own kernel sources, (b) those kernels run live where the reference-built library is
present, and (c) the reference's only known answers (SqueezeNet -> classes 292 / 611)."""
import os

import numpy as np
import pytest

import cases
import oracle
from oracle import graph

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz"))
TOL = 1e-4  # max|err| <= TOL * max|ref| : the fp32 parity bound of this project


def rel_err(got, ref):
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64))) / max(float(np.max(np.abs(ref))), 1e-30))


def restate(name):
    kind, kw = cases.GOLDEN_CASES[name]
    ins = cases.make_inputs(name)
    if kind in ("wino", "c1x1"):
        return oracle.conv2d(ins[0], ins[1], ins[2], (1, 1), kw["act"])
    if kind == "fc":
        return oracle.fc(ins[0], ins[1], ins[2], kw["act"])
    if kind == "pool":
        return oracle.pool(ins[0], (kw["k"], kw["k"], 1), (kw["stride"], kw["stride"], 1), kw["kind"])
    if kind == "softmax":
        return oracle.softmax(ins[0])
    raise KeyError(kind)


@pytest.mark.parametrize("name", [n for n, (k, _) in cases.GOLDEN_CASES.items() if k in ("wino", "c1x1", "fc", "pool", "softmax")])
def test_restatement_matches_reference_kernel_golden(name):
    got = restate(name)
    ref = GOLD[name]
    assert got.shape == ref.shape
    kind = cases.GOLDEN_CASES[name][0]
    if kind == "pool" and cases.GOLDEN_CASES[name][1]["kind"] == 0:
        assert np.array_equal(got, ref)          # max pooling is exact
    else:
        assert rel_err(got, ref) <= TOL


def test_winograd_restatement_matches_golden():
    for name, (kind, kw) in cases.GOLDEN_CASES.items():
        if kind != "wino":
            continue
        x, w, b = cases.make_inputs(name)
        assert rel_err(oracle.conv2d_winograd(x, w, b, kw["act"]), GOLD[name]) <= TOL


def test_elementwise_and_copies_match_golden():
    (x,) = cases.make_inputs("ew1_all")
    for op, s in cases.EW1_OPS:
        assert rel_err(oracle.elemwise1(x, op, s), GOLD["ew1_all_op%d" % op]) <= 1e-6
    a, b = cases.make_inputs("ew2_all")
    for op in cases.EW2_OPS:
        assert rel_err(oracle.elemwise2(a, b, op), GOLD["ew2_all_op%d" % op]) <= 1e-6
    (x,) = cases.make_inputs("slice_crop")
    assert np.array_equal(oracle.slice_(x, (2, 1, 1), (5, 6, 3)), GOLD["slice_crop_slice"])
    assert np.array_equal(oracle.croporpad(x, (11, 12, 6)), GOLD["slice_crop_pad"])
    assert np.array_equal(oracle.croporpad(x, (5, 4, 6)), GOLD["slice_crop_crop"])


def test_concat_restatement():
    a = cases.act_case("cat_a", 2, 3, 4, 5)
    b = cases.act_case("cat_b", 2, 2, 4, 5)
    assert np.array_equal(oracle.concat([a, b], 2), np.concatenate([a, b], axis=1))
    c = cases.act_case("cat_c", 2, 3, 4, 2)
    assert np.array_equal(oracle.concat([a, c], 0), np.concatenate([a, c], axis=3))


def test_strided_conv_against_numpy_definition():
    """out[o,y,x] = sum in[i, y*s+ky-1, x*s+kx-1] w[i,o,ky,kx] -- the documented formula, stride 2."""
    x, w, b = cases.conv_case("stride2", 1, 3, 4, 9, 8, 3)
    got = oracle.conv2d(x, w, b, (2, 2), act=0)
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (1, 1), (1, 1)))
    ref = np.zeros((1, 4, 4, 4))
    for o in range(4):
        for y in range(4):
            for xx in range(4):
                ref[0, o, y, xx] = b[o] + np.sum(xp[0, :, 2 * y:2 * y + 3, 2 * xx:2 * xx + 3] * w[:, o].astype(np.float64))
    assert got.shape == (1, 4, 4, 4)
    assert rel_err(got, ref) <= 1e-6


@pytest.mark.skipif(not oracle.ref_available(), reason="reference-built kernel library not present")
def test_live_reference_kernels_match_golden_and_restatement():
    for name, (kind, kw) in cases.GOLDEN_CASES.items():
        ins = cases.make_inputs(name)
        if kind == "wino":
            live = oracle.ref_conv2d_winograd(ins[0], ins[1], ins[2], kw["act"])
        elif kind == "c1x1":
            live = oracle.ref_conv2d_1x1(ins[0], ins[1], ins[2], kw["act"])
        elif kind == "fc":
            live = oracle.ref_fc(ins[0], ins[1], ins[2], kw["act"])
        else:
            continue
        assert rel_err(live, GOLD[name]) <= 1e-6
        assert rel_err(live, restate(name)) <= TOL


@pytest.mark.skipif(not oracle.ref_available(), reason="reference-built kernel library not present")
def test_reference_schedule_variants_agree():
    """Different emulated device limits change work-group shapes / summation order only."""
    x, w, b = cases.conv_case("sched", 1, 64, 64, 16, 16, 3)
    a = oracle.ref_conv2d_winograd(x, w, b, 1, lms=48 * 1024, mws=1024)
    c = oracle.ref_conv2d_winograd(x, w, b, 1, lms=32 * 1024, mws=256)
    assert rel_err(a, c) <= 1e-5
    assert rel_err(a, oracle.conv2d(x, w, b, (1, 1), 1)) <= TOL


@pytest.mark.skipif(oracle.staged_squeezenet_dir() is None, reason="pretrained SqueezeNet fixture not staged")
@pytest.mark.parametrize("img,cls", [("tiger", 292), ("puzzle", 611)])
def test_squeezenet_known_answer(img, cls):
    d = oracle.staged_squeezenet_dir()
    nodes = graph.parse_graph(d)
    a = np.fromfile(os.path.join(d, img + "_224x224x3_rgb_hwc.f32"), dtype=np.float32).reshape(224, 224, 3)
    x = np.ascontiguousarray(a.transpose(2, 0, 1))[None]
    y = graph.run_graph(nodes, [x], leg="restate").reshape(1000)
    assert int(y.argmax()) == cls
    assert rel_err(y, GOLD["kat_%s_softmax" % img]) <= 1e-4


def test_known_answer_golden_vectors_hold_the_reference_classes():
    assert int(GOLD["kat_tiger_softmax"].argmax()) == 292
    assert int(GOLD["kat_puzzle_softmax"].argmax()) == 611
