"""GPU parity tests on whole graphs: the reference's pretrained SqueezeNet (known answers 292 / 611),
synthetic SqueezeNet and VGG-style graphs against the CPU oracle running the same saved model folder,
batching, fusion and CUDA-graph replay equivalence, and size-independent properties at the
benchmark's full layer sizes."""
import os

import numpy as np
import pytest

import cases
import deepracin_b200 as dr
import nets
import oracle
from gpu_helpers import TOL_FP32, conv_build, rel_err, run_graph
from oracle import graph as ograph

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz"))


def load_kat_images():
    d = oracle.staged_squeezenet_dir()
    return d, np.stack([np.fromfile(os.path.join(d, n + "_224x224x3_rgb_hwc.f32"), dtype=np.float32).reshape(224, 224, 3)
                        for n in ("tiger", "puzzle")])


@pytest.mark.skipif(oracle.staged_squeezenet_dir() is None, reason="pretrained SqueezeNet fixture not staged")
@pytest.mark.parametrize("opts", [dict(), dict(fuse=False), dict(cuda_graph=True), dict(conv_algo="direct"), dict(autotune=True),
                                  dict(math="tf32"), dict(math="tf32", cuda_graph=True), dict(math="tf32", feed_overlap=True)])
def test_pretrained_squeezenet_known_answers(opts):
    d, imgs = load_kat_images()
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = 2
        for k, v in opts.items():
            setattr(g, k, v)
        nodes, feeds = dr.load_graph(g, d)
        dr.mark_as_output(nodes[-1])
        dr.mark_as_output(nodes[-2])
        dr.prepare(g)
        dr.feed_data(feeds[0], imgs)
        probs, logits = dr.apply(g)
        probs2, _ = dr.apply(g)
    probs, logits = probs.reshape(2, 1000), logits.reshape(2, 1000)
    assert [int(p.argmax()) for p in probs] == [292, 611]
    assert np.array_equal(probs, probs2.reshape(2, 1000))
    tf32 = opts.get("math") == "tf32"
    for i, name in enumerate(("tiger", "puzzle")):
        # FP32 kernels: per-layer bound 1e-4; TF32 tensor-core layers: 3e-3 per layer, looser on the softmax
        assert rel_err(logits[i], GOLD["kat_%s_logits" % name]) <= (1e-2 if tf32 else TOL_FP32)
        assert rel_err(probs[i], GOLD["kat_%s_softmax" % name]) <= (5e-2 if tf32 else 5e-4)


def run_vs_oracle(build, feed_hwc, tmp_path, tol=TOL_FP32, **opts):
    """Builds the net, saves it with dR_saveGraph, runs it on the GPU and runs the saved folder on the oracle."""
    n = feed_hwc.shape[0]
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = n
        for k, v in opts.items():
            setattr(g, k, v)
        x, out = build(g)
        dr.mark_as_output(out)
        dr.save_graph(g, str(tmp_path))
        dr.prepare(g)
        dr.feed_data(x, feed_hwc)
        (got,) = dr.apply(g)
    onodes = ograph.parse_graph(str(tmp_path / "dr_graph_export"))
    ref = ograph.run_graph(onodes, [np.ascontiguousarray(feed_hwc.transpose(0, 3, 1, 2))])
    got = got.reshape(ref.shape) if got.size == ref.size and got.ndim != 4 else got
    return got, ref


def test_synthetic_squeezenet_matches_oracle(tmp_path):
    imgs = nets.synthetic_images("sq_img", 2, 64)
    got, ref = run_vs_oracle(lambda g: nets.squeezenet11(g, size=64, classes=40), imgs, tmp_path)
    got = got.reshape(ref.shape)
    assert np.all(np.isfinite(ref))
    assert rel_err(got, ref) <= 5e-4
    assert np.array_equal(got.reshape(2, -1).argmax(1), ref.reshape(2, -1).argmax(1))


def test_small_vgg_matches_oracle(tmp_path):
    imgs = nets.synthetic_images("vgg_img", 3, 32)
    got, ref = run_vs_oracle(lambda g: nets.vgg16(g, size=32, width_div=8, fc_dims=(512, 512, 100)), imgs, tmp_path)
    got = got.reshape(ref.shape)
    assert np.all(np.isfinite(ref))
    assert rel_err(got, ref) <= 5e-4
    assert np.array_equal(got.reshape(3, -1).argmax(1), ref.reshape(3, -1).argmax(1))


@pytest.mark.parametrize("math,bound", [("fp32", 3e-4), ("fp32x3", 3e-4), ("tf32", 2e-2)])
def test_mid_size_vgg_at_batch_16_in_every_math_mode(tmp_path, math, bound):
    """A VGG-16 of half width at batch 16 against the oracle running the saved folder: in FP32 mode the 3x3 layers are Winograd
    F(4x4,3x3) with its fused pooling, in the FP32-accurate tensor mode the deep layers are Winograd on the tensor cores and the
    FC layers three-pass split-K GEMMs, in TF32 mode everything dense is a tensor kernel.  Logits, 16 layers deep."""
    imgs = nets.synthetic_images("vgg_mid", 16, 32)
    got, ref = run_vs_oracle(lambda g: nets.vgg16(g, size=32, width_div=2, fc_dims=(512, 512, 100), softmax=False), imgs, tmp_path, math=math)
    got = got.reshape(ref.shape)
    assert np.all(np.isfinite(ref))
    assert rel_err(got, ref) <= bound
    assert np.array_equal(got.reshape(16, -1).argmax(1), ref.reshape(16, -1).argmax(1))


def test_small_vgg_logits_match_oracle_per_layer_bound(tmp_path):
    imgs = nets.synthetic_images("vgg_img2", 2, 32)
    got, ref = run_vs_oracle(lambda g: nets.vgg16(g, size=32, width_div=8, fc_dims=(512, 512, 100), softmax=False), imgs, tmp_path)
    assert rel_err(got.reshape(ref.shape), ref) <= 3e-4     # 16 layers deep; each layer is within 1e-4


def test_batch_equals_loop_over_images(tmp_path):
    """A batch of n is n independent applications (the reference's own notion of a batch)."""
    imgs = nets.synthetic_images("loop_img", 3, 32)

    def run(batch_imgs):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = batch_imgs.shape[0]
            x, out = nets.squeezenet11(g, size=32, classes=16)
            dr.mark_as_output(out)
            dr.prepare(g)
            dr.feed_data(x, batch_imgs)
            return dr.apply(g)[0].reshape(batch_imgs.shape[0], -1)
    whole = run(imgs)
    single = np.concatenate([run(imgs[i:i + 1]) for i in range(3)])
    assert rel_err(whole, single) <= 1e-6


def test_conv_sweep_layers_direct_vs_winograd_at_full_size():
    """Benchmark conv-sweep shapes at batch 32: both FP32 kernel families agree, and the linear layer is
    homogeneous (conv(2x) == 2 conv(x) exactly in binary floating point)."""
    for cin, hw in ((64, 56), (128, 28), (256, 14)):
        x, wt, b = cases.conv_case("sweep%d" % cin, 32, cin, cin, hw, hw, 3)
        (d,) = run_graph(conv_build(wt, b, 1, 1, algo="direct"), [x])
        (w,) = run_graph(conv_build(wt, b, 1, 1, algo="winograd"), [x])
        assert rel_err(w, d) <= 2e-4
        ref0 = oracle.conv2d(x[:1], wt, b, (1, 1), 1)
        assert rel_err(d[:1], ref0) <= TOL_FP32
        (lin1,) = run_graph(conv_build(wt, None, 1, 0, algo="direct"), [x[:4]])
        (lin2,) = run_graph(conv_build(wt, None, 1, 0, algo="direct"), [2.0 * x[:4]])
        assert np.array_equal(lin2, 2.0 * lin1)


def test_vgg_fc_stack_at_full_size():
    """FC 25088 -> 4096 at batch 1 and 8: weight-streaming kernel against the oracle."""
    g = cases.rng("fc6")
    w = (g.standard_normal((25088, 4096), dtype=np.float32) * np.float32(np.sqrt(2.0 / 25088)))
    b = (g.standard_normal(4096, dtype=np.float32) * np.float32(0.1))
    x = g.standard_normal((8, 512, 7, 7), dtype=np.float32)
    ref = oracle.fc(x, w, b, 1)
    for n in (1, 8):
        (got,) = run_graph(lambda gr, f: dr.Fully_Connected(f[0], [25088, 4096], "relu", w, b), [x[:n]])
        assert rel_err(got, ref[:n]) <= TOL_FP32


def test_overlapped_feeding_gives_the_same_results_in_order():
    """dR_setFeedOverlap: batches copied on the second stream while the previous batch computes."""
    import ctypes
    batches = [nets.synthetic_images("ovl%d" % i, 2, 32) for i in range(5)]
    outs = {}
    for overlap in (False, True):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 2
            g.feed_overlap = overlap
            x, out = nets.squeezenet11(g, size=32, classes=16)
            dr.mark_as_output(out)
            dr.prepare(g)
            n_in, n_out = 2 * 32 * 32 * 3, 2 * 16
            pin_in = [dr.lib.dR_allocPinned(n_in * 4) for _ in batches]
            pin_out = [dr.lib.dR_allocPinned(n_out * 4) for _ in batches]
            for p, b in zip(pin_in, batches):
                # the feed buffer is [C][H][W] per image (reference interface layout)
                chw = np.ascontiguousarray(b.transpose(0, 3, 1, 2))             # named: it must outlive the copy
                ctypes.memmove(p, chw.ctypes.data, n_in * 4)
            for i in range(len(batches)):       # no synchronisation between steps
                assert dr.lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in[i], n_in)
                assert dr.lib.dR_apply(g.ptr)
                assert dr.lib.dR_fetchOutputAsync(g.ptr, 0, pin_out[i], n_out)
            dr.lib.dR_synchronize(g.ptr)
            outs[overlap] = [np.ctypeslib.as_array((ctypes.c_float * n_out).from_address(p)).copy() for p in pin_out]
            for p in pin_in + pin_out:
                dr.lib.dR_freePinned(p)
    for a, b in zip(outs[False], outs[True]):
        assert np.array_equal(a, b)
    assert not np.array_equal(outs[True][0], outs[True][1])


def test_full_size_vgg16_fp32_matches_reference_kernels_and_tf32_agrees(tmp_path):
    """VGG-16 at its real size (224x224, 13 conv + 3 FC): the FP32 path against the CPU oracle running the same
    saved model (the reference's own kernels where the reference-built library is present), and the TF32
    tensor-core path against the FP32 path: logits within the TF32 bound, same top-1."""
    imgs = nets.synthetic_images("vgg_full", 2, 224)
    res = {}
    for math in ("fp32", "tf32"):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 2
            g.math = math
            x, out = nets.vgg16(g, size=224, softmax=False)
            dr.mark_as_output(out)
            if math == "fp32":
                dr.save_graph(g, str(tmp_path))
            dr.prepare(g)
            dr.feed_data(x, imgs)
            res[math] = dr.apply(g)[0].reshape(2, 1000)
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
    onodes = ograph.parse_graph(str(tmp_path / "dr_graph_export"))
    ref = ograph.run_graph(onodes, [np.ascontiguousarray(imgs[:1].transpose(0, 3, 1, 2))], leg="ref").reshape(1, 1000)
    assert np.all(np.isfinite(ref))
    assert rel_err(res["fp32"][:1], ref) <= 5e-4                 # 16 layers, each within 1e-4
    assert rel_err(res["tf32"], res["fp32"]) <= 1e-2             # 13 TF32 layers deep; per layer 3e-3
    assert np.array_equal(res["tf32"].argmax(1), res["fp32"].argmax(1))


@pytest.mark.parametrize("fuse", [True, False])
def test_channel_reorder_in_the_middle_of_a_network(fuse):
    """conv -> {Slice(ch 2..3), Slice(ch 0..1) - 0.5} -> Concat -> conv: with fusion on the Concat's gather kernel reads the
    first convolution's output directly, so that buffer must stay alive (and distinct from the Concat's) until then."""
    x, w1, b1 = cases.conv_case("reorder_c1", 3, 3, 4, 9, 11, 3)
    _, w2, b2 = cases.conv_case("reorder_c2", 1, 4, 6, 9, 11, 3)
    a = oracle.conv2d(x, w1, b1, (1, 1), 1)
    mid = np.concatenate([a[:, 2:4], a[:, 0:2] - np.float32(0.5)], axis=1)
    ref = oracle.conv2d(mid, w2, b2, (1, 1), 1)

    def build(g, f):
        c1 = conv_build(w1, b1, 1, 1)(g, f)
        hi = dr.Slice(c1, (2, 0, 0), (2, 9, 11))
        lo = dr.Sub_Scalar(dr.Slice(c1, (0, 0, 0), (2, 9, 11)), 0.5)
        return conv_build(w2, b2, 1, 1)(g, [dr.Concat([hi, lo], 0)])
    (got,) = run_graph(build, [x], fuse=fuse)
    assert rel_err(got, ref) <= 2 * TOL_FP32


@pytest.mark.parametrize("overlap", [False, True])
def test_8bit_feed_equals_float_feed(overlap):
    """dR_feedDataU8Async: image bytes cross the host link, the cast to float runs on the device; results are bit-identical
    to feeding the same samples as floats, with and without double-buffered feeding, over several batches in a row."""
    import ctypes
    rng = np.random.default_rng(11)
    batches = [rng.integers(0, 256, size=(2, 32, 32, 3), dtype=np.uint8) for _ in range(4)]
    outs = {}
    for mode in ("float", "u8"):
        with dr.Environment() as env:
            g = env.create_graph("HWC")
            g.batch = 2
            g.math = "tf32"
            g.feed_overlap = overlap
            x, out = nets.squeezenet11(g, size=32, classes=16)
            dr.mark_as_output(out)
            dr.lib.dR_setInterfaceLayout(g.ptr, 1)
            dr.prepare(g)
            n_in, n_out = 2 * 32 * 32 * 3, 2 * 16
            pin_out = [dr.lib.dR_allocPinned(n_out * 4) for _ in batches]
            pin_in = [dr.lib.dR_allocPinned(n_in * 4) for _ in batches]
            for p, b in zip(pin_in, batches):
                if mode == "u8":
                    ctypes.memmove(p, b.ctypes.data, n_in)
                else:
                    as_float = np.ascontiguousarray(b.astype(np.float32))      # named: it must outlive the copy
                    ctypes.memmove(p, as_float.ctypes.data, n_in * 4)
            for i in range(len(batches)):
                if mode == "u8":
                    assert dr.lib.dR_feedDataU8Async(g.ptr, x.ptr, pin_in[i], n_in)
                else:
                    assert dr.lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in[i], n_in)
                assert dr.lib.dR_apply(g.ptr)
                assert dr.lib.dR_fetchOutputAsync(g.ptr, 0, pin_out[i], n_out)
            dr.lib.dR_synchronize(g.ptr)
            assert not dr.lib.dR_feedDataU8Async(g.ptr, x.ptr, pin_in[0], n_in - 1)      # wrong size is refused
            outs[mode] = [np.ctypeslib.as_array((ctypes.c_float * n_out).from_address(p)).copy() for p in pin_out]
            assert dr.lib.dR_getDeviceStatus(g.ptr) == 0
            for p in pin_in + pin_out:
                dr.lib.dR_freePinned(p)
    for a, b in zip(outs["float"], outs["u8"]):
        assert np.array_equal(a, b)
    assert not np.array_equal(outs["u8"][0], outs["u8"][1])
