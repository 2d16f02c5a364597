"""The drop-in boundary driven by the reference's own two callers instead of this repository's mirror of them:

* the reference's Python ctypes module (python/deepracin/__init__.py.in), rendered exactly as its build system would
  (the two ``${CMAKE_INSTALL_PREFIX}`` library paths at :11-14 substituted) and imported against ``libdeepracin.so``:
  every symbol it binds at import (:36-218) must exist, its layer constructors (:546, :603, :834, :900), its HWC <-> CHW
  handling on feed / fetch (:444-465, :487-489) and its weight transposes (:559-562) must give the right numbers;
* a C program in the style of examples/squeezenet-v1.1/squeezenet_deployed.c:95-207, compiled here with a C compiler
  against ``include/`` and linked to the library.

The module template is staged (never committed) by oracle/build_oracle.py where a reference checkout exists; the tests
skip without it.  CPU tests plan the graphs without a device (dR_setDryRun); GPU tests compute."""
import ctypes
import importlib.util
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "deepracin_b200", "libdeepracin.so")
needs_module = pytest.mark.skipif(oracle.staged_reference_python_module() is None, reason="reference Python module not staged")
needs_model = pytest.mark.skipif(oracle.staged_squeezenet_dir() is None, reason="pretrained SqueezeNet fixture not staged")


def load_reference_module(tmp_path):
    """Renders __init__.py.in with an install prefix under tmp_path that holds lib/deepracin/libdeepracin.so."""
    prefix = tmp_path / "prefix"
    libdir = prefix / "lib" / "deepracin"
    libdir.mkdir(parents=True, exist_ok=True)
    if not (libdir / "libdeepracin.so").exists():
        os.symlink(LIB, libdir / "libdeepracin.so")
    text = open(oracle.staged_reference_python_module()).read()
    assert text.count("${CMAKE_INSTALL_PREFIX}") == 2
    pkg = tmp_path / "deepracin"
    pkg.mkdir(exist_ok=True)
    (pkg / "__init__.py").write_text(text.replace("${CMAKE_INSTALL_PREFIX}", str(prefix)))
    spec = importlib.util.spec_from_file_location("deepracin_reference_binding", str(pkg / "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)        # binds every dR_* symbol the reference's Python layer uses
    return mod


def small_net(mod, graph, seed=3):
    r = np.random.default_rng(seed)
    w1 = (r.standard_normal((3, 3, 3, 8)) * 0.3).astype(np.float32)
    b1 = (r.standard_normal(8) * 0.1).astype(np.float32)
    w2 = (r.standard_normal((1, 1, 8, 16)) * 0.3).astype(np.float32)
    b2 = (r.standard_normal(16) * 0.1).astype(np.float32)
    wf = (r.standard_normal((5 * 6 * 16, 10)) * 0.1).astype(np.float32)
    bf = (r.standard_normal(10) * 0.1).astype(np.float32)
    x = mod.feed_node(graph, [10, 12, 3])                                       # H, W, C
    c1 = mod.Conv2d(x, [3, 3, 3, 8], [1, 1, 1, 1], "relu", w1, b1)
    c2 = mod.Conv2d(c1, [1, 1, 8, 16], [1, 1, 1, 1], "relu", w2, b2)
    p = mod.Pooling(c2, "max", [1, 2, 2, 1], [1, 2, 2, 1])
    fc = mod.Fully_Connected(p, [5 * 6 * 16, 10], "linear", wf, bf)
    sm = mod.Softmax(fc)
    mod.mark_as_output(sm)
    mod.mark_as_output(p)
    return x, (w1, b1, w2, b2, wf, bf)


def small_net_oracle(img_hwc, params):
    w1, b1, w2, b2, wf, bf = params
    x = np.ascontiguousarray(img_hwc.transpose(2, 0, 1))[None]
    a = oracle.conv2d(x, np.ascontiguousarray(w1.transpose(2, 3, 0, 1)), b1, (1, 1), 1)
    a = oracle.conv2d(a, np.ascontiguousarray(w2.transpose(2, 3, 0, 1)), b2, (1, 1), 1)
    p = oracle.pool(a, (2, 2, 1), (2, 2, 1), 0)
    f = oracle.fc(p, wf, bf, 0)
    return oracle.softmax(f).reshape(-1), p[0].transpose(1, 2, 0)


@needs_module
def test_reference_python_module_imports_and_plans_a_graph(tmp_path):
    mod = load_reference_module(tmp_path)
    mod.lib.dR_setDryRun.argtypes = [ctypes.c_void_p, ctypes.c_int]
    mod.lib.dR_setDryRun.restype = ctypes.c_int
    with mod.Environment() as env:
        graph = env.create_graph("HWC")
        assert mod.lib.dR_setDryRun(graph.ptr, 1)
        small_net(mod, graph)
        mod.prepare(graph)
        assert graph.outnodes[0].out_shape == [10, 1, 1]
        assert graph.outnodes[1].out_shape == [6, 5, 16]            # (W, H, C) after the 2x2/2 pool
        assert graph.feed_nodes[0].shape == [12, 10, 3]
        with pytest.raises(RuntimeError):
            mod.apply(graph)                                        # a dry run never computes
        # save through the reference's wrapper, load into a second graph through it as well
        mod.save_graph(graph, str(tmp_path / "m"))
        g2 = env.create_graph("HWC")
        nodes, feeds = mod.load_graph(g2, str(tmp_path / "m" / "dr_graph_export"))
        assert len(nodes) == 6 and len(feeds) == 1


@needs_module
def test_reference_python_module_stub_constructors_fail_cleanly(tmp_path):
    """Layers outside this build are exported so that the module imports; calling one reports failure, it does not crash."""
    mod = load_reference_module(tmp_path)
    with mod.Environment() as env:
        graph = env.create_graph("HWC")
        x = mod.feed_node(graph, [8, 8, 3])
        assert mod.RGB_to_gray(x).ptr is None               # NULL node, message on stdout, no crash
        assert x.ptr is not None


@pytest.mark.gpu
@needs_module
def test_reference_python_module_runs_a_graph_on_the_gpu(tmp_path):
    mod = load_reference_module(tmp_path)
    img = (np.random.default_rng(5).random((10, 12, 3), dtype=np.float32) * 2 - 1).astype(np.float32)
    with mod.Environment() as env:
        graph = env.create_graph("HWC")
        x, params = small_net(mod, graph)
        mod.prepare(graph)
        mod.feed_data(x, img)
        probs, pooled = mod.apply(graph)
    ref_probs, ref_pooled = small_net_oracle(img, params)
    assert np.max(np.abs(probs.reshape(-1) - ref_probs)) <= 1e-4 * np.max(np.abs(ref_probs))
    assert pooled.shape == ref_pooled.shape
    assert np.max(np.abs(pooled - ref_pooled)) <= 1e-4 * np.max(np.abs(ref_pooled))


@pytest.mark.gpu
@needs_module
@needs_model
def test_reference_python_module_pretrained_squeezenet_known_answers(tmp_path):
    """The reference's only golden answers (examples/squeezenet-v1.1/squeezenet_deployed.c:199-207) through its own binding."""
    mod = load_reference_module(tmp_path)
    d = oracle.staged_squeezenet_dir()
    with mod.Environment() as env:
        graph = env.create_graph("HWC")
        nodes, feeds = mod.load_graph(graph, d)
        mod.mark_as_output(nodes[-1])
        mod.prepare(graph)
        got = []
        for name in ("tiger", "puzzle", "tiger"):
            img = np.fromfile(os.path.join(d, name + "_224x224x3_rgb_hwc.f32"), dtype=np.float32).reshape(224, 224, 3)
            mod.feed_data(feeds[0], img)
            (probs,) = mod.apply(graph)
            got.append(int(np.argmax(probs)))
    assert got == [292, 611, 292]


# ------------------------------------------------------------------------------------------------ C caller
def build_c_client(tmp_path):
    exe = str(tmp_path / "squeezenet_client")
    src = os.path.join(ROOT, "tests", "c_client", "squeezenet_client.c")
    cmd = ["gcc", "-std=gnu99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-L", os.path.dirname(LIB), "-ldeepracin",
           "-Wl,-rpath," + os.path.dirname(LIB), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@needs_model
def test_c_client_compiles_against_the_headers_and_plans_the_pretrained_model(tmp_path):
    exe = build_c_client(tmp_path)
    r = subprocess.run([exe, oracle.staged_squeezenet_dir(), "--dry-run"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "nodes 48 feeds 1 in 224x224x3 out 1x1x1000" in r.stdout
    assert "dry run ok" in r.stdout


@pytest.mark.gpu
@needs_model
def test_c_client_classifies_the_reference_images(tmp_path):
    exe = build_c_client(tmp_path)
    d = oracle.staged_squeezenet_dir()
    imgs = [os.path.join(d, n + "_224x224x3_rgb_hwc.f32") for n in ("tiger", "puzzle", "tiger", "puzzle")]
    r = subprocess.run([exe, d] + imgs, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    classes = [int(line.split()[1]) for line in r.stdout.splitlines() if line.startswith("class ")]
    assert classes == [292, 611, 292, 611]
