"""The batch-sharded replica interface of the C library (include/dR_replicas.h): one graph, one host thread and one device
per replica, host-side scatter / gather, no collective.  A C program compiled against include/ drives it (planning without a
device on CPU, the pretrained SqueezeNet on a GPU -- two replicas may share device 0 where only one GPU is present), and a
ctypes test checks that R replicas of batch b give bit-for-bit what one graph of batch R*b gives."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import deepracin_b200 as dr
import nets
import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "deepracin_b200", "libdeepracin.so")
needs_model = pytest.mark.skipif(oracle.staged_squeezenet_dir() is None, reason="pretrained SqueezeNet fixture not staged")


def build_client(tmp_path):
    exe = str(tmp_path / "replicas_client")
    src = os.path.join(ROOT, "tests", "c_client", "replicas_client.c")
    r = subprocess.run(["gcc", "-std=gnu99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-L", os.path.dirname(LIB), "-ldeepracin",
                        "-Wl,-rpath," + os.path.dirname(LIB), "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@needs_model
def test_replicas_plan_without_a_device(tmp_path):
    exe = build_client(tmp_path)
    r = subprocess.run([exe, oracle.staged_squeezenet_dir(), "3", "0", "1", "2", "--dry-run"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "replicas 3 global batch 3" in r.stdout and "dry run ok" in r.stdout


def test_replicas_reject_bad_arguments():
    lib = dr.lib
    lib.dR_replicasLoad.restype = ctypes.c_void_p
    lib.dR_replicasLoad.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
    assert not lib.dR_replicasLoad(0, None, 1, b"/nonexistent", 0, 0)
    assert not lib.dR_replicasLoad(2, None, 0, b"/nonexistent", 0, 0)
    assert not lib.dR_replicasLoad(1, None, 1, None, 0, 0)


@pytest.mark.gpu
@needs_model
def test_replicas_classify_the_reference_images(tmp_path):
    exe = build_client(tmp_path)
    d = oracle.staged_squeezenet_dir()
    imgs = [os.path.join(d, n + "_224x224x3_rgb_hwc.f32") for n in ("tiger", "puzzle")]
    import torch
    second = "1" if torch.cuda.device_count() >= 2 else "0"
    r = subprocess.run([exe, d, "2", "0", second] + imgs, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    classes = [int(line.split()[1]) for line in r.stdout.splitlines() if line.startswith("class ")]
    assert classes == [292, 611, 292, 611]


@pytest.mark.gpu
def test_replicas_equal_one_graph_on_the_whole_batch(tmp_path):
    """2 replicas x batch 2 (on devices 0 and 1 where the box has two GPUs, else both on device 0) against one graph at batch 4 on
    the same saved model: identical outputs."""
    lib = dr.lib
    imgs = nets.synthetic_images("replicas_c", 4, 32)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = 4
        g.math = "tf32"
        x, out = nets.squeezenet11(g, size=32, classes=16)
        dr.mark_as_output(out)
        dr.save_graph(g, str(tmp_path))
        lib.dR_setInterfaceLayout(g.ptr, 1)
        dr.prepare(g)
        lib.dR_feedData(g.ptr, x.ptr, imgs.ctypes.data_as(dr._FP), 0, imgs.size)
        assert lib.dR_apply(g.ptr)
        whole = np.empty((4, 16), np.float32)
        bufs = (ctypes.c_void_p * 1)()
        assert lib.dR_getOutputBuffers(g.ptr, bufs) == 1
        lib.dR_downloadArray(g.ptr, b"", bufs[0], 0, whole.nbytes, whole.ctypes.data_as(ctypes.c_void_p))
    lib.dR_replicasLoad.restype = ctypes.c_void_p
    lib.dR_replicasLoad.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
    lib.dR_replicasApply.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    lib.dR_replicasDestroy.argtypes = [ctypes.c_void_p]
    lib.dR_replicasInputFloatsPerImage.restype = ctypes.c_size_t
    lib.dR_replicasInputFloatsPerImage.argtypes = [ctypes.c_void_p]
    import torch
    ordinals = (ctypes.c_int * 2)(0, 1 if torch.cuda.device_count() >= 2 else 0)
    print("replica devices:", list(ordinals))
    r = lib.dR_replicasLoad(2, ordinals, 2, str(tmp_path / "dr_graph_export").encode(), 1, 1)
    assert r
    assert lib.dR_replicasInputFloatsPerImage(r) == 32 * 32 * 3
    got = np.zeros((4, 16), np.float32)
    ms = ctypes.c_double(0.0)
    assert lib.dR_replicasApply(r, imgs.ctypes.data_as(ctypes.c_void_p), got.ctypes.data_as(ctypes.c_void_p), 3, ctypes.byref(ms))
    assert ms.value > 0.0
    lib.dR_replicasDestroy(r)
    assert np.array_equal(got, whole)
