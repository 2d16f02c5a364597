"""Build the CPU oracle libraries -- TEST INFRASTRUCTURE ONLY.

* ``oracle/libdroracle.so``   : the plain-C restatement (``dr_oracle.c``).
* ``oracle/_ref/libdrref.so`` : the reference's own kernel sources compiled as C through
  ``ref_shim/`` -- built only where a reference checkout is present (``DR_REF_DIR``, or a folder
  named ``reference`` beside this repository); the kernel files are compiled where they lie and
  are never copied.
* ``oracle/_ref/squeezenet/`` : the reference's pretrained SqueezeNet model folder and its two
  example images (as raw float32 W x H x 3 arrays), staged for the known-answer test.
* ``oracle/_ref/python/__init__.py.in`` : the reference's Python ctypes module, staged so that the tests can
  render it against ``libdeepracin.so`` and drive the library through the reference's own binding.

Run ``python oracle/build_oracle.py``.  Building the checker is not using it.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("DR_REF_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
CFLAGS = ["-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_restatement(force=False):
    src = os.path.join(HERE, "dr_oracle.c")
    out = os.path.join(HERE, "libdroracle.so")
    if force or _newer(out, [src]):
        # no -ffast-math: the restatement accumulates in double and must stay order-independent
        subprocess.check_call(["gcc", "-std=gnu99", *CFLAGS, src, "-o", out, "-lm"])
    return out


def build_reference_leg(force=False):
    """Compile the reference kernels in place; returns the .so path or None if no checkout."""
    kdir = os.path.join(REF_DIR, "Kernels")
    gdir = os.path.join(REF_DIR, "examples", "squeezenet-v1.1", "squeezenet_whole")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libdrref.so")
    if not os.path.isdir(kdir):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    src = os.path.join(HERE, "ref_shim", "ref_driver.c")
    if force or _newer(out, [src, os.path.join(HERE, "ref_shim", "cl_shim.h")]):
        # -ffast-math mirrors the reference's default -cl-fast-relaxed-math -cl-mad-enable
        subprocess.check_call(["gcc", "-std=gnu99", "-x", "c", *CFLAGS, "-ffast-math", "-w",
                               "-I", os.path.join(HERE, "ref_shim"), "-I", kdir, "-I", gdir,
                               src, "-o", out, "-lm"])
    return out


def stage_reference_fixtures():
    """Copy the pretrained SqueezeNet model folder and decode the two example PNGs."""
    ex = os.path.join(REF_DIR, "examples", "squeezenet-v1.1")
    dst = os.path.join(HERE, "_ref", "squeezenet")
    if not os.path.isdir(ex):
        return dst if os.path.isdir(dst) else None
    os.makedirs(dst, exist_ok=True)
    src_model = os.path.join(ex, "squeezenet_whole")
    for name in os.listdir(src_model):
        if name == "graph.dr" or name.endswith(".var"):
            target = os.path.join(dst, name)
            if not os.path.exists(target):
                shutil.copyfile(os.path.join(src_model, name), target)
    try:
        import numpy as np
        from PIL import Image
        for img in ("tiger", "puzzle"):
            target = os.path.join(dst, img + "_224x224x3_rgb_hwc.f32")
            if not os.path.exists(target):
                a = np.asarray(Image.open(os.path.join(ex, img + ".png")).convert("RGB"), dtype=np.float32)
                a.tofile(target)
    except ImportError:
        pass
    pysrc = os.path.join(REF_DIR, "python", "deepracin", "__init__.py.in")
    if os.path.exists(pysrc):
        os.makedirs(os.path.join(HERE, "_ref", "python"), exist_ok=True)
        shutil.copyfile(pysrc, os.path.join(HERE, "_ref", "python", "__init__.py.in"))
    return dst


def build_all(force=False):
    build_restatement(force)
    build_reference_leg(force)
    stage_reference_fixtures()


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle built")
