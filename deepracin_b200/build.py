"""Builds ``libdeepracin.so`` (C host API + CUDA sm_100a kernels) in-tree with nvcc.

``python deepracin_b200/build.py`` (a plain script: importing the package needs the library to exist).  Objects go to ``deepracin_b200/build/``,
the shared library to ``deepracin_b200/libdeepracin.so``.  nvcc cross-compiles without a GPU.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libdeepracin.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CSRC, "kernels")]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.c")) + glob.glob(os.path.join(CSRC, "*.cu")) +
                  glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def _headers():
    return glob.glob(os.path.join(ROOT, "include", "*.h")) + glob.glob(os.path.join(CSRC, "kernels", "*.cuh"))


def _compile(src, obj, verbose):
    cmd = [NVCC, *ARCH, *COMMON, "-c", src, "-o", obj]
    if src.endswith(".cu"):
        cmd += ["-std=c++17", "-Xptxas", "-v"] if verbose else ["-std=c++17"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return r.stderr


def build_library(force=False, verbose=False):
    bdir = os.path.join(PKG, "build")
    os.makedirs(bdir, exist_ok=True)
    hdr_time = max(os.path.getmtime(h) for h in _headers())
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(bdir, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            jobs.append((src, obj))
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=8) as ex:
            logs = list(ex.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    if jobs or not os.path.exists(OUT):
        cmd = [NVCC, *ARCH, "-shared", "-o", OUT, *objs, "-lcudart", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    if verbose:
        for log in logs:
            sys.stderr.write(log)
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
