import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200 box)")


def _ensure_built():
    """CPU-side artefacts the tests need: the oracle libraries and libdeepracin.so."""
    from oracle import build_oracle
    build_oracle.build_all()
    lib = os.path.join(ROOT, "deepracin_b200", "libdeepracin.so")
    if not os.path.exists(lib):
        import importlib.util
        spec = importlib.util.spec_from_file_location("dr_build", os.path.join(ROOT, "deepracin_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_library()


_ensure_built()
