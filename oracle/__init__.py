"""CPU oracle for the deepRacin CNN-layer hot path -- TEST INFRASTRUCTURE ONLY.

Two legs, both CPU:

* ``restate``  -- ``libdroracle.so`` (``dr_oracle.c``): a plain-C restatement of every op,
  double accumulation, handles batches and true strided convolution.
* ``ref``      -- ``_ref/libdrref.so`` (``ref_shim/ref_driver.c``): the reference's own OpenCL C
  kernel sources compiled as C and run under an NDRange emulator with the reference's own
  launch geometry.  Present only after ``build_oracle.py`` ran where a reference checkout exists
  (the built library travels with the working tree; the sources do not).

All tensors are numpy float32 in the reference's interface layout: ``[n, C, H, W]`` ("z major,
x minor"), conv weights ``[Cin, Cout, kh, kw]``, fully connected weights ``[Nin, Nout]`` with the
input flattened in (y, x, z) order.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package; the
shipped library never does.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = ctypes.POINTER(ctypes.c_float)
_restate = None
_ref = None

# emulated OpenCL device limits used for the reference leg's scheduling arithmetic
# (CL_DEVICE_LOCAL_MEM_SIZE / CL_DEVICE_MAX_WORK_GROUP_SIZE of an NVIDIA-like device)
REF_LMS = 48 * 1024
REF_MWS = 1024


def _p(a):
    return a.ctypes.data_as(_F) if a is not None else None


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n=None):
    """OpenMP thread count of the oracle libraries (default: all host cores).  Launchers such as torchrun
    export OMP_NUM_THREADS=1, which would silently make the CPU baseline single-threaded."""
    n = int(n or os.cpu_count() or 1)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass
    return n


def restate_lib():
    global _restate
    if _restate is None:
        path = os.path.join(_HERE, "libdroracle.so")
        if not os.path.exists(path):
            from . import build_oracle
            build_oracle.build_restatement()
        _restate = ctypes.CDLL(path)
    return _restate


def ref_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libdrref.so"))


def ref_lib():
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libdrref.so")
        if not os.path.exists(path):
            raise RuntimeError("reference-kernel oracle not built (needs a reference checkout): " + path)
        _ref = ctypes.CDLL(path)
    return _ref


def staged_squeezenet_dir():
    d = os.path.join(_HERE, "_ref", "squeezenet")
    return d if os.path.exists(os.path.join(d, "graph.dr")) else None


def staged_reference_python_module():
    """Path of the reference's Python ctypes module template (python/deepracin/__init__.py.in) if it was staged."""
    p = os.path.join(_HERE, "_ref", "python", "__init__.py.in")
    return p if os.path.exists(p) else None


# --------------------------------------------------------------------------- restatement leg
def conv2d(x, w, b, stride=(1, 1), act=1):
    x, w, b = _c(x), _c(w), _c(b)
    n, cin, h, wd = x.shape
    _, cout, kh, kw = w.shape
    sx, sy = stride
    out = np.empty((n, cout, h // sy, wd // sx), np.float32)
    restate_lib().dro_conv2d(_p(x), n, wd, h, cin, _p(w), _p(b), kw, kh, cout, sx, sy, int(act), _p(out))
    return out


def conv2d_winograd(x, w, b, act=1):
    x, w, b = _c(x), _c(w), _c(b)
    n, cin, h, wd = x.shape
    cout = w.shape[1]
    out = np.empty((n, cout, h, wd), np.float32)
    restate_lib().dro_conv2d_winograd(_p(x), n, wd, h, cin, _p(w), _p(b), cout, int(act), _p(out))
    return out


def fc(x, w, b, act=1):
    x, w, b = _c(x), _c(w), _c(b)
    n, c, h, wd = x.shape
    nout = w.shape[1]
    out = np.empty((n, 1, 1, nout), np.float32)     # the reference's FC output shape is (W=Nout, H=1, C=1)
    restate_lib().dro_fc(_p(x), n, wd, h, c, _p(w), _p(b), nout, int(act), _p(out))
    return out


def pool(x, size, stride, kind):
    """size/stride = (x, y, z); kind 0 max, 1 average."""
    x = _c(x)
    n, c, h, wd = x.shape
    sx, sy, sz = size
    stx, sty, stz = stride
    out = np.empty((n, -(-c // stz), -(-h // sty), -(-wd // stx)), np.float32)
    restate_lib().dro_pool(_p(x), n, wd, h, c, sx, sy, sz, stx, sty, stz, int(kind), _p(out))
    return out


def softmax(x):
    x = _c(x)
    out = np.empty_like(x)
    n = x.shape[0]
    restate_lib().dro_softmax(_p(x), n, x.size // n, _p(out))
    return out


def elemwise1(x, op, scalar=0.0):
    x = _c(x)
    out = np.empty_like(x)
    restate_lib().dro_elemwise1(_p(x), ctypes.c_size_t(x.size), int(op), ctypes.c_float(scalar), _p(out))
    return out


def elemwise2(a, b, op):
    a, b = _c(a), _c(b)
    out = np.empty_like(a)
    restate_lib().dro_elemwise2(_p(a), _p(b), ctypes.c_size_t(a.size), int(op), _p(out))
    return out


def slice_(x, origin, shape):
    """origin/shape = (x, y, z)."""
    x = _c(x)
    n, c, h, wd = x.shape
    out = np.empty((n, shape[2], shape[1], shape[0]), np.float32)
    restate_lib().dro_slice(_p(x), n, wd, h, c, origin[0], origin[1], origin[2], shape[0], shape[1], shape[2], _p(out))
    return out


def croporpad(x, shape):
    x = _c(x)
    n, c, h, wd = x.shape
    out = np.empty((n, shape[2], shape[1], shape[0]), np.float32)
    restate_lib().dro_croporpad(_p(x), n, wd, h, c, shape[0], shape[1], shape[2], _p(out))
    return out


def concat(xs, dim):
    """dim: 0 = x, 1 = y, 2 = z (the reference's axis numbering)."""
    xs = [_c(x) for x in xs]
    axis = {0: 3, 1: 2, 2: 1}[dim]
    shape = list(xs[0].shape)
    shape[axis] = sum(x.shape[axis] for x in xs)
    out = np.zeros(shape, np.float32)
    n, C, H, W = shape
    off = 0
    for x in xs:
        _, c, h, w = x.shape
        restate_lib().dro_concat_place(_p(x), n, w, h, c, dim, off, W, H, C, _p(out))
        off += x.shape[axis]
    return out


# ----------------------------------------------------------------------- reference-kernel leg
def ref_conv2d_winograd(x, w, b, act=1, lms=REF_LMS, mws=REF_MWS):
    x, w, b = _c(x), _c(w), _c(b)
    n, cin, h, wd = x.shape
    cout = w.shape[1]
    out = np.zeros((n, cout, h, wd), np.float32)
    r = ref_lib().drref_conv2d_winograd(_p(x), n, wd, h, cin, _p(w), _p(b), cout, int(act),
                                        ctypes.c_long(lms), ctypes.c_long(mws), _p(out))
    if r < 0:
        raise RuntimeError("reference Winograd schedule does not fit the emulated device")
    return out


def ref_conv2d_1x1(x, w, b, act=1, mws=REF_MWS):
    x, w, b = _c(x), _c(w), _c(b)
    n, cin, h, wd = x.shape
    cout = w.shape[1]
    out = np.zeros((n, cout, h, wd), np.float32)
    ref_lib().drref_conv2d_1x1(_p(x), n, wd, h, cin, _p(w), _p(b), cout, int(act), ctypes.c_long(mws), _p(out))
    return out


def ref_fc(x, w, b, act=1, lms=REF_LMS, mws=REF_MWS):
    x, w, b = _c(x), _c(w), _c(b)
    n, c, h, wd = x.shape
    nout = w.shape[1]
    out = np.zeros((n, 1, 1, nout), np.float32)
    r = ref_lib().drref_fc(_p(x), n, wd, h, c, _p(w), _p(b), nout, int(act), ctypes.c_long(lms), ctypes.c_long(mws), _p(out))
    if r < 0:
        raise RuntimeError("shape hits the reference FC kernels' partition-tail bug; not runnable")
    return out


_REF_POOLS = {(3, 0): 0, (2, 1): 1, (14, 1): 2}


def ref_pool(x, k, stride, kind):
    """Only the three generated pooling kernels the reference ships: 3x3 max, 2x2 avg, 14x14 avg."""
    x = _c(x)
    n, c, h, wd = x.shape
    which = _REF_POOLS[(k, kind)]
    out = np.zeros((n, c, -(-h // stride), -(-wd // stride)), np.float32)
    ref_lib().drref_pool(_p(x), n, wd, h, c, which, stride, stride, _p(out))
    return out


def ref_elemwise1(x, op, scalar=0.0):
    x = _c(x)
    out = np.empty_like(x)
    for i in range(x.shape[0]):
        _, c, h, wd = x.shape
        ref_lib().drref_elemwise1(_p(x[i]), wd, h, c, int(op), ctypes.c_float(scalar), _p(out[i]))
    return out


def ref_elemwise2(a, b, op):
    a, b = _c(a), _c(b)
    out = np.empty_like(a)
    for i in range(a.shape[0]):
        _, c, h, wd = a.shape
        ref_lib().drref_elemwise2(_p(a[i]), _p(b[i]), wd, h, c, int(op), _p(out[i]))
    return out


def ref_softmax(x):
    x = _c(x)
    out = np.empty_like(x)
    for i in range(x.shape[0]):
        _, c, h, wd = x.shape
        ref_lib().drref_softmax(_p(x[i]), wd, h, c, _p(out[i]))
    return out


def ref_slice(x, origin, shape):
    x = _c(x)
    n, c, h, wd = x.shape
    out = np.empty((n, shape[2], shape[1], shape[0]), np.float32)
    for i in range(n):
        ref_lib().drref_slice(_p(x[i]), wd, h, c, origin[0], origin[1], origin[2], shape[0], shape[1], shape[2], _p(out[i]))
    return out


def ref_croporpad(x, shape):
    x = _c(x)
    n, c, h, wd = x.shape
    out = np.empty((n, shape[2], shape[1], shape[0]), np.float32)
    for i in range(n):
        ref_lib().drref_croporpad(_p(x[i]), wd, h, c, shape[0], shape[1], shape[2], _p(out[i]))
    return out
