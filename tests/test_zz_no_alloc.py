"""GPU test of the allocation-free fully connected entry point.

Some users of the library may not allocate device memory once they are running (a control loop with a
frozen memory budget, a plug-in host that owns all device memory), so dRk_fc_f32_noalloc keeps its
split-K scratch in a fixed array inside the library.  This test drives it through the C ABI on
caller-owned buffers, twice in a row (the array keeps the previous call's contents), and requires the
same output as the ordinary entry point dRk_fc_f32 given caller-provided scratch.  It also checks that
a shape beyond the built-in array is refused instead of overrunning it.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

import cases
import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-4  # same bound as the other FP32 parity tests: max|err| <= 1e-4 * max|ref|


def _sig(lib):
    fp = ctypes.c_void_p
    lib.dRk_fc_f32_noalloc.restype = ctypes.c_int
    lib.dRk_fc_f32_noalloc.argtypes = [fp, fp, fp, fp, fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.dRk_fc_f32.restype = ctypes.c_int
    lib.dRk_fc_f32.argtypes = [fp, fp, fp, fp, fp, fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.dRk_fc_scratch_floats.restype = ctypes.c_size_t
    lib.dRk_fc_scratch_floats.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]


@pytest.mark.parametrize("n,c,h,w,nout,act", [(1, 32, 7, 7, 1000, 1), (8, 16, 4, 4, 64, 0), (40, 12, 5, 5, 200, 1)])
def test_no_alloc_fc_matches_regular_entry_point_twice(n, c, h, w, nout, act):
    import torch
    import deepracin_b200 as dr
    lib = dr.lib
    _sig(lib)
    nin = c * h * w
    x, wt, b = cases.fc_case("noalloc%d_%d" % (nin, nout), n, c, h, w, nout, True)
    ref = oracle.fc(x, wt, b, act).reshape(n, nout)
    dev = torch.device("cuda", 0)
    # N-HWC flattening of the activations is the input order of the kernel
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1)).reshape(n, nin)).to(dev)
    wd = torch.from_numpy(wt).to(dev)
    bd = torch.from_numpy(b).to(dev)
    scratch = torch.empty(int(lib.dRk_fc_scratch_floats(n, nin, nout)), dtype=torch.float32, device=dev)
    want = torch.empty(n, nout, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.dRk_fc_f32(stream, xin.data_ptr(), wd.data_ptr(), bd.data_ptr(), want.data_ptr(), scratch.data_ptr(), n, nin, nout, act) == 0
    torch.cuda.synchronize(dev)
    want_h = want.cpu().numpy()
    for call in range(2):
        got = torch.full((n, nout), float("nan"), dtype=torch.float32, device=dev)
        assert lib.dRk_fc_f32_noalloc(stream, xin.data_ptr(), wd.data_ptr(), bd.data_ptr(), got.data_ptr(), n, nin, nout, act) == 0
        torch.cuda.synchronize(dev)
        got_h = got.cpu().numpy()
        scale = max(float(np.max(np.abs(want_h))), 1e-30)
        assert float(np.max(np.abs(got_h - want_h))) <= TOL * scale, call
        assert float(np.max(np.abs(got_h - ref))) <= TOL * max(float(np.max(np.abs(ref))), 1e-30), call
        # a different problem in between leaves other partial sums behind in the shared array
        x2 = torch.randn(3, 640, device=dev)
        w2 = torch.randn(640, 48, device=dev)
        o2 = torch.empty(3, 48, device=dev)
        assert lib.dRk_fc_f32_noalloc(stream, x2.data_ptr(), w2.data_ptr(), None, o2.data_ptr(), 3, 640, 48, 0) == 0
        torch.cuda.synchronize(dev)
        assert torch.allclose(o2, x2 @ w2, rtol=1e-3, atol=1e-3)


def test_no_alloc_fc_refuses_shapes_beyond_its_array(capfd):
    import torch
    import deepracin_b200 as dr
    lib = dr.lib
    _sig(lib)
    n, nin, nout = 64, 25088, 4096
    assert lib.dRk_fc_scratch_floats(n, nin, nout) > (2 << 20)
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # refused before anything is launched, so the small dummy buffers are never touched
    rc = lib.dRk_fc_f32_noalloc(stream, dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), n, nin, nout, 1)
    assert rc == -4
    assert "built-in array holds" in capfd.readouterr().err
