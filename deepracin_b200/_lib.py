"""ctypes loader for ``libdeepracin.so`` with the argument types of the C API.

The library is the product; this module never falls back to anything else: if the shared
library is missing or cannot be loaded the import of the package fails with the reason.
"""
import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_double, c_float, c_int, c_long, c_size_t, c_void_p)

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libdeepracin.so")


class Shape2(Structure):
    _fields_ = [("s0", c_int), ("s1", c_int)]


class Shape3(Structure):
    _fields_ = [("s0", c_int), ("s1", c_int), ("s2", c_int)]


class Shape4(Structure):
    _fields_ = [("s0", c_int), ("s1", c_int), ("s2", c_int), ("s3", c_int)]


_F = POINTER(c_float)
_SIGS = {
    # public API (include/deepRACIN.h)
    "dR_NewGraph": (c_void_p, []),
    "dR_getOutputBuffers": (c_int, [c_void_p, POINTER(c_void_p)]),
    "dR_feedData": (None, [c_void_p, c_void_p, _F, c_int, c_int]),
    "dR_getFeedNodeInputShape": (POINTER(Shape3), [c_void_p]),
    "dR_setDataFeedNodeBuffer": (c_int, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "dR_setPreexistingOutputBuffer": (c_int, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "dR_setAsOutput": (c_int, [c_void_p, c_void_p]),
    "dR_initCL": (c_int, [c_void_p]),
    "dR_apply": (c_int, [c_void_p]),
    "dR_prepare": (c_int, [c_void_p]),
    "dR_cleanup": (None, [c_void_p, c_int]),
    "dR_saveGraph": (c_int, [c_void_p, c_char_p]),
    "dR_loadGraph": (c_void_p, [c_void_p, c_char_p, POINTER(POINTER(c_void_p)), POINTER(c_int), POINTER(POINTER(c_void_p)), POINTER(c_int)]),
    "dR_printNetObject": (None, [c_void_p, c_char_p]),
    "dR_setClEnvironment": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_long]),
    "dR_getClEnvironmentFrom": (None, [c_void_p, c_void_p]),
    "dR_config": (None, [c_void_p, c_char_p, c_int, c_int, c_int, c_int, c_char_p]),
    "dR_getOutputShape": (POINTER(Shape3), [c_void_p]),
    "dR_downloadArray": (None, [c_void_p, c_char_p, c_void_p, c_size_t, c_size_t, c_void_p]),
    "dR_uploadArray": (c_int, [c_void_p, c_char_p, c_void_p, c_size_t, c_size_t, c_void_p]),
    "dR_createFloatBuffer": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_int]),
    "dR_clMemoryBufferCleanup": (c_int, [c_void_p, c_void_p]),
    # node constructors
    "dR_Datafeednode": (c_void_p, [c_void_p, POINTER(Shape3)]),
    "dR_Conv2d": (c_void_p, [c_void_p, c_void_p, POINTER(Shape4), POINTER(Shape4), c_int, c_int]),
    "dR_Conv2d_setVariables": (None, [c_void_p, _F, _F]),
    "dR_FullyConnected": (c_void_p, [c_void_p, c_void_p, POINTER(Shape2), c_int, c_int]),
    "dR_FullyConnected_setVariables": (None, [c_void_p, _F, _F]),
    "dR_Pooling": (c_void_p, [c_void_p, c_void_p, POINTER(Shape4), POINTER(Shape4), c_int]),
    "dR_Softmax": (c_void_p, [c_void_p, c_void_p]),
    "dR_ElemWise1Operation": (c_void_p, [c_void_p, c_void_p, c_int, c_float]),
    "dR_ElemWise2Operation": (c_void_p, [c_void_p, c_void_p, c_void_p, c_int]),
    "dR_Slice": (c_void_p, [c_void_p, c_void_p, POINTER(Shape4), POINTER(Shape4)]),
    "dR_Concat": (c_void_p, [c_void_p, POINTER(c_void_p), c_int, c_int]),
    "dR_CropOrPad": (c_void_p, [c_void_p, c_void_p, POINTER(Shape3)]),
    "dR_ResolveRoI": (c_void_p, [c_void_p, c_void_p, POINTER(Shape3)]),
    "dR_RGB2gray": (c_void_p, [c_void_p, c_void_p]),
    # additions of the CUDA build (include/dR_b200.h)
    "dR_setBatchSize": (c_int, [c_void_p, c_int]),
    "dR_setMathMode": (c_int, [c_void_p, c_int]),
    "dR_setInterfaceLayout": (c_int, [c_void_p, c_int]),
    "dR_setConvAlgo": (c_int, [c_void_p, c_int]),
    "dR_setGraphConvAlgo": (c_int, [c_void_p, c_int]),
    "dR_setAutotune": (c_int, [c_void_p, c_int]),
    "dR_setFusion": (c_int, [c_void_p, c_int]),
    "dR_setCudaGraph": (c_int, [c_void_p, c_int]),
    "dR_setFeedOverlap": (c_int, [c_void_p, c_int]),
    "dR_setDevice": (c_int, [c_void_p, c_int]),
    "dR_synchronize": (c_int, [c_void_p]),
    "dR_applyTimed": (c_double, [c_void_p, c_int]),
    "dR_getConvAlgo": (c_int, [c_void_p]),
    "dR_getConvTensor": (c_int, [c_void_p]),
    "dR_getConvTensorKernel": (c_int, [c_void_p, POINTER(c_int)]),
    "dR_probeBoundedWait": (c_int, [c_void_p, c_int, POINTER(c_int)]),
    "dR_probeFfmaRate": (c_int, [c_void_p, c_int, POINTER(c_double)]),
    "dR_feedDataU8Async": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "dR_getNodeGpuMs": (c_double, [c_void_p]),
    "dR_getLaunchCount": (c_int, [c_void_p]),
    "dR_getDeviceStatus": (c_int, [c_void_p]),
    "dR_feedDataAsync": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "dR_fetchOutputAsync": (c_int, [c_void_p, c_int, c_void_p, c_size_t]),
    "dR_allocPinned": (c_void_p, [c_size_t]),
    "dR_freePinned": (None, [c_void_p]),
    "dR_timerStart": (None, [c_void_p]),
    "dR_timerStopMs": (c_double, [c_void_p]),
    "dR_setDryRun": (c_int, [c_void_p, c_int]),
    "dR_getScheduleLength": (c_int, [c_void_p]),
    "dR_getScheduledNodeId": (c_int, [c_void_p, c_int]),
    "dR_getNodeActAddress": (c_size_t, [c_void_p]),
    "dR_getNodeActFloats": (c_int, [c_void_p]),
    "dR_getNodeChannelStride": (c_int, [c_void_p]),
    "dR_getNodeChannelOffset": (c_int, [c_void_p]),
    "dR_getStreamBufferCount": (c_int, [c_void_p]),
    "dR_getScratchFloats": (c_size_t, [c_void_p]),
    "dR_b200_version": (c_char_p, []),
    # operator-level kernel ABI (include/dR_kernels.h)
    "dRk_launch_count": (c_long, []),
    "dRk_launch_count_reset": (None, []),
}

_lib = None


def load():
    """Loads the shared library (once) and applies the signatures.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("deepracin_b200: %s is missing -- run `python deepracin_b200/build.py` "
                          "(there is no CPU or Python fallback)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
