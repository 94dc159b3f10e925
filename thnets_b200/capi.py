"""ctypes binding of the thnets C API (thnets.h:582-598).

Works on any shared library that exports that API: the B200 library built from
`csrc/` (the default), or a CPU build of the reference used as a checker by the
tests.  Mirrors the reference's own `thnets.py` wrapper (thnets.py:7-34) and adds
the conversion entry points.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_HERE, "libthnets.so")

ENGINE_CPU, ENGINE_CUDA, ENGINE_OPENCL, ENGINE_OPENCLINIT, ENGINE_LOWP = range(5)


class THNetworkStruct(C.Structure):
    """Public head of THNETWORK (thnets.h:571-580)."""
    _fields_ = [("netobj", C.c_void_p), ("statobj", C.c_void_p), ("net", C.c_void_p),
                ("pynet", C.c_void_p), ("allpynodes", C.c_void_p), ("out", C.c_void_p),
                ("mean", C.c_float * 3), ("std", C.c_float * 3)]


class THNets:
    def __init__(self, libpath: str | None = None):
        path = libpath or DEFAULT_LIB
        if not os.path.exists(path):
            raise OSError(f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        self.lib = lib = C.CDLL(path, mode=C.RTLD_LOCAL)
        lib.THInit.restype = None
        lib.THLoadNetwork.restype = C.c_void_p
        lib.THLoadNetwork.argtypes = [C.c_char_p]
        lib.THFreeNetwork.argtypes = [C.c_void_p]
        lib.THFreeNetwork.restype = None
        lib.THLastError.restype = C.c_int
        lib.THMakeSpatial.argtypes = [C.c_void_p, C.c_int]
        lib.THMakeSpatial.restype = None
        lib.THProcessFloat.restype = C.c_int
        lib.THProcessFloat.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.POINTER(C.POINTER(C.c_float)), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        lib.THProcessImages.restype = C.c_int
        lib.THProcessImages.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.POINTER(C.POINTER(C.c_float)), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                        C.c_int]
        for name in ("THCreateCudaNetwork", "THCreateOpenCLNetwork"):
            getattr(lib, name).restype = C.c_void_p
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.THCreateLowpNetwork.restype = C.c_void_p
        lib.THCreateLowpNetwork.argtypes = [C.c_void_p, C.c_float]
        lib.THCudaHalfFloat.argtypes = [C.c_int]
        lib.THCudaHalfFloat.restype = C.c_int
        lib.THUseSpatialConvolutionMM.argtypes = [C.c_void_p, C.c_int]
        lib.THUseSpatialConvolutionMM.restype = C.c_int
        self.is_b200 = hasattr(lib, "THB200_SetPrecision")  # False for a CPU build of the reference
        if self.is_b200:
            lib.THB200_LastErrorString.restype = C.c_char_p
            lib.THB200_SetPrecision.argtypes = [C.c_int]
            lib.THB200_SetDevices.argtypes = [C.c_int]
            lib.THB200_LastDeviceMs.restype = C.c_float
            lib.THB200_LastDeviceMs.argtypes = [C.c_void_p]
            lib.THB200_TimeForward.restype = C.c_float
            lib.THB200_TimeForward.argtypes = [C.c_void_p, C.c_int]
            lib.THB200_HostAlloc.restype = C.c_void_p
            lib.THB200_HostAlloc.argtypes = [C.c_size_t]
            lib.THB200_HostFree.argtypes = [C.c_void_p]
            lib.THB200_DescribeNetwork.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        lib.THInit()

    # -- network life cycle ----------------------------------------------------
    def load_network(self, path: str):
        h = self.lib.THLoadNetwork(path.encode())
        if not h:
            raise RuntimeError(f"THLoadNetwork({path}) failed, THLastError() = {self.lib.THLastError()}")
        return h

    def free_network(self, h):
        self.lib.THFreeNetwork(h)

    def set_stats(self, h, mean, std):
        s = THNetworkStruct.from_address(h)
        for i in range(3):
            s.mean[i], s.std[i] = float(mean[i]), float(std[i])

    def make_spatial(self, h, size: int):
        self.lib.THMakeSpatial(h, size)

    def create_cuda_network(self, h, half=0):
        self.lib.THCudaHalfFloat(int(half))
        n = self.lib.THCreateCudaNetwork(h)
        if not n:
            raise RuntimeError("THCreateCudaNetwork returned NULL")
        return n

    def create_lowp_network(self, h, rng: float):
        n = self.lib.THCreateLowpNetwork(h, C.c_float(rng))
        if not n:
            raise RuntimeError("THCreateLowpNetwork returned NULL")
        return n

    # -- forward ---------------------------------------------------------------
    def process_float(self, h, batch: np.ndarray, copy_input=True):
        """batch: float32 [N,C,H,W].  The library normalises its input buffer in place
        (thapi.c:396-403), so by default a private copy is passed."""
        x = np.array(batch, dtype=np.float32, order="C", copy=True) if copy_input else batch
        assert x.dtype == np.float32 and x.flags.c_contiguous and x.ndim == 4
        n, c, hh, ww = x.shape
        res = C.POINTER(C.c_float)()
        ow, oh = C.c_int(), C.c_int()
        cnt = self.lib.THProcessFloat(h, x.ctypes.data_as(C.c_void_p), n, ww, hh, c,
                                      C.byref(res), C.byref(ow), C.byref(oh))
        out = np.ctypeslib.as_array(res, shape=(cnt,)).copy()
        return out, ow.value, oh.value

    def process_yuyv(self, h, frame, width, height):
        """frame: uint8 array of height*width*2 bytes (Y0 U Y1 V per pixel pair)."""
        f = np.ascontiguousarray(frame, np.uint8)
        res = C.POINTER(C.c_float)()
        ow, oh = C.c_int(), C.c_int()
        self.lib.THProcessYUYV.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.POINTER(C.c_float)),
                                           C.POINTER(C.c_int), C.POINTER(C.c_int)]
        self.lib.THProcessYUYV.restype = C.c_int
        cnt = self.lib.THProcessYUYV(h, f.ctypes.data, width, height, C.byref(res), C.byref(ow), C.byref(oh))
        if cnt <= 0:
            return None, 0, 0
        out = np.ctypeslib.as_array(res, shape=(cnt,)).copy()
        return out, ow.value, oh.value

    def process_images(self, h, images, bgr=0):
        """images: list of uint8 [H,W,3] arrays of equal size."""
        n = len(images)
        imgs = [np.ascontiguousarray(i, np.uint8) for i in images]
        hh, ww = imgs[0].shape[:2]
        stride = imgs[0].strides[0]
        ptrs = (C.c_void_p * n)(*[i.ctypes.data for i in imgs])
        res = C.POINTER(C.c_float)()
        ow, oh = C.c_int(), C.c_int()
        cnt = self.lib.THProcessImages(h, ptrs, n, ww, hh, stride, C.byref(res), C.byref(ow), C.byref(oh), bgr)
        out = np.ctypeslib.as_array(res, shape=(cnt,)).copy()
        return out, ow.value, oh.value
