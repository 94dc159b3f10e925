"""ctypes mirror of include/thb200_kernels.h (the thin kernel C ABI).

Used by the operator-level tests and by the benchmark to reach single kernels of
`libthnets.so` with raw device pointers.  Nothing here computes anything.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

THB_F32, THB_F16, THB_BF16, THB_U8 = 0, 1, 2, 3
ACT_NONE, ACT_THRESHOLD, ACT_LEAKY, ACT_PRELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3, 4, 5
ESIZE = {THB_F32: 4, THB_F16: 2, THB_BF16: 2, THB_U8: 1}
ALIGN = {THB_F32: 4, THB_F16: 8, THB_BF16: 8, THB_U8: 16}

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_HERE, "libthnets.so")


class Act(C.Structure):
    _fields_ = [("kind", C.c_int), ("threshold", C.c_float), ("value", C.c_float), ("alpha", C.c_float),
                ("slope", C.c_void_p)]


class TMap(C.Structure):
    _fields_ = [("opaque", C.c_ulonglong * 16)]
    _align_ = 64  # honoured by Python >= 3.13; callers allocate through aligned_tmap()


class ConvDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("N", C.c_int), ("H", C.c_int), ("W", C.c_int), ("Cin", C.c_int), ("in_ld", C.c_int),
        ("Cout", C.c_int), ("kH", C.c_int), ("kW", C.c_int), ("dH", C.c_int), ("dW", C.c_int),
        ("padH", C.c_int), ("padW", C.c_int), ("oH", C.c_int), ("oW", C.c_int), ("out_ld", C.c_int),
        ("scale", C.c_void_p), ("shift", C.c_void_p),
        ("res", C.c_void_p), ("res_ld", C.c_int),
        ("self_coef", C.c_float), ("res_coef", C.c_float),
        ("act", Act),
        ("a_offset", C.c_int), ("b_offset", C.c_int), ("c_offset", C.c_int), ("c_mult", C.c_int), ("c_shift", C.c_int),
        ("wsat", C.c_void_p), ("bias_add", C.c_void_p), ("csum", C.c_void_p),
        ("tail_start", C.c_int), ("relu_thr", C.c_int), ("relu_val", C.c_int),
        ("acc_out", C.c_void_p),
        ("w", C.c_void_p), ("kinfo", C.c_void_p), ("tmap", C.c_void_p),
        ("Cin_pad", C.c_int), ("Ktot_pad", C.c_int), ("Cout_pad", C.c_int), ("BN", C.c_int),
        ("status", C.c_void_p),
        ("in_row_pitch", C.c_int), ("in_pad_left", C.c_int),
        ("x2", C.c_void_p), ("x2_ld", C.c_int), ("x2_H", C.c_int), ("x2_W", C.c_int), ("x2_d", C.c_int), ("cin1", C.c_int),
        ("csum_out", C.c_void_p),
        ("scale_host", C.c_void_p), ("shift_host", C.c_void_p),
        ("splits", C.c_int), ("splitk_scratch", C.c_void_p),
    ]


def aligned_tmap():
    """A 64-byte aligned thb_tmap plus the buffer that keeps it alive."""
    raw = (C.c_ubyte * (128 + 64))()
    addr = (C.addressof(raw) + 63) & ~63
    return TMap.from_address(addr), raw


def load(libpath: str | None = None):
    path = libpath or DEFAULT_LIB
    if not os.path.exists(path):
        raise OSError(f"{path} is missing: build it first")
    lib = C.CDLL(path)
    vp, ci, cf, cl = C.c_void_p, C.c_int, C.c_float, C.c_long
    lib.thb_channel_align.argtypes = [ci]
    lib.thb_conv_geometry.argtypes = [C.POINTER(ConvDesc)]
    lib.thb_conv_weight_bytes.argtypes = [C.POINTER(ConvDesc)]
    lib.thb_conv_weight_bytes.restype = C.c_size_t
    lib.thb_conv_kinfo_words.argtypes = [C.POINTER(ConvDesc)]
    lib.thb_conv_kinfo_words.restype = C.c_size_t
    lib.thb_conv_pack_weights_host.argtypes = [C.POINTER(ConvDesc), vp, vp, vp, vp, vp]
    lib.thb_conv_make_tmap.argtypes = [C.POINTER(ConvDesc), C.POINTER(TMap)]
    lib.thb_conv_fwd.argtypes = [C.POINTER(ConvDesc), vp, vp, vp]
    lib.thb_gemv_fwd.argtypes = [ci, vp, ci, ci, ci, vp, ci, vp, vp, C.POINTER(Act), vp, ci, vp]
    lib.thb_preprocess.argtypes = [vp, vp, ci, ci, ci, ci, vp, vp, ci, vp, ci, cf, cf, vp]
    lib.thb_preprocess_images.argtypes = [vp, ci, ci, ci, ci, ci, ci, vp, vp, ci, vp, ci, vp]
    lib.thb_minmax_normalized.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, vp]
    lib.thb_postprocess.argtypes = [vp, ci, ci, ci, ci, ci, ci, cf, cf, vp, vp]
    lib.thb_maxpool.argtypes = [ci, vp] + [ci] * 13 + [vp, ci, vp]
    lib.thb_from_nchw.argtypes = [ci, vp, ci, ci, ci, ci, ci, vp, ci, vp]
    lib.thb_avgpool.argtypes = [ci, vp] + [ci] * 14 + [vp, ci, vp]
    lib.thb_affine_act.argtypes = [ci, vp, cl, ci, ci, vp, vp, C.POINTER(Act), vp, ci, vp]
    lib.thb_u8_threshold.argtypes = [vp, cl, ci, ci, ci, ci, vp, ci, vp]
    lib.thb_u8_combine.argtypes = [vp, ci, vp, ci, ci, ci, ci, ci, cl, ci, vp, ci, vp]
    lib.thb_combine.argtypes = [ci, ci, C.POINTER(vp), C.POINTER(ci), C.POINTER(cf), cl, ci, vp, ci, vp]
    lib.thb_copy_channels.argtypes = [ci, vp, cl, ci, ci, vp, ci, vp]
    lib.thb_softmax.argtypes = [ci, vp, cl, ci, ci, vp, ci, vp]
    lib.thb_col2im.argtypes = [ci, vp] + [ci] * 13 + [cf, vp, C.POINTER(Act), vp, ci, vp]
    lib.thb_u8_channel_sum.argtypes = [vp, cl, ci, ci, vp, vp]
    lib.thb_to_nchw.argtypes = [ci, vp, ci, ci, ci, ci, ci, vp, vp]
    lib.thb_last_cuda_error.restype = C.c_char_p
    lib.thb_kernel_launch_count.restype = ci
    return lib


def np_dtype(dtype):
    return {THB_F32: np.float32, THB_F16: np.float16, THB_U8: np.uint8}[dtype]
