"""Helpers for the operator-level GPU tests: device buffers (torch is only the allocator here),
NCHW <-> channels-innermost conversion, and a Python front end to thb_conv_fwd."""
import ctypes as C

import numpy as np
import torch

from thnets_b200 import kernels_abi as K

_TORCH = {K.THB_F32: torch.float32, K.THB_F16: torch.float16, K.THB_BF16: torch.bfloat16, K.THB_U8: torch.uint8}


def ru(v, m):
    return (v + m - 1) // m * m


def dev(arr):
    """numpy -> device tensor (kept alive by the caller)."""
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def dzeros(nbytes_or_shape, dtype=torch.uint8):
    return torch.zeros(nbytes_or_shape, dtype=dtype, device="cuda")


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def to_nhwc(x_nchw, dtype, ld=None, fill=0):
    """[N,C,H,W] numpy -> device [N,H,W,ld] tensor of the kernel dtype (extra channels = fill)."""
    n, c, h, w = x_nchw.shape
    ld = ld or ru(c, K.ALIGN[dtype])
    buf = np.full((n, h, w, ld), fill, dtype=np.float32 if dtype != K.THB_U8 else np.uint8)
    buf[..., :c] = np.transpose(x_nchw, (0, 2, 3, 1))
    t = torch.from_numpy(buf).cuda().to(_TORCH[dtype])
    return t, ld


def from_nhwc(t, c):
    """device [N,H,W,ld] -> numpy [N,C,H,W] float32 (uint8 stays uint8)."""
    a = t[..., :c]
    a = a.float().cpu().numpy() if t.dtype != torch.uint8 else a.cpu().numpy()
    return np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2)))


class Conv:
    """One convolution through the C ABI; keeps every device buffer it references alive."""

    def __init__(self, lib, dtype, x_shape, w_oihw, stride=(1, 1), pad=(0, 0), bn_tile=0, wq=None):
        self.lib, self.dtype = lib, dtype
        n, cin, h, w = x_shape
        cout, _, kh, kw = (w_oihw if wq is None else wq).shape
        d = self.d = K.ConvDesc()
        d.dtype = dtype
        d.N, d.H, d.W, d.Cin = n, h, w, cin
        d.Cout, d.kH, d.kW, d.dH, d.dW, d.padH, d.padW = cout, kh, kw, stride[0], stride[1], pad[0], pad[1]
        d.oH = (h + 2 * pad[0] - kh) // stride[0] + 1
        d.oW = (w + 2 * pad[1] - kw) // stride[1] + 1
        al = K.ALIGN[dtype]
        d.in_ld = ru(cin, al)
        d.out_ld = ru(cout, al)
        d.self_coef, d.res_coef = 1.0, 1.0
        d.relu_thr = -1
        d.BN = bn_tile
        assert lib.thb_conv_geometry(C.byref(d)) == 0
        nbytes = lib.thb_conv_weight_bytes(C.byref(d))
        packed = np.zeros(nbytes, np.uint8)
        kinfo = np.zeros(lib.thb_conv_kinfo_words(C.byref(d)), np.int32)
        wsat = np.zeros(cout * (kh + 1) * (kw + 1), np.int32)
        wf = np.ascontiguousarray(w_oihw, np.float32) if w_oihw is not None else None
        wqc = np.ascontiguousarray(wq, np.uint8) if wq is not None else None
        rc = lib.thb_conv_pack_weights_host(C.byref(d), wf.ctypes.data if wf is not None else None,
                                            wqc.ctypes.data if wqc is not None else None, packed.ctypes.data,
                                            kinfo.ctypes.data, wsat.ctypes.data)
        assert rc == 0, rc
        self.keep = [dev(packed), dev(kinfo), dev(wsat), dzeros(4, torch.int32)]
        d.w, d.kinfo, d.wsat, d.status = (t.data_ptr() for t in self.keep)
        if dtype != K.THB_F32:
            self.tmap, self._tmraw = K.aligned_tmap()
            assert lib.thb_conv_make_tmap(C.byref(d), C.byref(self.tmap)) == 0
            d.tmap = C.addressof(self.tmap)

    @staticmethod
    def _padded(v):
        """per-channel arrays are read in 16-byte groups: pad to a multiple of 64 floats like the planner does"""
        v = np.asarray(v, np.float32)
        out = np.zeros(ru(v.size, 64), np.float32)
        out[:v.size] = v
        return out

    def set_affine(self, scale, shift, host_copies=False):
        """host_copies: also fill thb_conv_desc.scale_host / shift_host (what the planner does)."""
        if scale is not None:
            h = self._padded(scale)
            t = dev(h); self.keep.append(t); self.d.scale = t.data_ptr()
            if host_copies:
                self.keep.append(h); self.d.scale_host = h.ctypes.data
        if shift is not None:
            h = self._padded(shift)
            t = dev(h); self.keep.append(t); self.d.shift = t.data_ptr()
            if host_copies:
                self.keep.append(h); self.d.shift_host = h.ctypes.data

    def set_act(self, kind, threshold=0.0, value=0.0, alpha=0.0, slope=None):
        a = self.d.act
        a.kind, a.threshold, a.value, a.alpha = kind, threshold, value, alpha
        if slope is not None:
            t = dev(self._padded(slope)); self.keep.append(t); a.slope = t.data_ptr()

    def set_residual(self, res_t, res_ld, self_coef, res_coef):
        self.keep.append(res_t)
        self.d.res, self.d.res_ld, self.d.self_coef, self.d.res_coef = res_t.data_ptr(), res_ld, self_coef, res_coef

    def run(self, x_t, out_ld=None, fill=None):
        d = self.d
        if out_ld:
            d.out_ld = out_ld
        y = torch.zeros((d.N, d.oH, d.oW, d.out_ld), dtype=_TORCH[self.dtype], device="cuda")
        if fill is not None:
            y.fill_(fill)
        rc = self.lib.thb_conv_fwd(C.byref(d), ptr(x_t), ptr(y), None)
        torch.cuda.synchronize()
        assert rc == 0, (rc, self.lib.thb_last_cuda_error())
        status = int(self.keep[3].cpu()[0])
        assert status == 0, f"kernel status word = {status} (a bounded wait gave up)"
        return y


    def run_pooled(self, x_t, pk, ppad, ph, pw, fill=None):
        """the convolution and the pk x pk / stride 2 max pooling after it in one launch (thb_conv_maxpool_fwd)"""
        d = self.d
        y = torch.zeros((d.N, ph, pw, d.out_ld), dtype=_TORCH[self.dtype], device="cuda")
        if fill is not None:
            y.fill_(fill)
        self.lib.thb_conv_maxpool_fwd.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                  C.c_void_p, C.c_int, C.c_void_p]
        rc = self.lib.thb_conv_maxpool_fwd(C.byref(d), pk, 2, ppad, ph, pw, ptr(x_t), ptr(y), d.out_ld, None)
        torch.cuda.synchronize()
        assert rc == 0, (rc, self.lib.thb_last_cuda_error())
        status = int(self.keep[3].cpu()[0])
        assert status == 0, f"kernel status word = {status} (a bounded wait gave up)"
        return y


def rel_err(a, ref):
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))
