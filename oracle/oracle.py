"""Python driver of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

Walks a `thnets_b200.fixtures.Graph` and evaluates it with the C restatement in
`liboracle.so` (oracle_fp32.c / oracle_lowp.c), the way the reference's executor
would: THProcessFloat normalisation (thapi.c:396-403), then one operator per
node.  `run_lowp` follows the reference's int8 route: THMakeSpatial
(thapi.c:642-690) then THLowp_ToLowp (lowp/lowp_basic.c:133-212), applied per image.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "liboracle.so")
REF_DIR = os.path.join(_HERE, "_ref")

_f = C.POINTER(C.c_float)
_u8 = C.POINTER(C.c_ubyte)


def reference_root():
    """Root of a checkout of the reference: $THNETS_REFERENCE, else a directory `reference` beside the repository."""
    cand = os.environ.get("THNETS_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "thnets.h")) else None


def build(ref_root=None):
    """Compile the C restatement and, when the reference tree is present, the reference itself."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"])
    ref_root = ref_root or reference_root()
    if ref_root and os.path.isdir(ref_root):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "reflowp", f"REF={ref_root}"])


def ref_lib(kind="auto"):
    """Path of a compiled reference library, or None when it was never built."""
    if kind == "auto":
        try:
            flags = open("/proc/cpuinfo").read()
        except OSError:
            flags = ""
        kind = "haswell" if (" avx2" in flags and " fma" in flags) else "penryn"
    p = os.path.join(REF_DIR, f"libthnets_ref_{kind}.so")
    return p if os.path.exists(p) else None


def yuyv_to_float(frame, width, height, mean, std):
    """The reference's YUYV frame -> normalised float RGB planes [3, height, width] (thapi.c:48-117): table-driven integer
    conversion (every quotient truncated towards zero, as C integer division does), saturation to a byte, then
    (byte * 0.003921568f - mean) * (1 / std) in float32.  Test infrastructure only."""
    q = np.asarray(frame, np.uint8).reshape(height, width // 2, 4).astype(np.int64)

    def tdiv(a):  # C division by 256
        return np.where(a >= 0, a // 256, -((-a) // 256))
    y0, u, y1, v = q[..., 0], q[..., 1] - 128, q[..., 2], q[..., 3] - 128
    yur, yub = tdiv(459 * v), tdiv(541 * u)
    yg = tdiv(-137 * u) + tdiv(-55 * v)
    out = np.empty((3, height, width), np.float32)
    mean = np.asarray(mean, np.float32)
    istd = (np.float32(1) / np.asarray(std, np.float32)).astype(np.float32)
    for k, yy in enumerate((y0, y1)):
        ys = tdiv((yy - 16) * 298)
        for c, term in enumerate((yur, yg, yub)):
            byte = np.clip(ys + term, 0, 255).astype(np.float32)
            out[c, :, k::2] = (byte * np.float32(0.003921568) - mean[c]) * istd[c]
    return out


def _fp(a):
    return a.ctypes.data_as(_f)


def _up(a):
    return a.ctypes.data_as(_u8)


class Oracle:
    def __init__(self):
        if not os.path.exists(LIB):
            build()
        self.lib = lib = C.CDLL(LIB)
        lib.orc_conv_out.restype = C.c_int
        lib.orc_pool_out.restype = C.c_int
        lib.orc_exp_minus_approx.restype = C.c_double
        lib.orc_exp_minus_approx.argtypes = [C.c_double]
        lib.orc_lowp_scale_float.restype = C.c_ubyte
        lib.orc_lowp_scale_float.argtypes = [C.c_float, C.c_float, C.c_float]
        lib.orc_lowp_requant.restype = C.c_ubyte
        lib.orc_batchnorm.argtypes = [_f, C.c_int, C.c_int, C.c_int, _f, _f, _f, _f, C.c_double, _f]
        lib.orc_threshold.argtypes = [_f, C.c_long, C.c_float, C.c_float, C.c_float, _f]
        lib.orc_lowp_gemm_params.argtypes = [C.c_float] * 6 + [C.POINTER(C.c_int)] * 5
        lib.orc_lowp_conv.argtypes = [_u8, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                      _u8, C.c_float, C.c_float, _u8, C.c_float, C.c_float] + \
                                     [C.c_int] * 7 + [C.c_float, C.c_float, _u8]
        lib.orc_lowp_dequantize.argtypes = [_u8, C.c_long, C.c_float, C.c_float, _f]
        lib.orc_lowp_quantize.argtypes = [_f, C.c_long, _u8, _f, _f]
        lib.orc_lowp_threshold.argtypes = [_u8, C.c_long, C.c_ubyte, C.c_ubyte, _u8]

    # ---- fp32 operators on NCHW arrays ---------------------------------------
    def conv2d(self, x, w, b, stride, pad):
        n, c, h, ww = x.shape
        co, _, kh, kw = w.shape
        oh = self.lib.orc_conv_out(h, kh, stride[0], pad[0])
        ow = self.lib.orc_conv_out(ww, kw, stride[1], pad[1])
        y = np.empty((n, co, oh, ow), np.float32)
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        self.lib.orc_conv2d(_fp(x), n, c, h, ww, _fp(w), _fp(b) if b is not None else None, co, kh, kw,
                            stride[0], stride[1], pad[0], pad[1], _fp(y))
        return y

    def fullconv2d(self, x, w, b, stride, pad, adj, strict_bias=0):
        n, c, h, ww = x.shape
        _, co, kh, kw = w.shape
        oh = (h - 1) * stride[0] - 2 * pad[0] + kh + adj[0]
        ow = (ww - 1) * stride[1] - 2 * pad[1] + kw + adj[1]
        y = np.empty((n, co, oh, ow), np.float32)
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        self.lib.orc_fullconv2d(_fp(x), n, c, h, ww, _fp(w), _fp(b) if b is not None else None, co, kh, kw,
                                stride[0], stride[1], pad[0], pad[1], adj[0], adj[1], strict_bias, _fp(y))
        return y

    def linear(self, x, w, b):
        n, k = x.shape
        m = w.shape[0]
        y = np.empty((n, m), np.float32)
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        self.lib.orc_linear(_fp(x), n, k, _fp(w), _fp(b) if b is not None else None, m, _fp(y))
        return y

    def batchnorm(self, x, gamma, beta, mean, var, eps):
        n, c = x.shape[:2]
        hw = int(np.prod(x.shape[2:]))
        y = np.empty_like(x)
        x = np.ascontiguousarray(x, np.float32)
        self.lib.orc_batchnorm(_fp(x), n, c, hw, _fp(mean), _fp(var), _fp(gamma) if gamma is not None else None,
                               _fp(beta) if beta is not None else None, eps, _fp(y))
        return y

    def threshold(self, x, th=0.0, val=0.0, alpha=0.0):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.orc_threshold(_fp(x), x.size, th, val, alpha, _fp(y))
        return y

    def prelu(self, x, w, nplanes):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        n, c = x.shape[:2]
        self.lib.orc_prelu(_fp(x), n, c, int(np.prod(x.shape[2:])), _fp(w), nplanes, _fp(y))
        return y

    def maxpool(self, x, k, stride, pad, ceil_mode=0):
        n, c, h, w = x.shape
        oh = self.lib.orc_pool_out(h, k[0], stride[0], pad[0], ceil_mode)
        ow = self.lib.orc_pool_out(w, k[1], stride[1], pad[1], ceil_mode)
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty((n, c, oh, ow), np.float32)
        self.lib.orc_maxpool(_fp(x), n, c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1], ceil_mode, _fp(y))
        return y

    def avgpool(self, x, k, stride, pad, ceil_mode=0, count_include_pad=0):
        n, c, h, w = x.shape
        kh, kw = (k[0] or h), (k[1] or w)
        oh = self.lib.orc_pool_out(h, kh, stride[0], pad[0], ceil_mode)
        ow = self.lib.orc_pool_out(w, kw, stride[1], pad[1], ceil_mode)
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty((n, c, oh, ow), np.float32)
        self.lib.orc_avgpool(_fp(x), n, c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1], ceil_mode,
                             count_include_pad, _fp(y))
        return y

    def softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        if x.ndim == 2:
            self.lib.orc_softmax(_fp(x), x.shape[0], x.shape[1], 1, _fp(y))
        else:
            self.lib.orc_softmax(_fp(x), x.shape[0], x.shape[1], int(np.prod(x.shape[2:])), _fp(y))
        return y

    def caddtable(self, ins, is_csub=0):
        ins = [np.ascontiguousarray(i, np.float32) for i in ins]
        y = np.empty_like(ins[0])
        ptrs = (_f * len(ins))(*[_fp(i) for i in ins])
        ns = (C.c_long * len(ins))(*[i.size for i in ins])
        self.lib.orc_caddtable(ptrs, ns, len(ins), is_csub, _fp(y))
        return y

    def join(self, ins):
        ins = [np.ascontiguousarray(i, np.float32) for i in ins]
        n = ins[0].shape[0]
        hw = int(np.prod(ins[0].shape[2:]))
        cs = (C.c_int * len(ins))(*[i.shape[1] for i in ins])
        y = np.empty((n, sum(i.shape[1] for i in ins)) + ins[0].shape[2:], np.float32)
        ptrs = (_f * len(ins))(*[_fp(i) for i in ins])
        self.lib.orc_join_channels(ptrs, cs, len(ins), n, hw, _fp(y))
        return y

    def normalize(self, x, mean, std):
        x = np.array(x, np.float32, order="C", copy=True)
        n, c, h, w = x.shape
        mean = np.asarray(mean, np.float32)
        std = np.asarray(std, np.float32)
        self.lib.orc_normalize(_fp(x), n, c, h, w, _fp(mean), _fp(std))
        return x

    # ---- the remaining operators (oracle_shape.c) -----------------------------
    def upsample2x(self, x):
        x = np.ascontiguousarray(x, np.float32)
        lead = x.shape[:-2]
        h, w = x.shape[-2:]
        y = np.empty(lead + (2 * h, 2 * w), np.float32)
        self.lib.orc_upsample2x(_fp(x), 1, int(np.prod(lead)), h, w, _fp(y))
        return y

    def zero_pad(self, x, pad_l, pad_r, pad_t, pad_b):
        x = np.ascontiguousarray(x, np.float32)
        lead = x.shape[:-2]
        h, w = x.shape[-2:]
        y = np.empty(lead + (h + pad_t + pad_b, w + pad_l + pad_r), np.float32)
        self.lib.orc_zero_pad(_fp(x), 1, int(np.prod(lead)), h, w, pad_l, pad_r, pad_t, pad_b, _fp(y))
        return y

    def slice(self, x, axis, start, stop):
        x = np.ascontiguousarray(x, np.float32)
        shape = list(x.shape)
        shape[axis] = stop - start
        y = np.empty(shape, np.float32)
        size = (C.c_long * x.ndim)(*x.shape)
        self.lib.orc_slice.argtypes = [_f, C.POINTER(C.c_long), C.c_int, C.c_int, C.c_long, C.c_long, _f]
        self.lib.orc_slice(_fp(x), size, x.ndim, axis, start, stop, _fp(y))
        return y

    def cmax(self, ins):
        ins = [np.ascontiguousarray(i, np.float32) for i in ins]
        y = np.empty_like(ins[0])
        ptrs = (_f * len(ins))(*[_fp(i) for i in ins])
        self.lib.orc_cmax.argtypes = [C.POINTER(_f), C.c_int, C.c_long, _f]
        self.lib.orc_cmax(ptrs, len(ins), ins[0].size, _fp(y))
        return y

    def logsoftmax(self, x, first_frame_quirk=1):
        """LogSoftMax.c over dimension 1 of [N,C] / [N,C,H,W], dimension 0 of [C] / [C,H,W]."""
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        if x.ndim in (1, 3):
            nframe, dim, stride = 1, x.shape[0], int(np.prod(x.shape[1:]))
        else:
            nframe, dim, stride = x.shape[0], x.shape[1], int(np.prod(x.shape[2:]))
        self.lib.orc_logsoftmax.argtypes = [_f, C.c_long, C.c_long, C.c_long, C.c_int, _f]
        self.lib.orc_logsoftmax(_fp(x), nframe, dim, stride, first_frame_quirk, _fp(y))
        return y

    def l2_normalize(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        per_row = 1 if x.ndim == 2 else 0
        rows = x.shape[0] if x.ndim == 2 else 1
        self.lib.orc_l2_normalize.argtypes = [_f, C.c_long, C.c_long, C.c_int, _f]
        self.lib.orc_l2_normalize(_fp(x), rows, x.size // rows, per_row, _fp(y))
        return y

    def max_unpool(self, v, pool_in, k, stride, pad, ceil_mode=0):
        v = np.ascontiguousarray(v, np.float32)
        pool_in = np.ascontiguousarray(pool_in, np.float32)
        n, c, h, w = pool_in.shape
        oh, ow = v.shape[2:]
        y = np.empty_like(pool_in)
        self.lib.orc_max_unpool(_fp(v), _fp(pool_in), n, c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1], oh, ow, _fp(y))
        return y

    # ---- graph execution -------------------------------------------------------
    def conv2d_as_onnx_asks(self, x, w, b, a):
        """What an ONNX convolution with ending pads / dilation / auto_pad / a reflect-mode Pad in front MEANS (the
        reference ignores all four): the input padded explicitly with NumPy, the kernel written out with zeros between
        its taps, then the plain convolution without padding."""
        sh, sw = a["stride"]
        dl = a.get("dilation", (1, 1))
        kh, kw = (w.shape[2] - 1) * dl[0] + 1, (w.shape[3] - 1) * dl[1] + 1
        pt, pl, pb, pr = a.get("pads4", tuple(a["padding"]) * 2)
        if a.get("auto_pad"):
            h, ww = x.shape[2:]
            th = max((-(-h // sh) - 1) * sh + kh - h, 0)
            tw = max((-(-ww // sw) - 1) * sw + kw - ww, 0)
            if a["auto_pad"] == "SAME_UPPER":
                pt, pl = th // 2, tw // 2
            else:
                pt, pl = th - th // 2, tw - tw // 2
            pb, pr = th - pt, tw - pl
        xp = np.pad(x, ((0, 0), (0, 0), (pt, pb), (pl, pr)), mode="reflect" if a.get("reflect") else "constant")
        wd = np.zeros(w.shape[:2] + (kh, kw), np.float32)
        wd[:, :, ::dl[0], ::dl[1]] = w
        return self.conv2d(xp, wd, b, (sh, sw), (0, 0))

    def run(self, graph, batch, keep=False, strict_bias=0, honour_pads=False):
        """fp32 forward of `graph` on a raw [N,C,H,W] batch (normalised here first).  honour_pads: convolutions compute what
        their ONNX-only attributes ask for instead of ignoring them as the reference does."""
        vals = {0: self.normalize(batch, graph.mean, graph.std)}
        for i, node in enumerate(graph.nodes):
            if i == 0:
                continue
            a = node.attrs
            ts = [t for _, t in node.tensors]
            xin = [vals[j] for j in node.inputs]
            x = xin[0]
            if node.op == "conv" and honour_pads and any(k in a for k in ("pads4", "dilation", "auto_pad", "reflect")):
                y = self.conv2d_as_onnx_asks(x, ts[0], ts[1] if len(ts) > 1 else None, a)
            elif node.op == "conv":
                y = self.conv2d(x, ts[0], ts[1] if len(ts) > 1 else None, a["stride"], a["padding"])
            elif node.op == "deconv":
                y = self.fullconv2d(x, ts[0], ts[1] if len(ts) > 1 else None, a["stride"], a["padding"],
                                    a["output_padding"], strict_bias)
            elif node.op == "linear":
                y = self.linear(x.reshape(x.shape[0], -1), ts[0], ts[1])
            elif node.op == "bn":
                y = self.batchnorm(x, ts[0], ts[1], ts[2], ts[3], a["eps"])
            elif node.op == "threshold":
                y = self.threshold(x, a["threshold"], a["value"], a.get("alpha", 0.0))
            elif node.op == "prelu":
                y = self.prelu(x, ts[0], a["planes"])
            elif node.op == "maxpool":
                y = self.maxpool(x, a["kernel_size"], a["stride"], a["padding"], a["ceil_mode"])
            elif node.op == "avgpool":
                y = self.avgpool(x, a["kernel_size"], a["stride"], a["padding"], a["ceil_mode"])
            elif node.op == "view":
                y = x.reshape(-1, a["sizes"][1])
            elif node.op == "reshape":
                # modules/Reshape.c:22-36: every image's elements, in order, as a [c, h, w] map
                y = x.reshape(-1, *a["sizes"])
            elif node.op == "dropout":
                y = x
            elif node.op == "softmax":
                y = self.softmax(x)
            elif node.op == "sigmoid":      # modules/Sigmoid.c:24, float arithmetic
                y = (np.float32(1) / (np.float32(1) + np.exp(-x.astype(np.float32)))).astype(np.float32)
            elif node.op == "tanh":         # modules/Tanh.c
                y = np.tanh(x.astype(np.float32)).astype(np.float32)
            elif node.op == "add":
                y = self.caddtable(xin)
            elif node.op == "concat":
                y = self.join(xin) if a.get("dim", 1) == 1 else np.concatenate(xin, axis=a["dim"])
            elif node.op == "upsample":
                y = self.upsample2x(x)
            elif node.op == "zeropad":
                y = self.zero_pad(x, a["pad_l"], a["pad_r"], a["pad_t"], a["pad_b"])
            elif node.op == "slice":
                y = self.slice(x, a["axis"], a["start"], a["stop"])
            elif node.op == "cmax":
                y = self.cmax(xin)
            elif node.op == "logsoftmax":
                y = self.logsoftmax(x)
            elif node.op == "l2normalize":
                y = self.l2_normalize(x)
            elif node.op == "unpool":
                pool = graph.nodes[a["pool"]]
                pa = pool.attrs
                y = self.max_unpool(x, vals[pool.inputs[0]], pa["kernel_size"], pa["stride"], pa["padding"], pa["ceil_mode"])
            else:
                raise ValueError(node.op)
            vals[i] = y
        return vals if keep else vals[graph.output]

    # ---- lowp ----------------------------------------------------------------
    def lowp_quantize(self, x):
        x = np.ascontiguousarray(x, np.float32)
        q = np.empty(x.shape, np.uint8)
        sub, mult = C.c_float(), C.c_float()
        self.lib.orc_lowp_quantize(_fp(x), x.size, _up(q), C.byref(sub), C.byref(mult))
        return q, sub.value, mult.value

    def lowp_dequantize(self, q, sub, mult):
        q = np.ascontiguousarray(q, np.uint8)
        x = np.empty(q.shape, np.float32)
        self.lib.orc_lowp_dequantize(_up(q), q.size, sub, mult, _fp(x))
        return x

    def lowp_gemm_params(self, w_sub, w_mult, in_sub, in_mult, out_sub, out_mult):
        v = [C.c_int() for _ in range(5)]
        self.lib.orc_lowp_gemm_params(w_sub, w_mult, in_sub, in_mult, out_sub, out_mult, *[C.byref(i) for i in v])
        return tuple(i.value for i in v)  # a_offset, b_offset, c_offset, c_mult, c_shift

    def lowp_conv(self, xq, in_sub, in_mult, wq, w_sub, w_mult, bq, b_sub, b_mult, stride, pad, out_sub, out_mult):
        n, c, h, w = xq.shape
        co, _, kh, kw = wq.shape
        oh = self.lib.orc_conv_out(h, kh, stride[0], pad[0])
        ow = self.lib.orc_conv_out(w, kw, stride[1], pad[1])
        y = np.empty((n, co, oh, ow), np.uint8)
        xq, wq, bq = (np.ascontiguousarray(t, np.uint8) for t in (xq, wq, bq))
        self.lib.orc_lowp_conv(_up(xq), n, c, h, w, in_sub, in_mult, _up(wq), w_sub, w_mult, _up(bq), b_sub, b_mult,
                               co, kh, kw, stride[0], stride[1], pad[0], pad[1], out_sub, out_mult, _up(y))
        return y

    def lowp_conv_acc(self, xq, wq, stride, pad, zero, a_off, b_off):
        """int32 accumulators of ONE image [C,H,W] -> [Cout, oH, oW]."""
        c, h, w = xq.shape
        co, _, kh, kw = wq.shape
        oh = self.lib.orc_conv_out(h, kh, stride[0], pad[0])
        ow = self.lib.orc_conv_out(w, kw, stride[1], pad[1])
        acc = np.empty((co, oh, ow), np.int32)
        xq, wq = np.ascontiguousarray(xq, np.uint8), np.ascontiguousarray(wq, np.uint8)
        self.lib.orc_lowp_conv_acc(_up(xq), c, h, w, _up(wq), co, kh, kw, stride[0], stride[1], pad[0], pad[1],
                                   int(zero), int(a_off), int(b_off), acc.ctypes.data_as(C.POINTER(C.c_int)))
        return acc

    def lowp_maxpool(self, xq, k, stride, pad, ceil_mode=0):
        n, c, h, w = xq.shape
        oh = self.lib.orc_pool_out(h, k[0], stride[0], pad[0], ceil_mode)
        ow = self.lib.orc_pool_out(w, k[1], stride[1], pad[1], ceil_mode)
        xq = np.ascontiguousarray(xq, np.uint8)
        y = np.empty((n, c, oh, ow), np.uint8)
        self.lib.orc_lowp_maxpool(_up(xq), n, c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1], ceil_mode,
                                  _up(y))
        return y

    def lowp_threshold(self, xq, sub, mult, th, val):
        t = self.lib.orc_lowp_scale_float(sub, mult, th)
        v = self.lib.orc_lowp_scale_float(sub, mult, val)
        xq = np.ascontiguousarray(xq, np.uint8)
        y = np.empty_like(xq)
        self.lib.orc_lowp_threshold(_up(xq), xq.size, t, v, _up(y))
        return y

    def lowp_images(self, images, mean, std, bgr=0):
        """lowp_basic.c:60-131: list of uint8 [H,W,3] images -> (planar uint8 [N,3,H,W], sub, mult)."""
        n = len(images)
        imgs = [np.ascontiguousarray(i, np.uint8) for i in images]
        h, w = imgs[0].shape[:2]
        ptrs = (C.POINTER(C.c_ubyte) * n)(*[i.ctypes.data_as(C.POINTER(C.c_ubyte)) for i in imgs])
        dst = np.empty((n, 3, h, w), np.uint8)
        sub, mult = C.c_float(), C.c_float()
        mean = np.ascontiguousarray(mean, np.float32)
        std = np.ascontiguousarray(std, np.float32)
        self.lib.orc_lowp_images(ptrs, n, w, h, imgs[0].strides[0], mean.ctypes.data_as(C.POINTER(C.c_float)),
                                 std.ctypes.data_as(C.POINTER(C.c_float)), bgr, _up(dst), C.byref(sub), C.byref(mult))
        return dst, float(sub.value), float(mult.value)

    def run_lowp(self, graph, batch, rng, spatial_size, keep=False, quantised_input=None):
        """uint8 forward of a conv/linear/relu/maxpool graph.

        The input is quantised over the WHOLE batch tensor (lowp_basic.c:15-35); every
        module output uses sub = -range/2, mult = 255/range (lowp_basic.c:137-148); the
        convolution runs per image.  View nodes vanish and Linear nodes become k x k
        convolutions exactly as THMakeSpatial does.

        Beyond what the reference's lowp engine converts (it refuses batch normalisation, average
        pooling and has no CAddTable, lowp_basic.c:150-208) three rules of this project's own let a
        residual network run; they have no reference counterpart and are pinned by nothing but this
        restatement:
          * conv -> bn: the normalisation is folded into weights and bias BEFORE they are quantised,
            w' = w*scale, b' = b*scale + shift with scale = gamma/sqrt(var+eps) (double, then float),
            shift = beta - mean*scale (the algebra of onnx.cc:537-548);
          * add of two tensors on the static quantisation (CAddTable with two inputs is a - b,
            CAddTable.c:59-69): sat_u8(qa - qb + 127), the byte the dequantise -> subtract ->
            THLowp_ScaleFloat chain gives in exact arithmetic (sub*mult = -127.5, truncation);
          * unpadded average pooling: floor(sum of bytes / window size).
        """
        if quantised_input is not None:      # the image loader's static range instead of the measured one
            q, sub, mult = quantised_input
        else:
            x = self.normalize(batch, graph.mean, graph.std)
            q, sub, mult = self.lowp_quantize(x)
        osub, omult = np.float32(-rng / 2), np.float32(np.float32(255) / np.float32(rng))
        users = {}
        for i, node in enumerate(graph.nodes):
            for j in node.inputs:
                users.setdefault(j, []).append(i)
        vals = {0: (q, sub, mult)}

        def conv_like(node, src, scale=None, shift=None):
            a = node.attrs
            ts = [t for _, t in node.tensors]
            q, sub, mult = src
            w, b = ts[0], (ts[1] if len(ts) > 1 else None)
            if scale is not None:
                w = (w * scale.reshape(-1, *([1] * (w.ndim - 1)))).astype(np.float32)
                b = ((b * scale if b is not None else np.zeros_like(shift)) + shift).astype(np.float32)
            if node.op == "linear":
                cin = q.shape[1]
                k = int(round((w.shape[1] / cin) ** 0.5))
                w = w.reshape(w.shape[0], cin, k, k)
                stride, pad = (1, 1), (0, 0)
            else:
                stride, pad = a["stride"], a["padding"]
            wq, wsub, wmult = self.lowp_quantize(w)
            bq, bsub, bmult = self.lowp_quantize(b)
            y = self.lowp_conv(q, sub, mult, wq, wsub, wmult, bq, bsub, bmult, stride, pad, float(osub), float(omult))
            return (y, float(osub), float(omult))

        cur = vals[0]
        for i, node in enumerate(graph.nodes):
            if i == 0:
                continue
            a = node.attrs
            ts = [t for _, t in node.tensors]
            src = vals[node.inputs[0]]
            if node.op in ("conv", "linear"):
                u = users.get(i, [])
                if len(u) == 1 and graph.nodes[u[0]].op == "bn":
                    cur = None           # computed at the batch-norm node, folded
                else:
                    cur = conv_like(node, src)
            elif node.op == "bn":
                prod = graph.nodes[node.inputs[0]]
                if prod.op != "conv" or vals[node.inputs[0]] is not None:
                    raise ValueError("lowp engine folds a batch-norm only into the convolution before it")
                gamma, beta, mean, var = ts[0], ts[1], ts[2], ts[3]
                invstd = (1.0 / np.sqrt(var.astype(np.float64) + a["eps"])).astype(np.float32)
                scale = (invstd * gamma).astype(np.float32)
                shift = (beta - (mean * scale).astype(np.float32)).astype(np.float32)
                cur = conv_like(prod, vals[prod.inputs[0]], scale, shift)
            elif node.op == "threshold":
                q, sub, mult = src
                cur = (self.lowp_threshold(q, sub, mult, a["threshold"], a["value"]), sub, mult)
            elif node.op == "maxpool":
                q, sub, mult = src
                cur = (self.lowp_maxpool(q, a["kernel_size"], a["stride"], a["padding"], a["ceil_mode"]), sub, mult)
            elif node.op == "avgpool":
                q, sub, mult = src
                (kh, kw), (sh, sw) = a["kernel_size"], a["stride"]
                if tuple(a["padding"]) != (0, 0):
                    raise ValueError("lowp engine has no padded average pooling")
                n, c, h, w_ = q.shape
                oh, ow = (h - kh) // sh + 1, (w_ - kw) // sw + 1
                y = np.empty((n, c, oh, ow), np.uint8)
                for r in range(oh):
                    for t in range(ow):
                        win = q[:, :, r * sh:r * sh + kh, t * sw:t * sw + kw].astype(np.int64)
                        y[:, :, r, t] = win.sum(axis=(2, 3)) // (kh * kw)
                cur = (y, sub, mult)
            elif node.op == "add":
                if len(node.inputs) != 2:
                    raise ValueError("lowp engine adds two tensors")
                (qa, sa, ma), (qb, sb, mb) = vals[node.inputs[0]], vals[node.inputs[1]]
                if (sa, ma) != (sb, mb) or sa != float(osub):
                    raise ValueError("lowp add needs the static output quantisation on both inputs")
                cur = (np.clip(qa.astype(np.int32) - qb.astype(np.int32) + 127, 0, 255).astype(np.uint8), sa, ma)
            elif node.op in ("view", "dropout"):
                cur = src
            else:
                raise ValueError("lowp engine has no " + node.op)
            vals[i] = cur
        out = self.lowp_dequantize(*cur)
        return (out, vals) if keep else out
