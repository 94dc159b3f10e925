"""thb_conv_u8_fwd_static -- the uint8 convolution whose channel-sum scratch is a fixed array in the library's
device image -- against the ordinary route (thb_u8_channel_sum into a caller buffer + thb_conv_fwd), through the
C ABI, on two calls in a row that use different inputs and different shapes, so that a stale or mis-sized scratch
would show.  Collected last on purpose: it has to pass both alone and after every other GPU test has run."""
import ctypes as C

import numpy as np
import pytest
import torch

from thnets_b200 import kernels_abi as K

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device")
    lib = K.load()
    lib.thb_conv_u8_fwd_static.restype = C.c_int
    lib.thb_conv_u8_fwd_static.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.thb_last_cuda_error.restype = C.c_char_p
    return lib


def _make(lib, G, case, seed):
    n, cin, h, w, cout, k, s, p = case
    rng = np.random.default_rng(seed)
    xq = rng.integers(0, 256, (n, cin, h, w), dtype=np.uint8)
    wq = rng.integers(0, 256, (cout, cin, k, k), dtype=np.uint8)
    conv = G.Conv(lib, K.THB_U8, xq.shape, None, (s, s), (p, p), wq=wq)
    d = conv.d
    d.a_offset, d.b_offset, d.c_offset, d.c_mult, d.c_shift = -131, -119, 2048, 11, 17
    ohw = d.oH * d.oW
    d.tail_start = ohw - ohw % 8
    d.relu_thr, d.relu_val = 40, 40
    badd = G.dev(rng.integers(-20, 20, cout).astype(np.int32))
    conv.keep.append(badd)
    d.bias_add = badd.data_ptr()
    xt, _ = G.to_nhwc(xq, K.THB_U8)
    return conv, xt


def _both_routes(lib, G, conv, xt):
    d = conv.d
    n_out = d.N * d.oH * d.oW * d.Cout
    # ordinary route: caller-owned csum buffer
    csum = G.dzeros(d.N * d.H * d.W, torch.int32)
    acc_a = G.dzeros(n_out, torch.int32)
    d.csum, d.acc_out = csum.data_ptr(), acc_a.data_ptr()
    assert lib.thb_u8_channel_sum(G.ptr(xt), d.N * d.H * d.W, d.Cin, d.in_ld, G.ptr(csum), None) == 0
    y_a = conv.run(xt)
    # static-scratch route: no csum given at all
    acc_b = G.dzeros(n_out, torch.int32)
    y_b = torch.zeros_like(y_a)
    d.csum, d.acc_out = None, acc_b.data_ptr()
    rc = lib.thb_conv_u8_fwd_static(C.byref(d), G.ptr(xt), G.ptr(y_b), None)
    torch.cuda.synchronize()
    assert rc == 0, (rc, lib.thb_last_cuda_error())
    assert int(conv.keep[3].cpu()[0]) == 0
    assert torch.equal(acc_a, acc_b), "int32 accumulators differ between the two routes"
    assert torch.equal(y_a, y_b), "outputs differ between the two routes"
    assert int(acc_a.abs().max()) > 0


def test_static_scratch_matches_caller_scratch_twice_in_a_row(lib):
    import gpu_util as G
    # first call: the larger input, so the second call reuses only a prefix of what the first one wrote
    conv1, x1 = _make(lib, G, (3, 40, 29, 31, 72, 3, 1, 1), seed=5)
    _both_routes(lib, G, conv1, x1)
    conv2, x2 = _make(lib, G, (2, 24, 17, 13, 40, 5, 2, 2), seed=6)
    _both_routes(lib, G, conv2, x2)
    # and the first one again, after the scratch held other contents
    _both_routes(lib, G, conv1, x1)


def test_static_scratch_refuses_oversized_inputs(lib):
    d = K.ConvDesc()
    d.dtype = K.THB_U8
    d.N, d.H, d.W, d.Cin = 64, 512, 512, 16          # 16.8M pixels > the array's 1M entries
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.thb_conv_u8_fwd_static(C.byref(d), C.c_void_p(dummy.data_ptr()), C.c_void_p(dummy.data_ptr()), None)
    assert rc == -4                                   # THB_ERR_ARG
    assert b"exceeds the static scratch" in lib.thb_last_cuda_error()
    d.dtype = K.THB_F16
    d.N = 1
    assert lib.thb_conv_u8_fwd_static(C.byref(d), C.c_void_p(dummy.data_ptr()), C.c_void_p(dummy.data_ptr()), None) == -4
