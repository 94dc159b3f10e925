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


def _both_routes(lib, G, conv, xt, with_acc=True):
    d = conv.d
    n_out = d.N * d.oH * d.oW * d.Cout if with_acc else 1
    # ordinary route: caller-owned csum buffer
    csum = G.dzeros(d.N * d.H * d.W, torch.int32)
    acc_a = G.dzeros(n_out, torch.int32)
    d.csum, d.acc_out = csum.data_ptr(), acc_a.data_ptr() if with_acc else None
    assert lib.thb_u8_channel_sum(G.ptr(xt), d.N * d.H * d.W, d.Cin, d.in_ld, G.ptr(csum), None) == 0
    y_a = conv.run(xt)
    # static-scratch route: no csum given at all
    acc_b = G.dzeros(n_out, torch.int32)
    y_b = torch.zeros_like(y_a)
    d.csum, d.acc_out = None, acc_b.data_ptr() if with_acc else None
    rc = lib.thb_conv_u8_fwd_static(C.byref(d), G.ptr(xt), G.ptr(y_b), None)
    torch.cuda.synchronize()
    assert rc == 0, (rc, lib.thb_last_cuda_error())
    assert int(conv.keep[3].cpu()[0]) == 0
    assert torch.equal(acc_a, acc_b), "int32 accumulators differ between the two routes"
    assert torch.equal(y_a, y_b), "outputs differ between the two routes"
    assert not with_acc or int(acc_a.abs().max()) > 0


def test_static_scratch_matches_caller_scratch_twice_in_a_row(lib):
    import gpu_util as G
    # first call: the larger input, so the second call reuses only a prefix of what the first one wrote
    conv1, x1 = _make(lib, G, (3, 40, 29, 31, 72, 3, 1, 1), seed=5)
    _both_routes(lib, G, conv1, x1)
    conv2, x2 = _make(lib, G, (2, 24, 17, 13, 40, 5, 2, 2), seed=6)
    _both_routes(lib, G, conv2, x2)
    # and the first one again, after the scratch held other contents
    _both_routes(lib, G, conv1, x1)


def test_static_scratch_matches_the_oracle(lib, oracle):
    """The static-scratch route against the CPU oracle itself (quantised as the lowp engine does), bit for bit."""
    import gpu_util as G
    case = (2, 24, 17, 13, 40, 3, 1, 1)
    n, cin, h, w, cout, k, s, p = case
    rng = np.random.default_rng(15)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    xq, xs, xm = oracle.lowp_quantize(x)
    wq, ws, wm = oracle.lowp_quantize(wt)
    bq, bs, bm = oracle.lowp_quantize(b)
    osub, omult = float(np.float32(-4.0)), float(np.float32(255) / np.float32(8.0))
    ref = oracle.lowp_conv(xq, xs, xm, wq, ws, wm, bq, bs, bm, (s, s), (p, p), osub, omult)
    conv = G.Conv(lib, K.THB_U8, xq.shape, None, (s, s), (p, p), wq=wq)
    d = conv.d
    d.a_offset, d.b_offset, d.c_offset, d.c_mult, d.c_shift = oracle.lowp_gemm_params(ws, wm, xs, xm, osub, omult)
    add = int(np.round(np.float32(bs) * np.float32(omult)))
    mul = np.float32(omult) / np.float32(bm)
    badd = G.dev(np.array([int(np.round(np.float32(q) * mul)) + add for q in bq], np.int32))
    conv.keep.append(badd)
    d.bias_add = badd.data_ptr()
    ohw = d.oH * d.oW
    d.tail_start = ohw - ohw % 8
    xt, _ = G.to_nhwc(xq, K.THB_U8)
    for _ in range(2):
        y = torch.zeros((n, d.oH, d.oW, d.out_ld), dtype=torch.uint8, device="cuda")
        rc = lib.thb_conv_u8_fwd_static(C.byref(d), G.ptr(xt), G.ptr(y), None)
        torch.cuda.synchronize()
        assert rc == 0, (rc, lib.thb_last_cuda_error())
        assert np.array_equal(G.from_nhwc(y, cout), ref)


@pytest.mark.parametrize("case", [(2, 64, 9, 11, 48, 3, 1, 1),       # Cin a multiple of 16
                                  (3, 2048, 5, 5, 32, 1, 1, 0),      # the one-block-per-pixel channel-sum kernel
                                  (4, 16, 512, 512, 16, 1, 1, 0)])   # N*H*W = the array's capacity exactly
def test_static_scratch_channel_counts_and_capacity(lib, case):
    import gpu_util as G
    conv, xt = _make(lib, G, case, seed=8)
    _both_routes(lib, G, conv, xt, with_acc=case[2] < 512)


def test_static_scratch_refuses_oversized_inputs(lib):
    d = K.ConvDesc()
    d.dtype = K.THB_U8
    d.N, d.H, d.W, d.Cin, d.Cout, d.in_ld = 64, 512, 512, 16, 16, 16          # 16.8M pixels > the array's 1M entries
    d.w = d.kinfo = d.tmap = d.wsat = d.status = 1 << 20                     # (never dereferenced: the call is refused first)
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.thb_conv_u8_fwd_static(C.byref(d), C.c_void_p(dummy.data_ptr()), C.c_void_p(dummy.data_ptr()), None)
    assert rc == -4                                   # THB_ERR_ARG
    assert b"exceeds the static scratch" in lib.thb_last_cuda_error()  # (a complete descriptor otherwise: the size check is what refuses)
    d.dtype = K.THB_F16
    d.N = 1
    assert lib.thb_conv_u8_fwd_static(C.byref(d), C.c_void_p(dummy.data_ptr()), C.c_void_p(dummy.data_ptr()), None) == -4


def test_static_scratch_refuses_rows_stored_with_padding(lib):
    """thb_conv_fwd accepts in_row_pitch for uint8; the static route indexes its sums densely and says so."""
    import gpu_util as G
    conv, xt = _make(lib, G, (2, 16, 9, 9, 32, 3, 1, 1), seed=9)
    d = conv.d
    d.in_row_pitch, d.in_pad_left = 12, 1
    y = torch.zeros((2, 9, 9, 32), dtype=torch.uint8, device="cuda")
    assert lib.thb_conv_u8_fwd_static(C.byref(d), G.ptr(xt), G.ptr(y), None) == -1     # THB_ERR_UNSUPPORTED
    assert b"in_row_pitch" in lib.thb_last_cuda_error()
