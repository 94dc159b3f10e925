"""Parity at benchmark size: the persistent multi-tile walk of the tensor-core convolution.

The operator tests elsewhere give each CTA at most one unit of work.  The cases below are the real ResNet-50 and
VGG-16 layer shapes at batches large enough that every CTA of the 148-SM grid walks several tiles, so that the
ring of TMEM accumulators wraps, the stage ring carries its phase across tiles, the epilogue groups walk many
tiles each, pair mode runs with hundreds of units and odd tile counts, and tiles are walked in both directions
(every second launch of a host thread walks its pixel tiles backwards, so each case is launched twice).
fp16 within 1e-2 of the CPU oracle (max-abs error / max-abs reference); uint8 bit-exact.  Launcher choices are
the defaults the planner would get.

Reference operators: modules/SpatialConvolutionMM.c:126-225, lowp/lowp_SpatialConvolution.c:90-187.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from thnets_b200 import kernels_abi as K  # noqa: E402

SMS = 148


@pytest.fixture(scope="module")
def lib():
    return K.load()


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


# name: (n, cin, h, w, cout, k, stride, pad, residual)
FP16_CASES = {
    # ResNet-50 stage 1 (56 x 56)
    "r50_3x3_64_64_56_b32": (32, 64, 56, 56, 64, 3, 1, 1, False),        # 784 tiles, pair mode: 392 units
    "r50_1x1_256_64_56_b25": (25, 256, 56, 56, 64, 1, 1, 0, False),      # 613 tiles (odd): pair mode with a phantom half
    "r50_1x1_64_256_56_res_b25": (25, 64, 56, 56, 256, 1, 1, 0, True),   # one K block, fused residual + ReLU
    "r50_1x1_64_256_56_b16": (16, 64, 56, 56, 256, 1, 1, 0, False),      # one K block, three epilogue groups
    # stride-2 transitions
    "r50_3x3s2_128_128_56_b48": (48, 128, 56, 56, 128, 3, 2, 1, False),
    "r50_1x1s2_256_512_56_b32": (32, 256, 56, 56, 512, 1, 2, 0, False),
    # deep, narrow maps: 256-channel tiles (two TMEM accumulators), three tiles per CTA
    "wide_3x3_64_256_14_b200": (200, 64, 14, 14, 256, 3, 1, 1, False),
    "r50_3x3_256_256_14_b64": (64, 256, 14, 14, 256, 3, 1, 1, False),
    "r50_1x1_512_2048_7_res_b128": (128, 512, 7, 7, 2048, 1, 1, 0, True),
    "r50_1x1_1024_256_14_b160": (160, 1024, 14, 14, 256, 1, 1, 0, False),
    # VGG-16 first stage
    "vgg_3x3_64_64_224_b2": (2, 64, 224, 224, 64, 3, 1, 1, False),
    # few input channels: the gather path with many tiles per CTA (VGG / segmentation first layer)
    "vgg_3x3_3_64_224_b2": (2, 3, 224, 224, 64, 3, 1, 1, False),
}


def _inputs(case, seed):
    n, cin, h, w, cout, k, s, p, _ = case
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float16).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float16).astype(np.float32)
    return rng, x, wt


def _units(lib, conv):
    d = conv.d
    return ((d.N * d.oH * d.oW + 127) // 128) * (d.Cout_pad // d.BN)


@pytest.mark.parametrize("name", list(FP16_CASES))
def test_conv_f16_many_tiles_per_cta(lib, G, oracle, name):
    case = FP16_CASES[name]
    n, cin, h, w, cout, k, s, p, residual = case
    rng, x, wt = _inputs(case, 101)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = (rng.standard_normal(cout) * 0.2).astype(np.float32)
    ref = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p))
    assert _units(lib, conv) > SMS, "the case must give CTAs more than one tile"
    conv.set_affine(scale, shift)
    conv.set_act(K.ACT_THRESHOLD)
    if residual:
        res = rng.standard_normal(ref.shape).astype(np.float16).astype(np.float32)
        rt, rld = G.to_nhwc(res, K.THB_F16)
        conv.set_residual(rt, rld, 1.0, -1.0)          # CAddTable of two inputs: a - b (CAddTable.c:59-69)
        ref = ref - res
    ref = np.maximum(ref, 0)
    xt, _ = G.to_nhwc(x, K.THB_F16)
    for launch in range(2):                            # forwards, then backwards over the pixel tiles
        got = G.from_nhwc(conv.run(xt, fill=5.0), cout)
        err = G.rel_err(got, ref)
        assert err < 1e-2, (name, launch, err)


@pytest.mark.parametrize("geom", [(16, 64, 256, 56, 56, 1, 256), (32, 128, 256, 28, 28, 2, 512)])
def test_conv_f16_two_operands_many_tiles(lib, G, oracle, geom):
    """The last 1x1 convolution of a bottleneck block and its projection shortcut as one convolution over two tensors
    (thb_conv_desc.x2), at the size the benchmark runs them: stage 1 (stride 1) and stage 2 (shortcut stride 2)."""
    n, c1, c2, oh, ow, d2, cout = geom
    rng = np.random.default_rng(103)
    half = lambda a: a.astype(np.float16).astype(np.float32)
    h2, w2 = (oh - 1) * d2 + 1 + (d2 - 1), (ow - 1) * d2 + 1 + (d2 - 1)
    x1 = half(rng.standard_normal((n, c1, oh, ow)).astype(np.float32))
    x2 = half(rng.standard_normal((n, c2, h2, w2)).astype(np.float32))
    w1 = half((rng.standard_normal((cout, c1, 1, 1)) * 0.1).astype(np.float32))
    w2_ = half((rng.standard_normal((cout, c2, 1, 1)) * 0.1).astype(np.float32))
    shift = rng.standard_normal(cout).astype(np.float32)
    ref = oracle.conv2d(x1, w1, None, (1, 1), (0, 0)) + oracle.conv2d(x2, w2_, None, (d2, d2), (0, 0)) + shift.reshape(1, -1, 1, 1)
    ref = np.maximum(ref, 0)
    conv = G.Conv(lib, K.THB_F16, (n, c1 + c2, oh, ow), np.concatenate([w1, w2_], axis=1))
    assert _units(lib, conv) > 2 * SMS
    conv.set_affine(None, shift)
    conv.set_act(K.ACT_THRESHOLD, 0.0, 0.0)
    d = conv.d
    xt1, ld1 = G.to_nhwc(x1, K.THB_F16)
    xt2, ld2 = G.to_nhwc(x2, K.THB_F16)
    conv.keep.append(xt2)
    d.in_ld, d.cin1 = ld1, c1
    d.x2, d.x2_ld, d.x2_H, d.x2_W, d.x2_d = xt2.data_ptr(), ld2, h2, w2, d2
    for launch in range(2):
        err = G.rel_err(G.from_nhwc(conv.run(xt1, fill=2.0), cout), ref)
        assert err < 1e-2, (geom, launch, err)


def test_conv_f16_stem_rows_stored_with_padding_many_tiles(lib, G, oracle):
    """The ResNet stem after the space-to-depth rewrite (7x7/s2 on 3 channels -> 4x4/s1 on 12, input rows stored with
    their zero padding, one copy per kernel row), batch 8: 784 tiles."""
    case = (8, 12, 112, 112, 64, 4, 1, 2, False)
    n, cin, h, w, cout, k, s, p, _ = case
    rng, x, wt = _inputs(case, 105)
    shift = (rng.standard_normal(cout) * 0.2).astype(np.float32)
    ref = np.maximum(oracle.conv2d(x, wt, shift, (s, s), (p, p))[:, :, :-1, :-1], 0)
    assert lib.thb_conv_padded_rows_supported(K.THB_F16) == 1
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p))
    conv.set_affine(None, shift)
    conv.set_act(K.ACT_THRESHOLD)
    d = conv.d
    d.oH, d.oW = ref.shape[2], ref.shape[3]
    pitch = (p + w + (k - 1 - p) + 3) & ~3
    buf = np.zeros((n, h, pitch, d.in_ld), np.float32)
    buf[:, :, p:p + w, :cin] = np.transpose(x, (0, 2, 3, 1))
    xt = torch.from_numpy(buf).cuda().half()
    d.in_row_pitch, d.in_pad_left = pitch, p
    for launch in range(2):
        err = G.rel_err(G.from_nhwc(conv.run(xt, fill=3.0), cout), ref)
        assert err < 1e-2, (launch, err)


def test_stem_and_max_pooling_in_one_launch_many_tiles(lib, G, oracle):
    """The ResNet stem (after the space-to-depth rewrite) + bias + ReLU + 3x3/s2/p1 max pooling as ONE launch
    (thb_conv_maxpool_fwd) at batch 6: 336 pooled tiles on 148 CTAs, every CTA walks two or three."""
    case = (6, 12, 112, 112, 64, 4, 1, 2, False)
    n, cin, h, w, cout, k, s, p, _ = case
    rng, x, wt = _inputs(case, 109)
    shift = (rng.standard_normal(cout) * 0.2).astype(np.float32)
    y0 = np.maximum(oracle.conv2d(x, wt, shift, (s, s), (p, p))[:, :, :-1, :-1], 0)
    ref = oracle.maxpool(np.ascontiguousarray(y0), (3, 3), (2, 2), (1, 1), 0)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    conv.set_affine(None, shift)
    conv.set_act(K.ACT_THRESHOLD)
    d = conv.d
    d.oH, d.oW = y0.shape[2], y0.shape[3]
    pitch = (p + w + (k - 1 - p) + 3) & ~3
    buf = np.zeros((n, h, pitch, d.in_ld), np.float32)
    buf[:, :, p:p + w, :cin] = np.transpose(x, (0, 2, 3, 1))
    xt = torch.from_numpy(buf).cuda().half()
    d.in_row_pitch, d.in_pad_left = pitch, p
    lib.thb_conv_maxpool_supported.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    if lib.thb_conv_maxpool_supported(C.byref(d), 3, 2, 1) != 1:
        pytest.skip("the driver refuses the overlapping-window descriptor; the planner then keeps the two launches")
    assert ref.shape[2:] == (56, 56)
    for launch in range(2):
        err = G.rel_err(G.from_nhwc(conv.run_pooled(xt, 3, 1, 56, 56, fill=3.0), cout), ref)
        assert err < 1e-2, (launch, err)


# ---------------------------------------------------------------------------------------------------- uint8
U8_CASES = {
    # name: (n, cin, h, w, cout, k, stride, pad, residual)
    "r50_3x3_64_64_56_b16": (16, 64, 56, 56, 64, 3, 1, 1, False),        # 64-byte taps, one column tile: csum_out stored
    "r50_1x1_64_256_56_res_b12": (12, 64, 56, 56, 256, 1, 1, 0, True),   # fused residual, several column tiles: csum_out by atomics
    "r50_1x1_256_64_56_b16": (16, 256, 56, 56, 64, 1, 1, 0, False),
    "r50_3x3s2_128_128_56_b32": (32, 128, 56, 56, 128, 3, 2, 1, False),
    "r50_3x3_256_256_14_b128": (128, 256, 14, 14, 256, 3, 1, 1, False),  # tail rows of a 14 x 14 plane (196 = 8*24 + 4)
    "r50_1x1_512_2048_7_b64": (64, 512, 7, 7, 2048, 1, 1, 0, False),     # 7 x 7 planes: one tail row each
    "vgg_3x3_64_64_224_b1": (1, 64, 224, 224, 64, 3, 1, 1, False),
    "vgg_3x3_3_64_224_b2": (2, 3, 224, 224, 64, 3, 1, 1, False),         # gathered first layer
}


@pytest.mark.parametrize("name", list(U8_CASES))
def test_conv_u8_many_tiles_per_cta_bit_exact(lib, G, oracle, name):
    case = U8_CASES[name]
    n, cin, h, w, cout, k, s, p, residual = case
    rng = np.random.default_rng(107)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    xq, xs, xm = oracle.lowp_quantize(x)
    wq, ws, wm = oracle.lowp_quantize(wt)
    bq, bs, bm = oracle.lowp_quantize(b)
    osub, omult = float(np.float32(-4.0)), float(np.float32(255) / np.float32(8.0))
    ref = oracle.lowp_conv(xq, xs, xm, wq, ws, wm, bq, bs, bm, (s, s), (p, p), osub, omult)
    thr = oracle.lib.orc_lowp_scale_float(osub, omult, 0.0)
    conv = G.Conv(lib, K.THB_U8, xq.shape, None, (s, s), (p, p), wq=wq)
    assert _units(lib, conv) > SMS
    d = conv.d
    d.a_offset, d.b_offset, d.c_offset, d.c_mult, d.c_shift = oracle.lowp_gemm_params(ws, wm, xs, xm, osub, omult)
    add = int(np.round(np.float32(bs) * np.float32(omult)))
    mul = np.float32(omult) / np.float32(bm)
    badd = G.dev(np.array([int(np.round(np.float32(q) * mul)) + add for q in bq], np.int32))
    ohw = d.oH * d.oW
    d.tail_start = ohw - ohw % 8
    d.relu_thr, d.relu_val = thr, thr
    if residual:
        res = rng.integers(0, 256, ref.shape).astype(np.uint8)
        rt, rld = G.to_nhwc(res, K.THB_U8)
        conv.set_residual(rt, rld, 1.0, -1.0)
        ref = np.clip(np.floor(ref.astype(np.float64) - res.astype(np.float64) + 127.5), 0, 255)
    ref = np.where(ref > thr, ref, thr).astype(np.uint8)
    xt, _ = G.to_nhwc(xq, K.THB_U8)
    csum = G.dzeros(n * h * w, torch.int32)
    csum_out = G.dzeros(n * ohw, torch.int32)
    d.bias_add, d.csum, d.csum_out = badd.data_ptr(), csum.data_ptr(), csum_out.data_ptr()
    assert lib.thb_u8_channel_sum(G.ptr(xt), n * h * w, cin, d.in_ld, G.ptr(csum), None) == 0
    for launch in range(2):
        csum_out.zero_()                               # several column tiles add into it with atomics
        got = G.from_nhwc(conv.run(xt), cout)
        assert np.array_equal(got, ref), (name, launch, int(np.abs(got.astype(int) - ref.astype(int)).max()))
        sums = csum_out.cpu().numpy().reshape(n, d.oH, d.oW)
        assert np.array_equal(sums, ref.astype(np.int64).sum(axis=1)), (name, launch, "channel sums of the output")
