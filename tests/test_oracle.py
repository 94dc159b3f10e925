"""The CPU oracle against the reference: golden vectors generated from the unmodified reference CPU
build (tests/golden/make_golden.py), and -- where that build is present on this machine -- the
reference library itself, operator by operator and network by network.  No GPU needed.
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle.oracle import REF_DIR, ref_lib
from thnets_b200 import fixtures as fx

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")


def rel_err(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(ref, np.float64)).max() / max(np.abs(ref).max(), 1e-30))


FP32_CASES = {
    "alexnet_owt": ("alexnet_owt", dict(width=0.25, size=224, classes=50, fc=128), 1),
    "resnet18": ("resnet18", dict(width=0.25, size=64, classes=10), 4),
    "resnet50": ("resnet50", dict(width=0.125, size=64, classes=10), 4),
    "segnet": ("segnet", dict(width=0.5, size=32, classes=21), 4),
    "segnet_bias": ("segnet", dict(width=0.5, size=32, classes=5, deconv_bias=0.1), 4),
    "vgg16": ("vgg16", dict(width=0.125, size=32, classes=10, fc=64), 4),
}


@pytest.mark.parametrize("name", list(FP32_CASES))
def test_fp32_oracle_matches_reference_golden(oracle, name):
    """Pins the fp32 restatement: the reference's two-input CAddTable subtraction, its x11 transposed-
    convolution bias, its polynomial softmax and its pooling shape rules all show up in these outputs.
    The reference differs from itself by a few 1e-6 between build flavours and thread counts."""
    gold = np.load(os.path.join(GOLD, "fp32_networks.npz"))
    builder, kw, batch = FP32_CASES[name]
    g = getattr(fx, builder)(**kw)
    y = oracle.run(g, g.make_input(batch))
    assert y.size == gold[name].size
    assert rel_err(y.ravel(), gold[name]) < 2e-5
    if y.ndim == 4:
        assert tuple(gold[name + "_wh"]) == (y.shape[3], y.shape[2])


@pytest.mark.parametrize("name,kw,rng", [("vgg16_r8", dict(width=0.125, size=32, classes=10, fc=64), 8.0),
                                         ("vgg16_r20", dict(width=0.25, size=64, classes=10, fc=64), 20.0),
                                         ("vgg16_r4", dict(width=0.25, size=32, classes=10, fc=64), 4.0)])
def test_lowp_oracle_matches_reference_golden_bit_exact(oracle, name, kw, rng):
    """The uint8 restatement against the reference's own lowp sources (batch 1, first forward) built around
    the 8-bit GEMM contract: identical dequantised outputs, i.e. identical bytes."""
    gold = np.load(os.path.join(GOLD, "lowp_networks.npz"))
    g = fx.vgg16(**kw)
    y = oracle.run_lowp(g, g.make_input(1), rng, kw["size"])
    assert np.array_equal(y.ravel(), gold[name])


def test_lowp_batch_is_per_image_with_whole_batch_input_scale(oracle):
    """Batch semantics of the uint8 oracle: image i of a batch equals the batch-1 result of the same image
    once the input scale is taken over the whole batch."""
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    x = g.make_input(3)
    full, vals = oracle.run_lowp(g, x, 8.0, 32, keep=True)
    q, sub, mult = vals[0]
    xn = oracle.normalize(x, g.mean, g.std)
    q_all, sub_all, mult_all = oracle.lowp_quantize(xn)
    assert (sub, mult) == (sub_all, mult_all) and np.array_equal(q, q_all)
    assert full.shape[0] == 3


def test_quirks_are_restated(oracle):
    a = np.array([[0.003874]], np.float32)
    b = np.array([[0.526965]], np.float32)
    assert abs(float(oracle.caddtable([a, b])[0, 0]) - (0.003874 - 0.526965)) < 1e-6       # CAddTable.c:59-69
    assert abs(float(oracle.caddtable([a, b], is_csub=1)[0, 0]) - (0.003874 + 0.526965)) < 1e-6
    assert np.allclose(oracle.caddtable([a, b, a]), 3 * a + b)                                # input 0 counted twice
    # exp(-x) polynomial: exact zero from 13 up, a few percent off at x = 8 (thbasic.c:462-491)
    assert oracle.lib.orc_exp_minus_approx(13.0) == 0.0
    assert abs(oracle.lib.orc_exp_minus_approx(8.0) / np.exp(-8.0) - 1) > 1e-2
    assert abs(oracle.lib.orc_exp_minus_approx(2.0) / np.exp(-2.0) - 1) < 1e-4
    # transposed convolution with bias: 11 * deconv + bias
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, 3, 4, 4)).astype(np.float32)
    w = rng.standard_normal((3, 2, 4, 4)).astype(np.float32)
    bias = np.array([100.0, -50.0], np.float32)
    plain = oracle.fullconv2d(x, w, None, (2, 2), (1, 1), (0, 0))
    biased = oracle.fullconv2d(x, w, bias, (2, 2), (1, 1), (0, 0))
    assert rel_err(biased, 11 * plain + bias[None, :, None, None]) < 1e-6
    # lowp: ReLU threshold byte is 127 for any symmetric range, truncating (lowp_basic.c:214-222)
    for r in (4.0, 8.0, 20.0):
        assert oracle.lib.orc_lowp_scale_float(-r / 2, np.float32(255) / np.float32(r), 0.0) == 127
    # the quantiser can produce 256 -> stored as 0 (two terms rounded separately)
    v = np.array([-54.5 / 1.0, 200.5], np.float32)
    q, sub, mult = oracle.lowp_quantize(v)
    assert mult == 1.0 and q[0] == 0 and q[1] == 0


def test_pool_shape_rules(oracle):
    out = oracle.lib.orc_pool_out
    assert out(112, 3, 2, 1, 0) == 56
    assert out(13, 3, 2, 0, 1) == 6 and out(13, 3, 2, 0, 0) == 6
    assert out(14, 3, 2, 0, 1) == 7 and out(14, 3, 2, 0, 0) == 6
    assert out(6, 2, 2, 1, 1) == 4          # ceil mode: the window that would start in the padding is dropped
    assert oracle.lib.orc_conv_out(224, 11, 4, 2) == 55


# ------------------------------------------------------------------------------ live reference (when built)
needs_ref = pytest.mark.skipif(ref_lib() is None, reason="oracle/_ref was not built on this machine")


@needs_ref
@pytest.mark.parametrize("name", ["resnet18", "segnet_bias", "alexnet_owt"])
def test_fp32_oracle_matches_live_reference(oracle, tmp_path, name):
    from thnets_b200.capi import THNets
    ref = THNets(ref_lib())
    builder, kw, batch = FP32_CASES[name]
    g = getattr(fx, builder)(**kw)
    x = g.make_input(batch, seed=99)
    p = str(tmp_path / "m.net")
    fx.write_pymodel(g, p)
    h = ref.load_network(p)
    ref.set_stats(h, g.mean, g.std)
    y, _, _ = ref.process_float(h, x)
    ref.free_network(h)
    assert rel_err(oracle.run(g, x).ravel(), y) < 2e-5


@needs_ref
def test_lowp_oracle_matches_live_reference(oracle, tmp_path):
    from thnets_b200.capi import THNets
    path = os.path.join(REF_DIR, "libthnets_ref_lowp.so")
    if not os.path.exists(path):
        pytest.skip("lowp reference build missing")
    ref = THNets(path)
    g = fx.vgg16(width=0.125, size=48, classes=7, fc=40)
    x = g.make_input(1, seed=5)
    d = str(tmp_path / "vgg")
    fx.write_torch7(g, d)
    h = ref.load_network(d)
    ref.make_spatial(h, 48)
    hl = ref.create_lowp_network(h, 6.0)
    y, _, _ = ref.process_float(hl, x)
    assert np.array_equal(oracle.run_lowp(g, x, 6.0, 48).ravel(), y)


@pytest.mark.parametrize("bgr", [0, 1])
def test_lowp_image_loader_matches_live_reference(oracle, tmp_path, bgr):
    """THProcessImages on the reference's lowp engine (Lowp_LoadImages, lowp/lowp_basic.c:82-131) against the restated
    loader feeding the restated network, batch 1 (the reference's lowp engine is only sound at batch 1)."""
    from thnets_b200.capi import THNets
    path = os.path.join(REF_DIR, "libthnets_ref_lowp.so")
    if not os.path.exists(path):
        pytest.skip("lowp reference build missing")
    ref = THNets(path)
    g = fx.vgg16(width=0.125, size=48, classes=7, fc=40)
    g.mean, g.std = np.array([0.45, 0.42, 0.40], np.float32), np.array([0.225, 0.23, 0.22], np.float32)
    img = np.random.default_rng(8).integers(0, 256, (48, 48, 3)).astype(np.uint8)
    d = str(tmp_path / "vggi")
    fx.write_torch7(g, d)
    h = ref.load_network(d)
    ref.make_spatial(h, 48)
    hl = ref.create_lowp_network(h, 6.0)
    y, _, _ = ref.process_images(hl, [img], bgr=bgr)
    mine = oracle.run_lowp(g, None, 6.0, 48, quantised_input=oracle.lowp_images([img], g.mean, g.std, bgr))
    assert np.array_equal(mine.ravel(), y)


@pytest.mark.parametrize("batch,zeropad", [(1, True), (3, False)])
def test_unpool_zeropad_logsoftmax_against_the_live_reference(oracle, tmp_path, batch, zeropad):
    """The restatements of SpatialZeroPadding, SpatialMaxPooling's indices + SpatialMaxUnpooling and LogSoftMax (with its
    first-frame quirk at batch 3) against the unmodified reference run on the same Torch7 file.  The zero padding is
    compared where the reference's own loop is sound: a square map, no right padding, and ONE image -- its batch loop
    shares the plane and row counters between OpenMP threads (SpatialZeroPadding.c:39-41), so larger batches race."""
    from oracle.oracle import ref_lib
    from thnets_b200 import fixtures as fx
    from thnets_b200.capi import THNets
    if ref_lib() is None:
        pytest.skip("reference library not built")
    g = fx.unpool_net(zeropad=zeropad)
    d = str(tmp_path / "unpool")
    fx.write_torch7(g, d)
    th = THNets(ref_lib())
    h = th.load_network(d)
    x = g.make_input(batch)
    out, _, _ = th.process_float(h, x)
    ref = oracle.run(g, x)
    assert out.size == ref.size
    assert np.abs(out - ref.ravel()).max() / np.abs(ref).max() < 2e-5


@pytest.mark.parametrize("batch", [1, 4])
def test_normalize_against_the_live_reference(oracle, tmp_path, batch):
    from oracle.oracle import ref_lib
    from thnets_b200 import fixtures as fx
    from thnets_b200.capi import THNets
    if ref_lib() is None:
        pytest.skip("reference library not built")
    g = fx.normalize_net()
    d = str(tmp_path / "norm")
    fx.write_torch7(g, d)
    th = THNets(ref_lib())
    h = th.load_network(d)
    x = g.make_input(batch)
    out, _, _ = th.process_float(h, x)
    ref = oracle.run(g, x)
    if batch == 1:
        ref = oracle.l2_normalize(oracle.run(g, x, keep=True)[len(g.nodes) - 2].ravel())   # View gives a 1-D tensor at batch 1
    assert np.abs(out - ref.ravel()).max() / np.abs(ref).max() < 2e-5


@pytest.mark.parametrize("batch", [1, 3])
def test_reshape_against_the_live_reference(oracle, tmp_path, batch):
    """nn.Reshape(c, h, w) after a Linear (modules/Reshape.c:22-36): one image gives a 3-D map (the tensor has exactly
    `nelement` elements and its first dimension is not 1), a batch gives [batch, c, h, w]; the convolution behind it sees
    the vector's elements in (channel, row, column) order either way."""
    from oracle.oracle import ref_lib
    from thnets_b200 import fixtures as fx
    from thnets_b200.capi import THNets
    if ref_lib() is None:
        pytest.skip("reference library not built")
    g = fx.reshape_net()
    d = str(tmp_path / "reshape")
    fx.write_torch7(g, d)
    th = THNets(ref_lib())
    h = th.load_network(d)
    x = g.make_input(batch)
    out, ow, oh = th.process_float(h, x)
    ref = oracle.run(g, x)
    assert (ow, oh) == (4, 5) and out.size == ref.size
    assert np.abs(out - ref.ravel()).max() / np.abs(ref).max() < 2e-5


@pytest.mark.parametrize("batch", [1, 3])
def test_prelu_against_the_live_reference(oracle, tmp_path, batch):
    """nn.PReLU (modules/PReLU.c:32-92) with a slope per plane on a map, with one shared slope, and per feature on the
    2-D (batch) or 1-D (one image) tensor behind a Linear, against the unmodified reference on the same Torch7 file."""
    from oracle.oracle import ref_lib
    from thnets_b200 import fixtures as fx
    from thnets_b200.capi import THNets
    if ref_lib() is None:
        pytest.skip("reference library not built")
    g = fx.prelu_net()
    d = str(tmp_path / "prelu")
    fx.write_torch7(g, d)
    th = THNets(ref_lib())
    h = th.load_network(d)
    x = g.make_input(batch)
    out, _, _ = th.process_float(h, x)
    ref = oracle.run(g, x)
    assert out.size == ref.size == batch * 5
    assert np.abs(out - ref.ravel()).max() / np.abs(ref).max() < 2e-5


def test_leaky_threshold_restatement(oracle):
    """Threshold.c:55-57: with alpha set the module computes x >= 0 ? x : alpha * x and ignores threshold and value"""
    x = np.array([-2.0, -0.0, 0.0, 0.5, 3.0], np.float32)
    assert np.array_equal(oracle.threshold(x, 1.0, 7.0, 0.25), np.array([-0.5, 0.0, 0.0, 0.5, 3.0], np.float32))
    assert np.array_equal(oracle.threshold(x, 1.0, 7.0, 0.0), np.array([7.0, 7.0, 7.0, 7.0, 3.0], np.float32))


def test_cmax_slice_against_the_live_reference(oracle, tmp_path):
    from oracle.oracle import ref_lib
    from thnets_b200 import fixtures as fx
    from thnets_b200.capi import THNets
    if ref_lib() is None:
        pytest.skip("reference library not built")
    g = fx.cmax_slice_net()
    p = str(tmp_path / "cmax.net")
    fx.write_pymodel(g, p)
    th = THNets(ref_lib())
    h = th.load_network(p)
    x = g.make_input(4)
    out, _, _ = th.process_float(h, x)
    ref = oracle.run(g, x)
    assert ref.shape[0] == 2 and out.size == ref.size
    assert np.abs(out - ref.ravel()).max() / np.abs(ref).max() < 2e-5


def test_upsample_restatement():
    """Upsample has an ONNX loader only in the reference, which cannot be built here; the restatement of its loop
    (Upsample.c:55-61) is checked against NumPy's repeat."""
    from oracle.oracle import Oracle
    o = Oracle()
    x = np.random.default_rng(3).standard_normal((2, 3, 4, 5)).astype(np.float32)
    assert np.array_equal(o.upsample2x(x), x.repeat(2, axis=2).repeat(2, axis=3))


@needs_ref
def test_yuyv_conversion_against_the_live_reference(oracle, tmp_path):
    """THProcessYUYV of the reference (thapi.c:575-612) on a Torch7 network = the oracle's forward of the frame converted by
    its restatement of yuyv2fRGB."""
    from oracle.oracle import yuyv_to_float
    from thnets_b200.capi import THNets
    g = fx.alexnet_owt(width=0.25, size=64, classes=10, fc=32)
    d = str(tmp_path / "alex")
    fx.write_torch7(g, d)
    ref = THNets(ref_lib())
    h = ref.load_network(d)
    rng = np.random.default_rng(8)
    frame = rng.integers(0, 256, 64 * 64 * 2).astype(np.uint8)
    out, _, _ = ref.process_yuyv(h, frame, 64, 64)
    ref.free_network(h)
    x = yuyv_to_float(frame, 64, 64, g.mean, g.std)[None]
    plain = fx.Graph()
    plain.nodes, plain.output = g.nodes, g.output   # same weights, identity statistics
    want = oracle.run(plain, x)
    assert rel_err(want.ravel(), out) < 2e-5
