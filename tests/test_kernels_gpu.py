"""Operator-level parity: every kernel, called through the C ABI of libthnets.so on raw device
pointers, against the CPU oracle on the same seeded inputs.

Tolerances: fp32 1e-4, fp16 1e-2 (max-abs error over max-abs reference, the metric used for whole
networks); uint8 bit-exact, including the int32 accumulators.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from thnets_b200 import kernels_abi as K  # noqa: E402


@pytest.fixture(scope="module")
def lib():
    return K.load()


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


@pytest.fixture
def knobs(lib, monkeypatch):
    """Set THB200_* launcher switches for one test: the library reads them once, so it is told to read them again."""
    def setter(**kw):
        for k, v in kw.items():
            monkeypatch.setenv(k, str(v))
        lib.thb_conv_reload_knobs()
    yield setter
    monkeypatch.undo()
    lib.thb_conv_reload_knobs()


TOL = {K.THB_F32: 1e-4, K.THB_F16: 1e-2}

CONV_CASES = [
    # n, cin, h, w, cout, k, stride, pad
    (2, 16, 12, 12, 32, 3, 1, 1),
    (1, 3, 35, 35, 24, 7, 2, 3),
    (3, 64, 9, 9, 64, 1, 1, 0),
    (2, 24, 17, 13, 40, 3, 2, 1),
    (1, 3, 67, 67, 16, 11, 4, 2),
    (2, 40, 7, 7, 136, 5, 1, 2),
    (5, 128, 7, 7, 72, 3, 1, 1),
    (1, 8, 30, 30, 300, 1, 2, 0),
    # whole 128-byte channel slabs per tap: the activation operand comes in by im2col-mode TMA
    (3, 64, 19, 23, 40, 3, 2, 1),
    (2, 128, 14, 14, 64, 1, 2, 0),
    (2, 64, 30, 17, 96, 5, 1, 2),
    (1, 192, 13, 13, 48, 3, 1, 0),
    (2, 256, 9, 11, 32, 2, 2, 0),
    # stride 1, same padding, whole channel slabs, tiles that span several image rows and images
    (2, 64, 20, 24, 64, 3, 1, 1),
    (3, 128, 21, 22, 128, 3, 1, 1),
    (1, 64, 33, 20, 64, 5, 1, 2),
    # few channels per pixel: several taps per K block, gathered (K padding: 49 taps)
    (2, 32, 15, 15, 64, 3, 1, 1),
    (1, 16, 20, 22, 64, 7, 2, 3),
    (2, 12, 23, 23, 72, 4, 1, 2),
]


def _conv_inputs(case, seed, half):
    n, cin, h, w, cout, k, s, p = case
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    if half:
        x = x.astype(np.float16).astype(np.float32)
        wt = wt.astype(np.float16).astype(np.float32)
    return x, wt


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_plain(lib, G, oracle, dtype, case):
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 1, dtype == K.THB_F16)
    bias = np.random.default_rng(2).standard_normal(cout).astype(np.float32)
    ref = oracle.conv2d(x, wt, bias, (s, s), (p, p))
    conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
    conv.set_affine(None, bias)
    xt, _ = G.to_nhwc(x, dtype)
    y = conv.run(xt, fill=7.0)
    got = G.from_nhwc(y, cout)
    assert G.rel_err(got, ref) < TOL[dtype], (case, G.rel_err(got, ref))
    # padded output channels are written as exact zeros
    pad = y[..., cout:G.ru(cout, K.ALIGN[dtype])]
    assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0


@pytest.mark.parametrize("case", [(1, 192, 13, 13, 384, 3, 1, 1), (1, 64, 27, 27, 192, 5, 1, 2), (2, 40, 9, 7, 72, 3, 2, 1)])
def test_conv_f32_reduction_split_over_a_cluster(lib, G, oracle, case, knobs):
    """fp32 convolution of few pixels (the batch-1 layers of AlexNet): the K steps are shared by the CTAs of a thread-block
    cluster and summed in rank order through distributed shared memory.  Within the fp32 tolerance of the oracle, equal
    from run to run (no atomics), and bias, residual and activation are applied once, by the cluster's first CTA."""
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 5, False)
    rng = np.random.default_rng(6)
    bias = rng.standard_normal(cout).astype(np.float32)
    conv_ref = oracle.conv2d(x, wt, bias, (s, s), (p, p))
    res = rng.standard_normal(conv_ref.shape).astype(np.float32)
    ref = np.maximum(conv_ref - res, 0.0)
    outs = []
    for no_split in (0, 1, 0):
        knobs(THB200_NO_SPLITK=no_split)
        conv = G.Conv(lib, K.THB_F32, x.shape, wt, (s, s), (p, p))
        conv.set_affine(None, bias)
        rt, rld = G.to_nhwc(res, K.THB_F32)
        conv.set_residual(rt, rld, 1.0, -1.0)
        conv.set_act(K.ACT_THRESHOLD)
        xt, _ = G.to_nhwc(x, K.THB_F32)
        outs.append(G.from_nhwc(conv.run(xt, fill=3.0), cout))
        assert G.rel_err(outs[-1], ref) < TOL[K.THB_F32], (case, no_split, G.rel_err(outs[-1], ref))
    assert np.array_equal(outs[0], outs[2])            # the split sum does not depend on timing
    assert G.rel_err(outs[0], outs[1]) < 1e-5          # and differs from the unsplit one by rounding order only


@pytest.mark.parametrize("dtype", [K.THB_F16, K.THB_BF16])
@pytest.mark.parametrize("case", [(1, 512, 7, 7, 512, 3, 1, 1), (4, 256, 14, 14, 256, 3, 1, 1), (2, 1024, 14, 14, 256, 1, 1, 0),
                                  (2, 128, 28, 28, 256, 3, 2, 1), (2, 256, 9, 9, 200, 3, 1, 1), (1, 192, 13, 13, 384, 3, 1, 1)])
def test_conv_tc_reduction_split_over_ctas(lib, G, oracle, case, dtype):
    """Tensor-core convolutions of few tiles (the batch-1 and small-batch layers): thb_conv_splitk_plan proposes how many
    CTAs share each tile's K blocks; they store fp32 partial tiles and a second launch adds them in split order and runs
    the epilogue (scale, shift, residual, PReLU).  Within tolerance of the oracle, equal from run to run, and equal to the
    unsplit launch up to the rounding order of the sums."""
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 81, True)
    rng = np.random.default_rng(82)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    slope = rng.uniform(0.05, 0.3, cout).astype(np.float32)
    conv_ref = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    res = rng.standard_normal(conv_ref.shape).astype(np.float16).astype(np.float32)
    v = conv_ref - res
    ref = np.where(v > 0, v, v * slope[None, :, None, None])
    tol = 1e-2 if dtype == K.THB_F16 else 6e-2
    outs = []
    for split in (True, False, True):
        conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
        conv.set_affine(scale, shift, host_copies=True)
        rt, rld = G.to_nhwc(res, dtype)
        conv.set_residual(rt, rld, 1.0, -1.0)
        conv.set_act(K.ACT_PRELU, slope=slope)
        if split:
            nbytes = C.c_size_t(0)
            lib.thb_conv_splitk_plan.argtypes = [C.c_void_p, C.POINTER(C.c_size_t)]
            S = lib.thb_conv_splitk_plan(C.byref(conv.d), C.byref(nbytes))
            assert S > 1 and nbytes.value > 0, "the case must be one the planner would split"
            scratch = torch.full((nbytes.value // 4,), float("nan"), dtype=torch.float32, device="cuda")
            conv.keep.append(scratch)
            conv.d.splits, conv.d.splitk_scratch = S, scratch.data_ptr()
        xt, _ = G.to_nhwc(x, dtype)
        outs.append(G.from_nhwc(conv.run(xt, fill=3.0), cout))
        assert G.rel_err(outs[-1], ref) < tol, (case, split, G.rel_err(outs[-1], ref))
    assert np.array_equal(outs[0], outs[2])
    assert G.rel_err(outs[0], outs[1]) < (2e-3 if dtype == K.THB_F16 else 2e-2)


@pytest.mark.parametrize("gather_only", [False, True])
@pytest.mark.parametrize("crop", [0, 1])
def test_conv_f16_rows_stored_with_padding(lib, G, oracle, gather_only, crop, knobs):
    """Input rows stored with their horizontal zero padding (thb_conv_desc.in_row_pitch): four taps of 16 channels fill
    one 128-byte K block, so one copy fetches a kernel row.  crop = 1 drops the last output row and column, as the
    space-to-depth rewrite of a stride-2 first layer does.  The gather path must read the same layout."""
    case = (3, 12, 21, 19, 72, 4, 1, 2)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 9, True)
    bias = np.random.default_rng(2).standard_normal(cout).astype(np.float32)
    ref = oracle.conv2d(x, wt, bias, (s, s), (p, p))
    if crop:
        ref = ref[:, :, :-1, :-1]
    assert lib.thb_conv_padded_rows_supported(K.THB_F16) == 1
    if gather_only:
        knobs(THB200_A_TMA=0)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p))
    conv.set_affine(None, bias)
    d = conv.d
    d.oH, d.oW = ref.shape[2], ref.shape[3]
    pitch = p + w + (k - 1 - p) + 2
    ld = d.in_ld
    buf = np.zeros((n, h, pitch, ld), np.float32)
    buf[:, :, p:p + w, :cin] = np.transpose(x, (0, 2, 3, 1))
    xt = torch.from_numpy(buf).cuda().half()
    d.in_row_pitch, d.in_pad_left = pitch, p
    got = G.from_nhwc(conv.run(xt, fill=3.0), cout)
    assert G.rel_err(got, ref) < 1e-2, G.rel_err(got, ref)


@pytest.mark.parametrize("case", [(3, 64, 19, 23, 40, 3, 2, 1), (2, 64, 30, 17, 96, 5, 1, 2), (3, 128, 21, 22, 128, 3, 1, 1),
                                  (3, 64, 9, 9, 64, 1, 1, 0), (5, 128, 7, 7, 72, 3, 1, 1), (2, 128, 14, 14, 64, 1, 2, 0)])
@pytest.mark.parametrize("residual", [False, True])
def test_conv_f16_two_tiles_per_cta(lib, G, oracle, case, residual, knobs):
    """Pair mode (two vertically adjacent pixel tiles per CTA sharing one weight tile per K block), forced on shapes
    small enough for the oracle: odd and even tile counts, ragged last tiles, with and without a fused residual."""
    knobs(THB200_PAIR_MIN_UNITS=1, THB200_PAIR_MIN_KB=1)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 21, True)
    rng = np.random.default_rng(22)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    y0 = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p))
    conv.set_affine(scale, shift)
    if residual:
        res = rng.standard_normal(y0.shape).astype(np.float16).astype(np.float32)
        rt, rld = G.to_nhwc(res, K.THB_F16)
        conv.set_residual(rt, rld, 1.0, -1.0)
        conv.set_act(K.ACT_THRESHOLD)
        ref = np.maximum(y0 - res, 0)
    else:
        ref = y0
    xt, _ = G.to_nhwc(x, K.THB_F16)
    got = G.from_nhwc(conv.run(xt, fill=5.0), cout)
    assert G.rel_err(got, ref) < 1e-2, (case, residual, G.rel_err(got, ref))


@pytest.mark.parametrize("bn_tile", [32, 64, 128, 256])
def test_conv_f16_all_tile_widths(lib, G, oracle, bn_tile):
    case = (2, 72, 14, 14, 264, 3, 1, 1)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 3, True)
    ref = oracle.conv2d(x, wt, None, (s, s), (p, p))
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=bn_tile)
    xt, _ = G.to_nhwc(x, K.THB_F16)
    got = G.from_nhwc(conv.run(xt), cout)
    assert G.rel_err(got, ref) < 1e-2, (bn_tile, G.rel_err(got, ref))


def test_conv_f16_long_k(lib, G, oracle):
    """K = 7*7*512 = 25088 (the VGG FC6-as-convolution shape): 392 pipeline stages."""
    rng = np.random.default_rng(4)
    x = rng.standard_normal((4, 512, 7, 7)).astype(np.float16).astype(np.float32)
    wt = (rng.standard_normal((96, 512, 7, 7)) * 0.01).astype(np.float16).astype(np.float32)
    ref = oracle.conv2d(x, wt, None, (1, 1), (0, 0))
    conv = G.Conv(lib, K.THB_F16, x.shape, wt)
    xt, _ = G.to_nhwc(x, K.THB_F16)
    got = G.from_nhwc(conv.run(xt), 96)
    assert G.rel_err(got, ref) < 1e-2


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
def test_conv_fused_epilogue(lib, G, oracle, dtype):
    """BN scale/shift, residual with the reference's a - b sign, then ReLU; then PReLU and leaky."""
    case = (2, 32, 10, 10, 48, 3, 1, 1)
    n, cin, h, w, cout, k, s, p = case
    half = dtype == K.THB_F16
    x, wt = _conv_inputs(case, 5, half)
    rng = np.random.default_rng(6)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    res = rng.standard_normal((n, cout, h, w)).astype(np.float32)
    if half:
        res = res.astype(np.float16).astype(np.float32)
    base = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    xt, _ = G.to_nhwc(x, dtype)
    rt, rld = G.to_nhwc(res, dtype)
    for self_c, res_c in ((1.0, -1.0), (-1.0, 1.0), (1.0, 1.0)):
        conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
        conv.set_affine(scale, shift)
        conv.set_residual(rt, rld, self_c, res_c)
        conv.set_act(K.ACT_THRESHOLD, 0.0, 0.0)
        ref = oracle.threshold(self_c * base + res_c * res, 0.0, 0.0)
        got = G.from_nhwc(conv.run(xt), cout)
        assert G.rel_err(got, ref) < TOL[dtype]
    slope = rng.uniform(0.1, 0.3, cout).astype(np.float32)
    conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
    conv.set_affine(scale, shift)
    conv.set_act(K.ACT_PRELU, slope=slope)
    assert G.rel_err(G.from_nhwc(conv.run(xt), cout), oracle.prelu(base, slope, cout)) < TOL[dtype]
    conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
    conv.set_affine(scale, shift)
    conv.set_act(K.ACT_LEAKY, alpha=0.1)
    assert G.rel_err(G.from_nhwc(conv.run(xt), cout), oracle.threshold(base, 0, 0, 0.1)) < TOL[dtype]
    conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
    conv.set_affine(scale, shift)
    conv.set_act(K.ACT_THRESHOLD, 0.5, -1.0)
    assert G.rel_err(G.from_nhwc(conv.run(xt), cout), oracle.threshold(base, 0.5, -1.0)) < TOL[dtype]


@pytest.mark.parametrize("case", [(2, 64, 20, 24, 64, 3, 1, 1), (3, 64, 9, 7, 24, 3, 1, 0), (1, 64, 57, 61, 40, 3, 1, 1), (2, 64, 30, 18, 64, 2, 1, 1),
                                  (2, 16, 21, 19, 56, 4, 1, 2), (3, 12, 15, 33, 64, 5, 1, 2), (1, 16, 40, 40, 48, 3, 1, 1),
                                  (2, 64, 5, 300, 64, 3, 1, 1), (2, 16, 300, 6, 64, 3, 1, 1), (4, 64, 4, 4, 64, 3, 1, 1), (4, 64, 2, 2, 64, 3, 1, 1)])
@pytest.mark.parametrize("host_copies", [False, True])
def test_conv_patch_path(lib, G, oracle, case, host_copies):
    """Stride-1 convolutions on 16 or 64 channels per pixel with at most 64 output channels take the patch kernel (one raw
    input patch per unit, every tap reads it in place): maps narrower and wider than a patch row, odd sizes, every
    padding, Cout below 64, several patches per image.  The descriptor must qualify, so a silent fall-back cannot pass."""
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 51, True)
    rng = np.random.default_rng(52)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    ref = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    conv.set_affine(scale, shift, host_copies)   # (constants from the descriptor's host copies, or read back per launch)
    lib.thb_conv_patch_supported.argtypes = [C.c_void_p]
    assert lib.thb_conv_patch_supported(C.byref(conv.d)) == 1, "the case must qualify for the patch kernel"
    xt, _ = G.to_nhwc(x, K.THB_F16)
    y = conv.run(xt, fill=7.0)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < 1e-2, (case, G.rel_err(G.from_nhwc(y, cout), ref))
    pad = y[..., cout:G.ru(cout, 8)]
    assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0


@pytest.mark.parametrize("coefs", [(1.0, -1.0), (-1.0, 1.0), (1.0, 1.0)])
@pytest.mark.parametrize("case", [(2, 64, 20, 24, 64, 3, 1, 1), (3, 16, 9, 7, 24, 3, 1, 1), (1, 64, 57, 61, 40, 3, 1, 1),
                                  (8, 64, 56, 56, 64, 3, 1, 1), (2, 64, 5, 300, 64, 3, 1, 1)])
def test_conv_patch_residual(lib, G, oracle, case, coefs):
    """The patch kernel with a fused residual: y = relu(self * (conv * scale + shift) + res_coef * r), the residual tile
    copied into the output tile one unit ahead.  One tile and many tiles per CTA (8 x 56 x 56: 3 units per CTA), ragged
    edges, every sign combination CAddTable / CSubTable produce."""
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 71, True)
    rng = np.random.default_rng(72)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    conv_ref = oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None]
    res = rng.standard_normal(conv_ref.shape).astype(np.float16).astype(np.float32)
    ref = np.maximum(coefs[0] * conv_ref + coefs[1] * res, 0.0)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    conv.set_affine(scale, shift, host_copies=True)
    rt, rld = G.to_nhwc(res, K.THB_F16)
    conv.set_residual(rt, rld, coefs[0], coefs[1])
    conv.set_act(K.ACT_THRESHOLD)
    lib.thb_conv_patch_supported.argtypes = [C.c_void_p]
    assert lib.thb_conv_patch_supported(C.byref(conv.d)) == 1, "the case must qualify for the patch kernel"
    xt, _ = G.to_nhwc(x, K.THB_F16)
    y = conv.run(xt, fill=7.0)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < 1e-2, (case, G.rel_err(G.from_nhwc(y, cout), ref))
    pad = y[..., cout:G.ru(cout, 8)]
    assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0


def test_conv_patch_constants_are_not_cached_by_address(lib, G, oracle):
    """Two layers of one shape whose buffers sit at the same device addresses, with other scale / shift values in them:
    the second launch must use the second values (the launcher keeps tensor maps per address, never the constants)."""
    case = (2, 64, 12, 12, 64, 3, 1, 1)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 61, True)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    xt, _ = G.to_nhwc(x, K.THB_F16)
    rng = np.random.default_rng(62)
    plain = oracle.conv2d(x, wt, None, (s, s), (p, p))
    sc_t = G.dev(np.zeros(64, np.float32)); sh_t = G.dev(np.zeros(64, np.float32))
    conv.keep += [sc_t, sh_t]
    conv.d.scale, conv.d.shift = sc_t.data_ptr(), sh_t.data_ptr()
    y = torch.zeros((n, conv.d.oH, conv.d.oW, conv.d.out_ld), dtype=torch.float16, device="cuda")
    for _ in range(2):
        scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        shift = rng.standard_normal(cout).astype(np.float32)
        sc_t.copy_(torch.from_numpy(scale)); sh_t.copy_(torch.from_numpy(shift))
        assert lib.thb_conv_fwd(C.byref(conv.d), G.ptr(xt), G.ptr(y), None) == 0
        torch.cuda.synchronize()
        ref = plain * scale[None, :, None, None] + shift[None, :, None, None]
        assert G.rel_err(G.from_nhwc(y, cout), ref) < 1e-2


@pytest.mark.parametrize("pool", [(3, 1, 0), (2, 0, 0), (3, 0, 1), (2, 0, 1)], ids=["3s2p1", "2s2", "3s2ceil", "2s2ceil"])
@pytest.mark.parametrize("case", [(2, 64, 20, 24, 40, 3, 1, 1), (3, 64, 17, 15, 64, 3, 1, 1), (1, 16, 33, 37, 24, 5, 1, 2),
                                  (2, 64, 9, 9, 64, 1, 1, 0), (4, 64, 4, 4, 64, 3, 1, 1)])
def test_conv_maxpool_fused(lib, G, oracle, case, pool):
    """Convolution + bias + ReLU + stride-2 max pooling in one launch (thb_conv_maxpool_fwd) against the oracle's
    convolution, Threshold and SpatialMaxPooling (windows clipped to the image, ceil and floor output sizes): maps that
    are not multiples of the pooled tile, several tiles per image, channels below 64."""
    n, cin, h, w, cout, k, s, p = case
    pk, ppad, ceil_mode = pool
    x, wt = _conv_inputs(case, 41, True)
    rng = np.random.default_rng(42)
    scale = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    shift = rng.standard_normal(cout).astype(np.float32)
    y0 = np.maximum(oracle.conv2d(x, wt, None, (s, s), (p, p)) * scale[None, :, None, None] + shift[None, :, None, None], 0)
    ref = oracle.maxpool(y0, (pk, pk), (2, 2), (ppad, ppad), ceil_mode)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    conv.set_affine(scale, shift)
    conv.set_act(K.ACT_THRESHOLD)
    lib.thb_conv_maxpool_supported.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    assert lib.thb_conv_maxpool_supported(C.byref(conv.d), pk, 2, ppad) == 1
    xt, _ = G.to_nhwc(x, K.THB_F16)
    y = conv.run_pooled(xt, pk, ppad, ref.shape[2], ref.shape[3], fill=9.0)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < 1e-2, (case, pool, G.rel_err(G.from_nhwc(y, cout), ref))
    pad = y[..., cout:G.ru(cout, 8)]
    assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0
    # bit-identical to the two launches it replaces
    two = torch.zeros_like(y)
    assert lib.thb_maxpool(K.THB_F16, G.ptr(conv.run(xt)), n, y0.shape[2], y0.shape[3], cout, conv.d.out_ld, pk, pk, 2, 2, ppad, ppad,
                           ref.shape[2], ref.shape[3], G.ptr(two), conv.d.out_ld, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(y[..., :cout], two[..., :cout])


@pytest.mark.parametrize("prelu", [False, True])
def test_conv_maxpool_fused_rows_stored_with_padding(lib, G, oracle, prelu):
    """The same through the kernel-row-per-copy path of a space-to-depth first layer (input rows stored with their
    zero padding, thb_conv_desc.in_row_pitch), cropped output as the stride-2 rewrite produces, then 3x3/s2/p1 pooling."""
    case = (3, 12, 21, 19, 56, 4, 1, 2)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 43, True)
    rng = np.random.default_rng(44)
    shift = rng.standard_normal(cout).astype(np.float32)
    slope = rng.uniform(0.1, 0.3, cout).astype(np.float32)
    y0 = oracle.conv2d(x, wt, shift, (s, s), (p, p))[:, :, :-1, :-1]
    y0 = oracle.prelu(np.ascontiguousarray(y0), slope, cout) if prelu else np.maximum(y0, 0)
    ref = oracle.maxpool(np.ascontiguousarray(y0), (3, 3), (2, 2), (1, 1), 0)
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p), bn_tile=64)
    conv.set_affine(None, shift)
    if prelu:
        conv.set_act(K.ACT_PRELU, slope=slope)
    else:
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
    y = conv.run_pooled(xt, 3, 1, ref.shape[2], ref.shape[3], fill=4.0)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < 1e-2


def test_bounded_wait_gives_up_and_the_next_launch_is_correct(lib, G, oracle, knobs):
    """Every device-side wait is bounded.  Here one runs out on purpose: a test switch makes the copy producer withhold
    the last K block of each CTA's last tile (nothing else is in flight by then), with the limit shortened to ~10 ms.
    The kernel must come back by itself with a non-zero status word, and the context must stay usable: the same
    convolution launched again without the switch gives the right answer."""
    case = (2, 64, 12, 12, 64, 1, 1, 0)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 61, True)
    ref = oracle.conv2d(x, wt, None, (s, s), (p, p))
    conv = G.Conv(lib, K.THB_F16, x.shape, wt, (s, s), (p, p))
    xt, _ = G.to_nhwc(x, K.THB_F16)
    d = conv.d
    y = torch.zeros((n, d.oH, d.oW, d.out_ld), dtype=torch.float16, device="cuda")
    knobs(THB200_TEST_WITHHOLD=1, THB200_WAIT_LIMIT_CYCLES=20000000)
    assert lib.thb_conv_fwd(C.byref(d), G.ptr(xt), G.ptr(y), None) == 0       # the launch itself succeeds
    torch.cuda.synchronize()                                                   # ... and the kernel returns
    status = int(conv.keep[3].cpu()[0])
    assert status != 0, "the wait should have run out"
    conv.keep[3].zero_()
    knobs(THB200_TEST_WITHHOLD=0, THB200_WAIT_LIMIT_CYCLES=4000000000)
    got = G.from_nhwc(conv.run(xt), cout)
    assert G.rel_err(got, ref) < 1e-2


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
def test_conv_strided_views(lib, G, oracle, dtype):
    """Input read from, and output written into, channel slices of wider buffers."""
    case = (2, 16, 8, 8, 32, 3, 1, 1)
    n, cin, h, w, cout, k, s, p = case
    x, wt = _conv_inputs(case, 7, dtype == K.THB_F16)
    ref = oracle.conv2d(x, wt, None, (s, s), (p, p))
    xt, ld = G.to_nhwc(x, dtype, ld=48, fill=3.0)
    conv = G.Conv(lib, dtype, x.shape, wt, (s, s), (p, p))
    conv.d.in_ld = ld
    y = conv.run(xt, out_ld=64, fill=9.0)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < TOL[dtype]
    assert float((y[..., cout:].float() - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("geom", [(3, 64, 128, 12, 12, 1, 256), (2, 128, 64, 14, 10, 2, 136), (5, 64, 64, 7, 7, 2, 64)])
def test_conv_f16_two_activation_operands(lib, G, oracle, geom):
    """A 1x1 convolution whose input channels come from two tensors (thb_conv_desc.x2): the sum of a 1x1 convolution of x
    and a strided 1x1 convolution of x2 in one accumulator, as a bottleneck block's last convolution and its projection
    shortcut are run.  No reference counterpart as one operator; the oracle adds the two convolutions."""
    n, c1, c2, oh, ow, d2, cout = geom
    rng = np.random.default_rng(71)
    half = lambda a: a.astype(np.float16).astype(np.float32)
    h2, w2 = (oh - 1) * d2 + 1 + (d2 - 1), (ow - 1) * d2 + 1     # trailing rows the stride never reaches are allowed
    x1 = half(rng.standard_normal((n, c1, oh, ow)).astype(np.float32))
    x2 = half(rng.standard_normal((n, c2, h2, w2)).astype(np.float32))
    w1 = half((rng.standard_normal((cout, c1, 1, 1)) * 0.1).astype(np.float32))
    w2_ = half((rng.standard_normal((cout, c2, 1, 1)) * 0.1).astype(np.float32))
    shift = rng.standard_normal(cout).astype(np.float32)
    ref = oracle.conv2d(x1, w1, None, (1, 1), (0, 0)) + oracle.conv2d(x2, w2_, None, (d2, d2), (0, 0)) + shift.reshape(1, -1, 1, 1)
    ref = np.maximum(ref, 0)
    conv = G.Conv(lib, K.THB_F16, (n, c1 + c2, oh, ow), np.concatenate([w1, w2_], axis=1))
    conv.set_affine(None, shift)
    conv.set_act(K.ACT_THRESHOLD, 0.0, 0.0)
    d = conv.d
    xt1, ld1 = G.to_nhwc(x1, K.THB_F16)
    xt2, ld2 = G.to_nhwc(x2, K.THB_F16)
    conv.keep.append(xt2)
    d.in_ld, d.cin1 = ld1, c1
    d.x2, d.x2_ld, d.x2_H, d.x2_W, d.x2_d = xt2.data_ptr(), ld2, h2, w2, d2
    y = conv.run(xt1)
    assert G.rel_err(G.from_nhwc(y, cout), ref) < TOL[K.THB_F16]


# ---------------------------------------------------------------------------------------------- uint8
def _lowp_case(oracle, G, case, seed, rng_range=8.0):
    n, cin, h, w, cout, k, s, p = case
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    xq, xs, xm = oracle.lowp_quantize(x)
    wq, ws, wm = oracle.lowp_quantize(wt)
    bq, bs, bm = oracle.lowp_quantize(b)
    osub, omult = float(np.float32(-rng_range / 2)), float(np.float32(255) / np.float32(rng_range))
    return (xq, xs, xm), (wq, ws, wm), (bq, bs, bm), (osub, omult)


@pytest.mark.parametrize("case", CONV_CASES + [(2, 72, 14, 14, 264, 3, 1, 1)])
@pytest.mark.parametrize("relu", [False, True])
def test_conv_u8_bit_exact(lib, G, oracle, case, relu):
    n, cin, h, w, cout, k, s, p = case
    (xq, xs, xm), (wq, ws, wm), (bq, bs, bm), (osub, omult) = _lowp_case(oracle, G, case, 11)
    ref = oracle.lowp_conv(xq, xs, xm, wq, ws, wm, bq, bs, bm, (s, s), (p, p), osub, omult)
    a_off, b_off, c_off, c_mult, c_shift = oracle.lowp_gemm_params(ws, wm, xs, xm, osub, omult)
    zero = int(np.round(np.float32(-xs) * np.float32(xm)))
    thr = oracle.lib.orc_lowp_scale_float(osub, omult, 0.0)
    if relu:
        ref = oracle.lowp_threshold(ref, osub, omult, 0.0, 0.0)
    conv = G.Conv(lib, K.THB_U8, xq.shape, None, (s, s), (p, p), wq=wq)
    d = conv.d
    d.a_offset, d.b_offset, d.c_offset, d.c_mult, d.c_shift = a_off, b_off, c_off, c_mult, c_shift
    # bias addend exactly as lowp_SpatialConvolution.c:112-119 computes it (float math on the host)
    add = int(np.round(np.float32(bs) * np.float32(omult)))
    mul = np.float32(omult) / np.float32(bm)
    badd = np.array([int(np.round(np.float32(q) * mul)) + add for q in bq], np.int32)
    ohw = d.oH * d.oW
    d.tail_start = ohw - ohw % 8
    d.relu_thr, d.relu_val = (thr, thr) if relu else (-1, 0)
    xt, _ = G.to_nhwc(xq, K.THB_U8)
    csum = G.dzeros(n * h * w, torch.int32)
    acc = G.dzeros(n * ohw * cout, torch.int32)
    tb = G.dev(badd)
    d.bias_add, d.csum, d.acc_out = tb.data_ptr(), csum.data_ptr(), acc.data_ptr()
    assert lib.thb_u8_channel_sum(G.ptr(xt), n * h * w, cin, d.in_ld, G.ptr(csum), None) == 0
    y = conv.run(xt)
    got = G.from_nhwc(y, cout)
    acc_ref = np.stack([oracle.lowp_conv_acc(xq[i], wq, (s, s), (p, p), zero, a_off, b_off) for i in range(n)])
    acc_got = acc.cpu().numpy().reshape(n, d.oH, d.oW, cout).transpose(0, 3, 1, 2)
    assert np.array_equal(acc_got, acc_ref), ("int32 accumulators differ", int(np.abs(acc_got - acc_ref).max()))
    assert np.array_equal(got, ref), ("requantised outputs differ", int(np.abs(got.astype(int) - ref.astype(int)).max()))


@pytest.mark.parametrize("case", [(2, 64, 12, 12, 72, 1, 1, 0), (3, 128, 9, 11, 64, 3, 1, 1), (2, 64, 15, 15, 40, 3, 2, 1)])
@pytest.mark.parametrize("coefs", [(1.0, -1.0), (1.0, 1.0)])
def test_conv_u8_fused_residual(lib, G, oracle, case, coefs):
    """uint8 convolution with the residual add fused into its epilogue (an extension, see thb_u8_combine): the bytes equal
    those of the plain convolution followed by sat(floor(ca*q + cb*r - (ca+cb-1)*127.5)) and the Threshold."""
    n, cin, h, w, cout, k, s, p = case
    (xq, xs, xm), (wq, ws, wm), (bq, bs, bm), (osub, omult) = _lowp_case(oracle, G, case, 13)
    conv_ref = oracle.lowp_conv(xq, xs, xm, wq, ws, wm, bq, bs, bm, (s, s), (p, p), osub, omult)
    rng = np.random.default_rng(14)
    res = rng.integers(0, 256, conv_ref.shape).astype(np.uint8)
    ca, cb = coefs
    ref = np.clip(np.floor(ca * conv_ref.astype(np.float64) + cb * res.astype(np.float64) - (ca + cb - 1) * 127.5), 0, 255)
    thr = oracle.lib.orc_lowp_scale_float(osub, omult, 0.0)
    ref = np.where(ref > thr, ref, thr).astype(np.uint8)
    a_off, b_off, c_off, c_mult, c_shift = oracle.lowp_gemm_params(ws, wm, xs, xm, osub, omult)
    conv = G.Conv(lib, K.THB_U8, xq.shape, None, (s, s), (p, p), wq=wq)
    d = conv.d
    d.a_offset, d.b_offset, d.c_offset, d.c_mult, d.c_shift = a_off, b_off, c_off, c_mult, c_shift
    add = int(np.round(np.float32(bs) * np.float32(omult)))
    mul = np.float32(omult) / np.float32(bm)
    badd = np.array([int(np.round(np.float32(q) * mul)) + add for q in bq], np.int32)
    ohw = d.oH * d.oW
    d.tail_start = ohw - ohw % 8
    d.relu_thr, d.relu_val = thr, thr
    xt, _ = G.to_nhwc(xq, K.THB_U8)
    rt, rld = G.to_nhwc(res, K.THB_U8)
    csum = G.dzeros(n * h * w, torch.int32)
    tb = G.dev(badd)
    d.bias_add, d.csum = tb.data_ptr(), csum.data_ptr()
    conv.set_residual(rt, rld, ca, cb)
    assert lib.thb_u8_channel_sum(G.ptr(xt), n * h * w, cin, d.in_ld, G.ptr(csum), None) == 0
    y = conv.run(xt)
    assert np.array_equal(G.from_nhwc(y, cout), ref)


# ---------------------------------------------------------------------------------------- other kernels
@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
@pytest.mark.parametrize("n", [1, 3, 8])
def test_gemv(lib, G, oracle, dtype, n):
    rng = np.random.default_rng(20)
    kdim, m = 1064, 203
    x = rng.standard_normal((n, kdim)).astype(np.float32)
    w = (rng.standard_normal((m, kdim)) * 0.05).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    if dtype == K.THB_F16:
        x, w = x.astype(np.float16).astype(np.float32), w.astype(np.float16).astype(np.float32)
    ref = oracle.threshold(oracle.linear(x, w, b), 0, 0)
    td = torch.float32 if dtype == K.THB_F32 else torch.float16
    xt, wt_, bt = G.dev(x).to(td), G.dev(w).to(td), G.dev(b)
    yld = G.ru(m, K.ALIGN[dtype])
    y = torch.full((n, yld), 5.0, dtype=td, device="cuda")
    act = K.Act(K.ACT_THRESHOLD, 0.0, 0.0, 0.0, None)
    rc = lib.thb_gemv_fwd(dtype, G.ptr(xt), n, kdim, kdim, G.ptr(wt_), m, None, G.ptr(bt), C.byref(act), G.ptr(y), yld, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert G.rel_err(y[:, :m].float().cpu().numpy(), ref) < TOL[dtype]
    assert float(y[:, m:].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16, K.THB_U8])
@pytest.mark.parametrize("geom", [(3, 2, 0, 0), (3, 2, 1, 0), (2, 2, 0, 0), (3, 2, 0, 1)])
def test_maxpool(lib, G, oracle, dtype, geom):
    k, s, p, ceil_mode = geom
    rng = np.random.default_rng(30)
    n, c, h, w = 2, 20, 13, 11
    if dtype == K.THB_U8:
        x = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
        ref = oracle.lowp_maxpool(x, (k, k), (s, s), (p, p), ceil_mode)
    else:
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
        if dtype == K.THB_F16:
            x = x.astype(np.float16).astype(np.float32)
        ref = oracle.maxpool(x, (k, k), (s, s), (p, p), ceil_mode)
    oh, ow = ref.shape[2:]
    xt, ld = G.to_nhwc(x, dtype)
    y = torch.zeros((n, oh, ow, ld), dtype=xt.dtype, device="cuda")
    rc = lib.thb_maxpool(dtype, G.ptr(xt), n, h, w, c, ld, k, k, s, s, p, p, oh, ow, G.ptr(y), ld, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(G.from_nhwc(y, c), ref)


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
def test_vector_per_image_to_map(lib, G, dtype):
    """Reshape to [c, h, w] (modules/Reshape.c:22-36): row n of the input holds the map in (channel, row, column) order;
    the result is channels-innermost with its padded channels zeroed, whatever was in the buffer."""
    rng = np.random.default_rng(33)
    n, c, h, w, x_ld = 3, 5, 4, 7, 144
    x = rng.standard_normal((n, x_ld)).astype(np.float32)
    td = torch.float32 if dtype == K.THB_F32 else torch.float16
    xt = torch.from_numpy(x).cuda().to(td)
    y_ld = G.ru(c, K.ALIGN[dtype]) + K.ALIGN[dtype]          # one more group of channels than the padding: left untouched
    y = torch.full((n, h, w, y_ld), 7.0, dtype=td, device="cuda")
    rc = lib.thb_from_nchw(dtype, G.ptr(xt), n, h, w, c, x_ld, G.ptr(y), y_ld, None)
    torch.cuda.synchronize()
    assert rc == 0
    got = y.float().cpu().numpy()
    ref = xt.float().cpu().numpy()[:, :c * h * w].reshape(n, c, h, w).transpose(0, 2, 3, 1)
    pad = G.ru(c, K.ALIGN[dtype])
    assert np.array_equal(got[..., :c], ref)
    assert np.all(got[..., c:pad] == 0) and np.all(got[..., pad:] == 7.0)
    assert lib.thb_from_nchw(dtype, G.ptr(xt), n, h, w, c, c * h * w - 1, G.ptr(y), y_ld, None) != 0   # rows shorter than a map


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
@pytest.mark.parametrize("geom", [(7, 7, 0), (3, 2, 1), (2, 2, 0)])
def test_avgpool(lib, G, oracle, dtype, geom):
    k, s, p = geom
    rng = np.random.default_rng(31)
    n, c, h, w = 3, 24, 7, 7
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    if dtype == K.THB_F16:
        x = x.astype(np.float16).astype(np.float32)
    ref = oracle.avgpool(x, (k, k), (s, s), (p, p))
    oh, ow = ref.shape[2:]
    xt, ld = G.to_nhwc(x, dtype)
    y = torch.zeros((n, oh, ow, ld), dtype=xt.dtype, device="cuda")
    rc = lib.thb_avgpool(dtype, G.ptr(xt), n, h, w, c, ld, k, k, s, s, p, p, oh, ow, 0, G.ptr(y), ld, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert G.rel_err(G.from_nhwc(y, c), ref) < (1e-6 if dtype == K.THB_F32 else 2e-3)


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
def test_affine_act_combine_copy(lib, G, oracle, dtype):
    rng = np.random.default_rng(32)
    n, c, h, w = 2, 20, 5, 6
    half = dtype == K.THB_F16
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if half else (lambda a: a)
    x = rnd(rng.standard_normal((n, c, h, w)).astype(np.float32))
    x2 = rnd(rng.standard_normal((n, c, h, w)).astype(np.float32))
    gamma, beta = rng.uniform(0.8, 1.2, c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
    mean, var = rng.standard_normal(c).astype(np.float32), rng.uniform(0.5, 1.5, c).astype(np.float32)
    ref = oracle.threshold(oracle.batchnorm(x, gamma, beta, mean, var, 1e-5), 0, 0)
    invstd = (1.0 / np.sqrt(var.astype(np.float64) + 1e-5)).astype(np.float32)
    scale = invstd * gamma
    shift = beta - mean * scale
    xt, ld = G.to_nhwc(x, dtype)
    x2t, _ = G.to_nhwc(x2, dtype)
    y = torch.zeros_like(xt)
    st, sh = G.dev(scale), G.dev(shift)
    act = K.Act(K.ACT_THRESHOLD, 0.0, 0.0, 0.0, None)
    assert lib.thb_affine_act(dtype, G.ptr(xt), n * h * w, c, ld, G.ptr(st), G.ptr(sh), C.byref(act), G.ptr(y), ld, None) == 0
    torch.cuda.synchronize()
    assert G.rel_err(G.from_nhwc(y, c), ref) < (2e-6 if not half else 2e-3)
    # two-input CAddTable = a - b, three-input = 2a + b + c
    for ins, coefs, refv in (((xt, x2t), (1.0, -1.0), oracle.caddtable([x, x2])),
                             ((xt, xt, x2t, xt), (1.0, 1.0, 1.0, 1.0), oracle.caddtable([x, x2, x]))):
        ptrs = (C.c_void_p * len(ins))(*[t.data_ptr() for t in ins])
        lds = (C.c_int * len(ins))(*[ld] * len(ins))
        cf = (C.c_float * len(ins))(*coefs)
        assert lib.thb_combine(dtype, len(ins), ptrs, lds, cf, n * h * w, c, G.ptr(y), ld, None) == 0
        torch.cuda.synchronize()
        assert G.rel_err(G.from_nhwc(y, c), refv) < (1e-6 if not half else 2e-3)
    # channel-slice copy = JoinTable along channels
    al = K.ALIGN[dtype]
    c1 = 2 * al
    a = rnd(rng.standard_normal((n, c1, h, w)).astype(np.float32))
    at, ald = G.to_nhwc(a, dtype)
    wide = torch.zeros((n, h, w, c1 + ld), dtype=xt.dtype, device="cuda")
    assert lib.thb_copy_channels(dtype, G.ptr(at), n * h * w, c1, ald, G.ptr(wide), c1 + ld, None) == 0
    off = C.c_void_p(wide.data_ptr() + c1 * K.ESIZE[dtype])
    assert lib.thb_copy_channels(dtype, G.ptr(xt), n * h * w, c, ld, off, c1 + ld, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(G.from_nhwc(wide, c1 + c), oracle.join([a, x]))


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
def test_softmax(lib, G, oracle, dtype):
    rng = np.random.default_rng(33)
    x = (rng.standard_normal((5, 1000)) * 4).astype(np.float32)
    if dtype == K.THB_F16:
        x = x.astype(np.float16).astype(np.float32)
    ref = oracle.softmax(x)
    td = torch.float32 if dtype == K.THB_F32 else torch.float16
    xt = G.dev(x).to(td)
    y = torch.zeros_like(xt)
    assert lib.thb_softmax(dtype, G.ptr(xt), 5, 1000, 1000, G.ptr(y), 1000, None) == 0
    torch.cuda.synchronize()
    assert G.rel_err(y.float().cpu().numpy(), ref) < (1e-5 if dtype == K.THB_F32 else 2e-3)


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16])
@pytest.mark.parametrize("with_bias", [False, True])
def test_fullconv_gemm_col2im(lib, G, oracle, dtype, with_bias):
    """SpatialFullConvolution = 1x1 convolution to the column matrix, then the col2im gather;
    with a bias the reference result is 11*deconv + bias."""
    rng = np.random.default_rng(34)
    n, cin, h, w, cout, k, s, p = 2, 24, 6, 5, 12, 4, 2, 1
    half = dtype == K.THB_F16
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if half else (lambda a: a)
    x = rnd(rng.standard_normal((n, cin, h, w)).astype(np.float32))
    wt = rnd((rng.standard_normal((cin, cout, k, k)) * 0.1).astype(np.float32))
    bias = rng.standard_normal(cout).astype(np.float32) if with_bias else None
    ref = oracle.fullconv2d(x, wt, bias, (s, s), (p, p), (0, 0))
    al = K.ALIGN[dtype]
    cp = G.ru(cout, al)
    # column index (kh*kW + kw)*cp + co  <-  W[ci][co][kh][kw]
    w1 = np.zeros((k * k * cp, cin, 1, 1), np.float32)
    for kh in range(k):
        for kw in range(k):
            w1[(kh * k + kw) * cp:(kh * k + kw) * cp + cout, :, 0, 0] = wt[:, :, kh, kw].T
    conv = G.Conv(lib, dtype, x.shape, w1)
    xt, _ = G.to_nhwc(x, dtype)
    cols = conv.run(xt)
    oh, ow = ref.shape[2:]
    y = torch.zeros((n, oh, ow, cp), dtype=xt.dtype, device="cuda")
    bt = G.dev(bias) if with_bias else None
    rc = lib.thb_col2im(dtype, G.ptr(cols), n, h, w, cout, k, k, s, s, p, p, oh, ow, conv.d.out_ld, 11.0, G.ptr(bt), None,
                        G.ptr(y), cp, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert G.rel_err(G.from_nhwc(y, cout), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [K.THB_F32, K.THB_F16, K.THB_U8])
def test_pre_and_postprocess(lib, G, oracle, dtype):
    rng = np.random.default_rng(35)
    n, c, h, w = 3, 3, 9, 10
    x = rng.random((n, c, h, w), dtype=np.float32)
    mean, std = np.array([0.45, 0.4, 0.5], np.float32), np.array([0.225, 0.25, 0.2], np.float32)
    norm = oracle.normalize(x, mean, std)
    xd = G.dev(x)
    mt, st = mean, std
    ld = K.ALIGN[dtype]
    tdt = {K.THB_F32: torch.float32, K.THB_F16: torch.float16, K.THB_U8: torch.uint8}[dtype]
    y = torch.zeros((n, h, w, ld), dtype=tdt, device="cuda")
    qsub = qmult = 0.0
    if dtype == K.THB_U8:
        mm = G.dzeros(2, torch.float32)
        assert lib.thb_minmax_normalized(G.ptr(xd), n, c, h, w, mt.ctypes.data, st.ctypes.data, G.ptr(mm), None) == 0
        torch.cuda.synchronize()
        mn, mx = (float(v) for v in mm.cpu())
        refq, rsub, rmult = oracle.lowp_quantize(norm)
        assert mn == rsub
        qsub, qmult = mn, float(np.float32(255.0 / (np.float64(np.float32(mx) - np.float32(mn)))))
        assert qmult == rmult
    rc = lib.thb_preprocess(G.ptr(xd), G.ptr(xd), n, c, h, w, mt.ctypes.data, st.ctypes.data, dtype, G.ptr(y), ld,
                            qsub, qmult, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(xd.cpu().numpy(), norm)          # in-place normalisation of the fp32 input
    got = G.from_nhwc(y, c)
    if dtype == K.THB_U8:
        assert np.array_equal(got, refq)
    elif dtype == K.THB_F32:
        assert np.array_equal(got, norm)
    else:
        assert np.array_equal(got, norm.astype(np.float16).astype(np.float32))
    # back to NCHW fp32
    out = G.dzeros((n, c, h, w), torch.float32)
    inv = float(np.float32(1.0 / np.float64(np.float32(qmult)))) if dtype == K.THB_U8 else 1.0
    assert lib.thb_postprocess(G.ptr(y), dtype, n, h, w, c, ld, qsub, inv, G.ptr(out), None) == 0
    torch.cuda.synchronize()
    if dtype == K.THB_U8:
        assert np.array_equal(out.cpu().numpy(), oracle.lowp_dequantize(refq, rsub, rmult))
    else:
        assert np.array_equal(out.cpu().numpy(), got)


@pytest.mark.parametrize("coefs", [(1, -1), (1, 1), (-1, 1)])
@pytest.mark.parametrize("thr", [-1, 127])
def test_u8_combine(lib, G, coefs, thr):
    """The uint8 CAddTable of residual networks (no reference counterpart): sat(floor(ca*qa + cb*qb - (ca+cb-1)*127.5)),
    then the Threshold bytes; padded channels stay zero."""
    rng = np.random.default_rng(61)
    n, c, h, w = 2, 20, 5, 7
    a = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
    b = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
    ca, cb = coefs
    ref = np.floor(ca * a.astype(np.float64) + cb * b.astype(np.float64) - (ca + cb - 1) * 127.5)
    ref = np.clip(ref, 0, 255)
    if thr >= 0:
        ref = np.where(ref > thr, ref, 127)
    at, ld = G.to_nhwc(a, K.THB_U8)
    bt, _ = G.to_nhwc(b, K.THB_U8)
    y = torch.full((n, h, w, ld), 9, dtype=torch.uint8, device="cuda")
    rc = lib.thb_u8_combine(G.ptr(at), ld, G.ptr(bt), ld, ca, cb, thr, 127, n * h * w, c, G.ptr(y), ld, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(G.from_nhwc(y, c), ref.astype(np.uint8))
    assert int(y[..., c:].max()) == 0


def test_u8_avgpool(lib, G):
    """Unpadded uint8 average pooling = floor(sum / window) (extension for residual networks)."""
    rng = np.random.default_rng(62)
    n, c, h, w, k = 3, 40, 7, 7, 7
    x = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
    ref = (x.astype(np.int64).sum(axis=(2, 3)) // (k * k)).astype(np.uint8).reshape(n, c, 1, 1)
    xt, ld = G.to_nhwc(x, K.THB_U8)
    y = torch.zeros((n, 1, 1, ld), dtype=torch.uint8, device="cuda")
    rc = lib.thb_avgpool(K.THB_U8, G.ptr(xt), n, h, w, c, ld, k, k, k, k, 0, 0, 1, 1, 0, G.ptr(y), ld, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(G.from_nhwc(y, c), ref)


@pytest.mark.parametrize("shape", [(37, 40), (5, 2500), (300, 64), (3, 25088)])
def test_u8_channel_sum(lib, G, shape):
    """per-pixel sum of the first C bytes (both the thread-per-pixel and the block-per-pixel kernel)"""
    pixels, c = shape
    ld = G.ru(c, 16) + 16
    x = np.random.default_rng(40).integers(0, 256, (pixels, ld), dtype=np.uint8)
    xt = G.dev(x)
    out = G.dzeros(pixels, torch.int32)
    assert lib.thb_u8_channel_sum(G.ptr(xt), pixels, c, ld, G.ptr(out), None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), x[:, :c].astype(np.int64).sum(axis=1))
