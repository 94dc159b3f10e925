"""Whole-network parity through the public C API (THLoadNetwork / THCreate*Network / THProcessFloat)
on the GPU, against the CPU oracle on the same seeded fixture files and inputs.

The five benchmark architectures run at reduced width / size so that the CPU side finishes in seconds.
Metric: max|y - ref| / max|ref| per output tensor; fp32 <= 1e-4, fp16/bf16 <= 1e-2; uint8 bit-exact.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
os.environ.setdefault("THB200_NO_EXIT", "1")

from thnets_b200 import fixtures as fx  # noqa: E402
from thnets_b200.capi import THNets  # noqa: E402

# bf16 keeps 8 mantissa bits (unit round-off 3.9e-3, fp16: 4.9e-4): a ten-layer network lands at a few 1e-2
TOL = {0: 1e-4, 1: 1e-2, 2: 6e-2}

NETS = {
    "alexnet_owt": (lambda: fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128), 1, "t7"),
    "alexnet_owt_b5": (lambda: fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128), 5, "t7"),
    "resnet18": (lambda: fx.resnet18(width=0.25, size=64, classes=10), 4, "py"),
    "resnet50": (lambda: fx.resnet50(width=0.125, size=64, classes=10), 3, "py"),
    "segnet": (lambda: fx.segnet(width=0.5, size=32, classes=21), 2, "py"),
    "segnet_bias": (lambda: fx.segnet(width=0.5, size=32, classes=5, deconv_bias=0.1), 2, "py"),
    "vgg16": (lambda: fx.vgg16(width=0.125, size=32, classes=10, fc=64), 2, "t7"),
    "resnet18_b9": (lambda: fx.resnet18(width=0.25, size=64, classes=10), 9, "py"),
}


@pytest.fixture(scope="module")
def th():
    return THNets()


def rel_err(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(ref, np.float64)).max() / max(np.abs(ref).max(), 1e-30))


def _load(th, g, kind, tmp_path, name):
    if kind == "t7":
        d = str(tmp_path / name)
        fx.write_torch7(g, d)
        return th.load_network(d)
    p = str(tmp_path / (name + ".net"))
    fx.write_pymodel(g, p)
    h = th.load_network(p)
    th.set_stats(h, g.mean, g.std)
    return h


@pytest.mark.parametrize("mode", [0, 1, 2], ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("name", list(NETS))
def test_network_parity(th, oracle, tmp_path, name, mode):
    build, batch, kind = NETS[name]
    g = build()
    x = g.make_input(batch)
    ref = oracle.run(g, x)
    h = _load(th, g, kind, tmp_path, name)
    th.lib.THB200_SetPrecision(mode)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)  # the converted network must own everything it needs
    out, ow, oh = th.process_float(hc, x)
    assert out.size == ref.size, (out.size, ref.shape)
    if ref.ndim == 4:
        assert (ow, oh) == (ref.shape[3], ref.shape[2])
    else:
        assert (ow, oh) == (1, 1)
    err = rel_err(out, ref.ravel())
    assert err < TOL[mode], (name, mode, err)
    # a second forward on the same handle gives the same answer (nothing is consumed by a forward)
    out2, _, _ = th.process_float(hc, x)
    assert np.array_equal(out, out2)
    th.free_network(hc)


@pytest.mark.parametrize("name", ["alexnet_owt_b5", "resnet18", "resnet50", "segnet_bias", "vgg16"])
@pytest.mark.parametrize("variant", [{}, {"bias_as_add": True, "pad_nodes": True}], ids=["plain", "add_pad"])
def test_onnx_network_parity(th, oracle, tmp_path, name, variant):
    """The same networks through the ONNX reader (batch-norm absorbed into the convolutions in fp32 as absorb_bn does,
    onnx.cc:472-570): fp32 results within 1e-4 of the CPU oracle."""
    build, batch, _ = NETS[name]
    g = build()
    x = g.make_input(batch)
    ref = oracle.run(g, x)
    p = str(tmp_path / (name + ".onnx"))
    fx.write_onnx(g, p, **variant)
    h = th.load_network(p)
    th.set_stats(h, g.mean, g.std)
    hc = th.lib.THCreateCudaNetwork(h)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)
    out, _, _ = th.process_float(hc, x)
    assert out.size == ref.size
    assert rel_err(out, ref.ravel()) < 1e-4
    th.free_network(hc)


@pytest.mark.parametrize("mode", [0, 1], ids=["fp32", "fp16"])
def test_onnx_sigmoid_tanh(th, oracle, tmp_path, mode):
    """Sigmoid and Tanh exist on the ONNX route only, as in the reference (onnx.cc:59-60, modules/Sigmoid.c, Tanh.c):
    fused into the convolution before them or run as a kernel of their own (after the pooling)."""
    g = fx.Graph(7)
    g.input_shape = (3, 20, 20)
    x = g.sigmoid(g.conv(0, 3, 12, 3, 1, 1, bias=0.1))
    x = g.tanh(g.maxpool(x, 2, 2))
    x = g.tanh(g.conv(x, 12, 20, 3, 1, 1, bias=0.1))
    x = g.view(x, 20 * 10 * 10)
    g.sigmoid(g.linear(x, 20 * 10 * 10, 7, bias=0.1))
    xin = g.make_input(3)
    ref = oracle.run(g, xin)
    p = str(tmp_path / "st.onnx")
    fx.write_onnx(g, p)
    h = th.load_network(p)
    th.lib.THB200_SetPrecision(mode)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)
    out, _, _ = th.process_float(hc, xin)
    assert rel_err(out, ref.ravel()) < TOL[mode]
    th.free_network(hc)


def test_unconverted_network_runs_on_gpu_fp32(th, oracle, tmp_path):
    g = fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128)
    x = g.make_input(1)
    h = _load(th, g, "t7", tmp_path, "alex")
    buf = np.array(x, copy=True)
    out, _, _ = th.process_float(h, buf, copy_input=False)
    assert rel_err(out, oracle.run(g, x).ravel()) < 1e-4
    # the caller's buffer now holds the normalised input, as with the reference (thapi.c:396-403)
    assert np.array_equal(buf, oracle.normalize(x, g.mean, g.std))
    th.free_network(h)


@pytest.mark.parametrize("batch", [1, 2, 5])
def test_lowp_vgg_bit_exact(th, oracle, tmp_path, batch):
    """THMakeSpatial + THCreateLowpNetwork: every output byte equals the oracle's (dequantised floats equal)."""
    size, rng = 32, 8.0
    g = fx.vgg16(width=0.125, size=size, classes=10, fc=64)
    x = g.make_input(batch)
    ref = oracle.run_lowp(g, x, rng, size)
    h = _load(th, g, "t7", tmp_path, "vgg")
    th.make_spatial(h, size)
    hl = th.create_lowp_network(h, rng)
    th.free_network(h)
    out, ow, oh = th.process_float(hl, x)
    assert (ow, oh) == (1, 1)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    out2, _, _ = th.process_float(hl, x)      # the reference loses its scales after one forward; this does not
    assert np.array_equal(out2, out)
    th.free_network(hl)


@pytest.mark.parametrize("prec", [0, 1])
def test_join_without_copies(th, oracle, tmp_path, monkeypatch, prec):
    """JoinTable along the channels: the producers of the joined tensors (here the col2im of a transposed convolution and
    an encoder convolution that a pooling reads as well) write straight into their channel slice of the joined buffer.
    Same numbers as with the copies (THB200_JOIN_COPY=1), fewer launches, and both match the oracle."""
    g = fx.segnet(width=0.5, size=32, classes=7)
    x = g.make_input(3)
    ref = oracle.run(g, x)
    outs, launches = [], []
    for keep in ("0", "1"):
        monkeypatch.setenv("THB200_JOIN_COPY", keep)
        h = _load(th, g, "py", tmp_path, "seg" + keep)
        th.lib.THB200_SetPrecision(prec)
        hc = th.lib.THCreateCudaNetwork(h)
        th.free_network(h)
        th.process_float(hc, x)                     # plans and warms up
        n0 = th.lib.THB200_KernelLaunches()
        out, _, _ = th.process_float(hc, x)
        launches.append(th.lib.THB200_KernelLaunches() - n0)
        outs.append(out.copy())
        th.free_network(hc)
    th.lib.THB200_SetPrecision(0)
    assert np.array_equal(outs[0], outs[1])
    assert launches[0] <= launches[1] - 6, launches   # four joins of two tensors, at least six copies gone
    err = np.abs(outs[0] - ref.ravel()).max() / np.abs(ref).max()
    assert err < (1e-4 if prec == 0 else 1e-2), err


def test_lowp_rejects_what_the_reference_rejects(th, tmp_path):
    """SpatialFullConvolution and JoinTable have no lowp implementation (lowp_basic.c:197-208)."""
    g = fx.segnet(width=0.25, size=32, classes=5)
    h = _load(th, g, "py", tmp_path, "seg")
    hl = th.lib.THCreateLowpNetwork(h, 8.0)
    if hl:
        x = g.make_input(1)
        n = th.lib.THProcessFloat
        import ctypes as C
        res = C.POINTER(C.c_float)()
        ow, oh = C.c_int(), C.c_int()
        assert n(hl, x.ctypes.data_as(C.c_void_p), 1, 32, 32, 3, C.byref(res), C.byref(ow), C.byref(oh)) == 0
        assert b"lowp" in th.lib.THB200_LastErrorString().lower()
        th.free_network(hl)
    th.free_network(h)


@pytest.mark.parametrize("arch,width", [("resnet18", 0.25), ("resnet50", 0.125)])
@pytest.mark.parametrize("batch", [1, 3])
def test_lowp_residual_network_bit_exact(th, oracle, tmp_path, arch, width, batch):
    """uint8 residual networks: an extension with no reference counterpart (the reference's lowp engine refuses batch
    normalisation and average pooling and converts no CAddTable).  Folded batch-norm, the uint8 a - b of CAddTable and
    the floor-mean pooling follow the rules stated in oracle.run_lowp; every output byte equals that restatement's."""
    size, rng = 64, 20.0
    g = getattr(fx, arch)(width=width, size=size, classes=10, fc_bias=0.05)
    x = g.make_input(batch)
    ref = oracle.run_lowp(g, x, rng, size)
    h = _load(th, g, "py", tmp_path, arch)
    hl = th.create_lowp_network(h, rng)
    th.free_network(h)
    out, _, _ = th.process_float(hl, x)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    assert len(np.unique(out)) > 3          # the logits are not a saturated constant
    th.free_network(hl)


def test_process_images_matches_float_path(th, oracle, tmp_path):
    g = fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128)
    h = _load(th, g, "t7", tmp_path, "alex")
    rng = np.random.default_rng(3)
    for batch in (1, 3):
        imgs = [rng.integers(0, 256, (224, 224, 3)).astype(np.uint8) for _ in range(batch)]
        out, _, _ = th.process_images(h, imgs, bgr=0)
        import ctypes as C
        dst = np.empty((batch, 3, 224, 224), np.float32)
        ptrs = (C.POINTER(C.c_ubyte) * batch)(*[i.ctypes.data_as(C.POINTER(C.c_ubyte)) for i in imgs])
        oracle.lib.orc_images_to_float(ptrs, batch, 224, 224, 224 * 3, 3, g.mean.ctypes.data_as(C.POINTER(C.c_float)),
                                       g.std.ctypes.data_as(C.POINTER(C.c_float)), 0, dst.ctypes.data_as(C.POINTER(C.c_float)))
        plain = fx.Graph()
        plain.nodes, plain.output = g.nodes, g.output   # same weights, identity statistics
        ref = oracle.run(plain, dst)
        assert rel_err(out, ref.ravel()) < 1e-4
    th.free_network(h)


def test_pageable_batches_are_staged_through_pinned_memory(th, tmp_path, monkeypatch):
    """A float batch in ordinary host memory (>= 8 MB) is copied into the library's pinned buffer by the host threads, slice
    by slice, and sent from there: same result as handing the pointer to the driver (THB200_NO_STAGING=1), with and
    without sub-batches, and the caller's buffer gets its in-place normalisation either way."""
    g = fx.alexnet_owt(width=0.25, size=224, classes=20, fc=64)
    x = g.make_input(16)                                   # 9.6 MB
    h = _load(th, g, "t7", tmp_path, "alexpg")
    outs, bufs = [], []
    for chunks, nostage in ((1, "0"), (2, "0"), (1, "1"), (2, "1")):
        monkeypatch.setenv("THB200_NO_STAGING", nostage)
        th.lib.THB200_SetPipelineChunks(chunks)
        buf = np.array(x, copy=True)
        out, _, _ = th.process_float(h, buf, copy_input=False)
        outs.append(out)
        bufs.append(buf)
    th.lib.THB200_SetPipelineChunks(0)
    th.free_network(h)
    assert np.array_equal(outs[0], outs[2]) and np.array_equal(outs[1], outs[3])      # staged == not staged
    assert rel_err(outs[1], outs[0]) < 1e-5     # (sub-batches of 6 and 10 images may take other fp32 tile shapes than 16)
    assert all(np.array_equal(bufs[0], b) for b in bufs[1:])
    assert np.array_equal(bufs[0], (x - np.float32(0.45)) / np.float32(0.225))   # normalised in place: thapi.c:396-403
    # byte images that follow one another in ordinary memory take the same route
    h = _load(th, g, "t7", tmp_path, "alexpg2")
    imgs = np.random.default_rng(4).integers(0, 256, (64, 224, 224, 3)).astype(np.uint8)   # 9.6 MB
    got = []
    for nostage in ("0", "1"):
        monkeypatch.setenv("THB200_NO_STAGING", nostage)
        got.append(th.process_images(h, list(imgs))[0])
    th.free_network(h)
    assert np.array_equal(got[0], got[1])


def test_in_place_normalisation_of_a_page_locked_batch(th, tmp_path):
    """THProcessFloat leaves (x - mean) / std in the caller's tensor (thapi.c:396-403).  For a batch in page-locked memory
    the device normalises and the values come back on a stream of their own beside the forward: when the call returns the
    buffer holds them, and the result equals that of the same batch in ordinary memory."""
    g = fx.alexnet_owt(width=0.25, size=224, classes=20, fc=64)
    x = g.make_input(3)                                    # 1.8 MB: below the size from which ordinary memory is staged
    h = _load(th, g, "t7", tmp_path, "alexpin")
    p = th.lib.THB200_HostAlloc(C.c_size_t(x.nbytes))
    assert p
    pinned = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=x.shape)
    want = (x - np.float32(0.45)) / np.float32(0.225)
    for _ in range(3):                                     # direct launches, the capture, a replay
        pinned[...] = x
        out, _, _ = th.process_float(h, pinned, copy_input=False)
        assert np.array_equal(pinned, want)
        plain = np.array(x, copy=True)
        out2, _, _ = th.process_float(h, plain, copy_input=False)
        assert np.array_equal(plain, want) and np.array_equal(out, out2)
    th.free_network(h)
    th.lib.THB200_HostFree(C.c_void_p(p))


@pytest.mark.parametrize("entry", ["float", "images"])
def test_first_layer_on_sixteen_stored_channels(th, oracle, tmp_path, monkeypatch, entry):
    """A stride-1 first convolution on three channels (VGG, the segmentation net) in the 16-bit modes: the input is staged
    with 16 channels per pixel (zeros behind the real ones) and the layer runs as a 16-channel convolution through the
    patch kernel.  Same result as the gathered 8-channel layout (THB200_NO_PAD16=1) within fp16 rounding, both within
    tolerance of the oracle, through both entry points."""
    g = fx.vgg16(width=0.25, size=64, classes=10, fc=64)
    rng = np.random.default_rng(11)
    if entry == "float":
        x = g.make_input(3)
        ref = oracle.run(g, x).ravel()
    else:
        imgs = [rng.integers(0, 256, (64, 64, 3)).astype(np.uint8) for _ in range(3)]
        import ctypes as C
        dst = np.empty((3, 3, 64, 64), np.float32)
        ptrs = (C.POINTER(C.c_ubyte) * 3)(*[i.ctypes.data_as(C.POINTER(C.c_ubyte)) for i in imgs])
        oracle.lib.orc_images_to_float(ptrs, 3, 64, 64, 64 * 3, 3, g.mean.ctypes.data_as(C.POINTER(C.c_float)),
                                       g.std.ctypes.data_as(C.POINTER(C.c_float)), 0, dst.ctypes.data_as(C.POINTER(C.c_float)))
        plain = fx.Graph()
        plain.nodes, plain.output = g.nodes, g.output
        ref = oracle.run(plain, dst).ravel()
    outs = []
    for off in ("0", "1"):
        monkeypatch.setenv("THB200_NO_PAD16", off)
        hc = _convert(th, g, "t7", tmp_path, "vggp16" + off + entry, 1)
        out = th.process_float(hc, x)[0] if entry == "float" else th.process_images(hc, imgs)[0]
        th.free_network(hc)
        assert rel_err(out, ref) < 1e-2
        outs.append(out)
    assert rel_err(outs[0], outs[1]) < 5e-3


@pytest.mark.parametrize("batch", [1, 3])
def test_lowp_first_layer_staged_as_neighbourhoods(th, oracle, tmp_path, monkeypatch, batch):
    """uint8 engine, VGG's first layer (3x3 / stride 1 / pad 1 on three planes): the boundary kernel stages every pixel's 27
    quantised neighbours (the byte of 0.0 outside the image) and the layer runs as a 1x1 convolution.  Every output byte
    equals the gathered 3x3 layer's (THB200_NO_NEIGH_U8=1) and the lowp oracle's; the caller's buffer is normalised in
    place the same way."""
    rng_ = 16.0
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    x = g.make_input(batch)
    ref = oracle.run_lowp(g, x, rng_, 32)
    outs, bufs = [], []
    for off in ("0", "1"):
        monkeypatch.setenv("THB200_NO_NEIGH_U8", off)
        h = _load(th, g, "t7", tmp_path, "vggn" + off)
        th.make_spatial(h, 32)
        hl = th.create_lowp_network(h, rng_)
        th.free_network(h)
        buf = np.array(x, copy=True)
        out, _, _ = th.process_float(hl, buf, copy_input=False)
        th.free_network(hl)
        assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
        outs.append(out)
        bufs.append(buf)
    assert np.array_equal(bufs[0], bufs[1])


def test_split_reductions_on_request(th, oracle, tmp_path, monkeypatch):
    """THB200_SPLITK=1: few-tile layers of the 16-bit engines (here every layer of a small-batch VGG and its Linear layers)
    share their reductions among CTAs.  Within tolerance of the oracle and of the default plan; off by default because a
    sharded batch would no longer reproduce the whole batch bit for bit."""
    g = fx.vgg16(width=0.5, size=32, classes=10, fc=256)
    x = g.make_input(4)
    ref = oracle.run(g, x).ravel()
    outs, launches = [], []
    for on in ("0", "1"):
        monkeypatch.setenv("THB200_SPLITK", on)
        hc = _convert(th, g, "t7", tmp_path, "vggsk" + on, 1)
        th.process_float(hc, x)
        n0 = th.lib.THB200_KernelLaunches()
        monkeypatch.setenv("THB200_NO_GRAPH", "1")
        out = th.process_float(hc, x)[0]
        launches.append(th.lib.THB200_KernelLaunches() - n0)
        th.free_network(hc)
        assert rel_err(out, ref) < 1e-2
        outs.append(out)
    assert launches[1] > launches[0], launches           # the finishing launches of the split layers
    assert rel_err(outs[1], outs[0]) < 5e-3


def test_process_yuyv(th, oracle, tmp_path):
    """THProcessYUYV (thapi.c:575-612): the frame is converted on the GPU with the reference's integer tables; a network
    as loaded takes it, a converted one refuses it as the reference's converted networks do."""
    from oracle.oracle import yuyv_to_float
    g = fx.alexnet_owt(width=0.25, size=64, classes=10, fc=32)
    h = _load(th, g, "t7", tmp_path, "alexyuv")
    rng = np.random.default_rng(8)
    frame = rng.integers(0, 256, 64 * 64 * 2).astype(np.uint8)
    frame[:64] = np.tile(np.array([0, 0, 255, 255, 16, 128, 235, 128], np.uint8), 8)   # the corners of the tables
    out, ow, oh = th.process_yuyv(h, frame, 64, 64)
    x = yuyv_to_float(frame, 64, 64, g.mean, g.std)[None]
    plain = fx.Graph()
    plain.nodes, plain.output = g.nodes, g.output
    ref = oracle.run(plain, x)
    assert (ow, oh) == (1, 1)
    assert rel_err(out, ref.ravel()) < 1e-4
    hc = th.lib.THCreateCudaNetwork(h)
    th.free_network(h)
    none, _, _ = th.process_yuyv(hc, frame, 64, 64)
    assert none is None and b"not supported" in th.lib.THB200_LastErrorString()
    th.free_network(hc)


def _convert(th, g, kind, tmp_path, name, mode):
    h = _load(th, g, kind, tmp_path, name)
    th.lib.THB200_SetPrecision(mode)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)
    return hc


@pytest.mark.parametrize("chunks", [2, 3, 4])
def test_pipelined_sub_batches_give_the_same_result(th, oracle, tmp_path, chunks):
    """THProcessFloat may cut the batch into sub-batches whose copies overlap the kernels of the previous one: every
    image is computed by the same kernels in the same order, so the result is identical bit for bit."""
    g = fx.resnet18(width=0.25, size=64, classes=10)
    x = g.make_input(9)
    hc = _convert(th, g, "py", tmp_path, "r18p", 1)
    try:
        th.lib.THB200_SetPipelineChunks(1)
        whole, _, _ = th.process_float(hc, x)
        th.lib.THB200_SetPipelineChunks(chunks)
        for _ in range(3):   # direct launches, then graph capture, then graph replay
            cut, _, _ = th.process_float(hc, x)
            assert np.array_equal(whole, cut)
    finally:
        th.lib.THB200_SetPipelineChunks(0)
    assert rel_err(whole, oracle.run(g, x).ravel()) < TOL[1]
    th.free_network(hc)


def test_pipelined_images_give_the_same_result(th, tmp_path):
    """THProcessImages pipelines sub-batches the same way (device-side conversion of each sub-batch's bytes)."""
    g = fx.resnet18(width=0.25, size=64, classes=10)
    hc = _convert(th, g, "py", tmp_path, "r18i", 1)
    rng = np.random.default_rng(5)
    imgs = [rng.integers(0, 256, (64, 64, 3)).astype(np.uint8) for _ in range(7)]
    try:
        th.lib.THB200_SetPipelineChunks(1)
        whole = th.process_images(hc, imgs, bgr=0)[0].copy()
        for chunks in (2, 3):
            th.lib.THB200_SetPipelineChunks(chunks)
            for _ in range(3):
                assert np.array_equal(whole, th.process_images(hc, imgs, bgr=0)[0])
    finally:
        th.lib.THB200_SetPipelineChunks(0)
    th.free_network(hc)


def test_graph_replay_matches_direct_launches(th, tmp_path):
    g = fx.resnet50(width=0.125, size=64, classes=10)
    x = g.make_input(3)
    hc = _convert(th, g, "py", tmp_path, "r50g", 1)
    outs = [th.process_float(hc, x)[0].copy() for _ in range(4)]   # 1st: direct; 2nd: captured; then replays
    for o in outs[1:]:
        assert np.array_equal(outs[0], o)
    th.free_network(hc)


def test_lowp_graph_replay_follows_the_input_range(th, oracle, tmp_path):
    """The uint8 engine measures the input's quantisation per batch (lowp_basic.c:299-321): the convolutions that read
    the network input are launched directly with that batch's parameters and only the launches after them are replayed
    from the graph.  Batches of different ranges, one after the other through the same network: every result equals the
    oracle's for that batch."""
    size, rng = 64, 20.0
    g = fx.resnet50(width=0.125, size=size, classes=10, fc_bias=0.05)
    h = _load(th, g, "py", tmp_path, "r50lg")
    hl = th.create_lowp_network(h, rng)
    th.free_network(h)
    x0 = g.make_input(3)
    for k, gain in enumerate([1.0, 0.37, 2.5, 1.0, 0.05]):      # 1st: direct; 2nd: captured; then replays
        x = (x0 * gain + 0.1 * k).astype(np.float32)
        ref = oracle.run_lowp(g, x, rng, size)
        out, _, _ = th.process_float(hl, x.copy())
        assert np.array_equal(out, ref.ravel()), (k, np.abs(out - ref.ravel()).max())
    th.free_network(hl)


def test_batch_sharded_over_two_gpus(th, oracle, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    g = fx.resnet18(width=0.25, size=64, classes=10)
    x = g.make_input(9)
    one = _convert(th, g, "py", tmp_path, "r18one", 1)
    ref, _, _ = th.process_float(one, x)
    th.free_network(one)
    for gather in ("peer", "host"):
        os.environ["THB200_GATHER"] = gather
        th.lib.THB200_SetDevices(2)
        try:
            two = _convert(th, g, "py", tmp_path, "r18two" + gather, 1)
        finally:
            th.lib.THB200_SetDevices(1)
            os.environ.pop("THB200_GATHER", None)
        out, _, _ = th.process_float(two, x)
        assert np.array_equal(out, ref), gather
        th.free_network(two)


@pytest.mark.parametrize("bgr", [0, 1])
@pytest.mark.parametrize("batch", [1, 3])
def test_lowp_images_bit_exact(th, oracle, tmp_path, batch, bgr):
    """THProcessImages on the uint8 engine: the image loader's static input range (lowp_basic.c:82-131), then the same
    network as test_lowp_vgg_bit_exact; every output byte equals the oracle's."""
    size, rng = 32, 8.0
    g = fx.vgg16(width=0.125, size=size, classes=10, fc=64)
    g.mean, g.std = np.array([0.45, 0.42, 0.40], np.float32), np.array([0.225, 0.23, 0.22], np.float32)
    r = np.random.default_rng(17)
    imgs = [r.integers(0, 256, (size, size, 3)).astype(np.uint8) for _ in range(batch)]
    ref = oracle.run_lowp(g, None, rng, size, quantised_input=oracle.lowp_images(imgs, g.mean, g.std, bgr))
    h = _load(th, g, "t7", tmp_path, "vggi")
    th.make_spatial(h, size)
    hl = th.create_lowp_network(h, rng)
    th.free_network(h)
    out, ow, oh = th.process_images(hl, imgs, bgr=bgr)
    assert (ow, oh) == (1, 1)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    th.free_network(hl)


# ------------------------------------------------------------------------------------------ full-width networks
# The benchmark architectures at their real channel widths and input sizes (small batches, so that the CPU oracle
# finishes in seconds): every layer runs with the tile shapes, pipeline depths and fusions the benchmark uses.
FULL = {
    "resnet50": (lambda: fx.resnet50(), 4, "py"),
    "resnet18": (lambda: fx.resnet18(), 4, "py"),
    "alexnet_owt": (lambda: fx.alexnet_owt(), 1, "t7"),
    "vgg16": (lambda: fx.vgg16(fc=512), 1, "t7"),
    "segnet": (lambda: fx.segnet(size=256), 2, "py"),
}


@pytest.mark.parametrize("name,mode", [("resnet50", 1), ("resnet50", 0), ("resnet18", 1), ("alexnet_owt", 0), ("vgg16", 1),
                                       ("segnet", 1)])
def test_full_width_network_parity(th, oracle, tmp_path, name, mode):
    build, batch, kind = FULL[name]
    g = build()
    x = g.make_input(batch)
    ref = oracle.run(g, x)
    hc = _convert(th, g, kind, tmp_path, name + "_full", mode)
    out, _, _ = th.process_float(hc, x)
    assert out.size == ref.size
    err = rel_err(out, ref.ravel())
    assert err < TOL[mode], (name, mode, err)
    if ref.ndim == 2:
        agree = float((out.reshape(ref.shape).argmax(1) == ref.argmax(1)).mean())
        assert agree == 1.0, (name, "arg-max agreement", agree)
    th.free_network(hc)


def test_full_width_resnet50_uint8_bit_exact(th, oracle, tmp_path):
    """ResNet-50 at full width and 224 x 224 through the uint8 engine, range 20 (the benchmark's int8 configuration at
    batch 2): every output byte equals the restatement's (see test_lowp_residual_network_bit_exact for its rules)."""
    g = fx.resnet50(fc_bias=0.01)
    x = g.make_input(2)
    ref = oracle.run_lowp(g, x, 20.0, 224)
    h = _load(th, g, "py", tmp_path, "r50u8")
    hl = th.create_lowp_network(h, 20.0)
    th.free_network(h)
    out, _, _ = th.process_float(hl, x)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    assert len(np.unique(out)) > 3
    th.free_network(hl)


def test_full_width_vgg16_uint8_bit_exact(th, oracle, tmp_path):
    """VGG-16 at full width and 224 x 224 through THMakeSpatial + THCreateLowpNetwork, range 20, batch 2 (the hidden
    classifier layers narrowed to 512 to keep the fixture file small): bit-exact."""
    g = fx.vgg16(fc=512)
    x = g.make_input(2)
    ref = oracle.run_lowp(g, x, 20.0, 224)
    h = _load(th, g, "t7", tmp_path, "vggu8")
    th.make_spatial(h, 224)
    hl = th.create_lowp_network(h, 20.0)
    th.free_network(h)
    out, _, _ = th.process_float(hl, x)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    th.free_network(hl)


def test_lowp_first_convolution_15x15_stride_2(th, oracle, tmp_path):
    """A uint8 network whose first convolution is 15x15 / stride 2 / pad 7 on three channels: after the space-to-depth
    rewrite its kernel row is 8 taps of 16 bytes, the shape for which 16-bit types store the staged rows with padding.
    The uint8 loader and channel sums use dense rows, and the result must be bit-exact all the same."""
    g = fx.Graph(11)
    g.input_shape, g.input_dist = (3, 48, 48), "uniform"
    x = g.relu(g.conv(0, 3, 24, 15, 2, 7, bias=0.05))
    x = g.maxpool(x, 2, 2)
    x = g.relu(g.conv(x, 24, 32, 3, 1, 1, bias=0.05))
    g.conv(x, 32, 10, 12, 1, 0, bias=0.05)
    xin = g.make_input(3)
    ref = oracle.run_lowp(g, xin, 8.0, 48)
    h = _load(th, g, "t7", tmp_path, "first15")
    hl = th.create_lowp_network(h, 8.0)
    th.free_network(h)
    out, _, _ = th.process_float(hl, xin)
    assert np.array_equal(out, ref.ravel()), np.abs(out - ref.ravel()).max()
    th.free_network(hl)


# ------------------------------------------------------------------------- operators outside the benchmark networks
@pytest.mark.parametrize("case", [("unpool_zeropad_b1", lambda: fx.unpool_net(), "t7", 1, 0),
                                  ("unpool_b3", lambda: fx.unpool_net(zeropad=False), "t7", 3, 0),
                                  ("unpool_zeropad_b3", lambda: fx.unpool_net(), "t7", 3, 0),
                                  ("normalize_b1", lambda: fx.normalize_net(), "t7", 1, 0),
                                  ("normalize_b4", lambda: fx.normalize_net(), "t7", 4, 0),
                                  ("normalize_b4_fp16", lambda: fx.normalize_net(), "t7", 4, 1),
                                  ("reshape_b1", lambda: fx.reshape_net(), "t7", 1, 0),
                                  ("reshape_b3", lambda: fx.reshape_net(), "t7", 3, 0),
                                  ("reshape_b3_fp16", lambda: fx.reshape_net(), "t7", 3, 1),
                                  ("prelu_b1", lambda: fx.prelu_net(), "t7", 1, 0),
                                  ("prelu_b3", lambda: fx.prelu_net(), "t7", 3, 0),
                                  ("prelu_b3_fp16", lambda: fx.prelu_net(), "t7", 3, 1),
                                  ("prelu_leaky_onnx_b3", lambda: fx.prelu_net(onnx_form=True), "onnx", 3, 0),
                                  ("prelu_leaky_onnx_b3_fp16", lambda: fx.prelu_net(onnx_form=True), "onnx", 3, 1),
                                  ("cmax_slice_b4", lambda: fx.cmax_slice_net(), "py", 4, 0),
                                  ("cmax_slice_b4_fp16", lambda: fx.cmax_slice_net(), "py", 4, 1),
                                  ("onnx_ops_b3", lambda: fx.onnx_ops_net(), "onnx", 3, 0),
                                  ("onnx_ops_b1", lambda: fx.onnx_ops_net(), "onnx", 1, 0)], ids=lambda c: c[0])
def test_remaining_operators(th, oracle, tmp_path, case):
    """SpatialZeroPadding, SpatialMaxUnpooling (positions recomputed from the pooling's input), LogSoftMax (with the
    reference's first-frame quirk), Normalize, Reshape to a [c, h, w] map (with and without a batch dimension), PReLU (a
    slope per channel, one shared slope, on maps and on vectors) and the leaky Threshold an ONNX LeakyRelu makes, Cmax,
    Slice along every dimension and Upsample, through the three loaders,
    against the oracle functions that are pinned to the live reference."""
    name, build, kind, batch, mode = case
    g = build()
    x = g.make_input(batch)
    ref = oracle.run(g, x)
    if name == "normalize_b1":
        ref = oracle.l2_normalize(oracle.run(g, x, keep=True)[len(g.nodes) - 2].ravel())   # View gives a 1-D tensor at batch 1
    if kind == "onnx":
        p = str(tmp_path / (name + ".onnx"))
        fx.write_onnx(g, p)
        h = th.load_network(p)
        th.set_stats(h, g.mean, g.std)
    else:
        h = _load(th, g, kind, tmp_path, name)
    th.lib.THB200_SetPrecision(mode)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)
    out, _, _ = th.process_float(hc, x)
    assert out.size == ref.size, (out.size, ref.shape)
    err = rel_err(out, ref.ravel())
    assert err < (1e-4 if mode == 0 else 2e-2), (name, err)
    th.free_network(hc)


def test_concat_along_the_batch_dimension(th, oracle, tmp_path):
    """JoinTable along dimension 0 of 4-D tensors (JoinTable.c:46-57): the inputs' images one after the other."""
    g = fx.Graph(9)
    g.input_shape = (3, 10, 10)
    x = g.relu(g.conv(0, 3, 8, 3, 1, 1, bias=0.1))
    a = g.conv(x, 8, 6, 3, 1, 1, bias=0.1)
    b = g.conv(x, 8, 6, 1, 1, 0, bias=0.1)
    j = g.concat([a, b], 0)
    g.conv(j, 6, 4, 3, 1, 1, bias=0.1)
    xin = g.make_input(3)
    ref = oracle.run(g, xin)
    assert ref.shape[0] == 6
    hc = _convert(th, g, "py", tmp_path, "cat0", 0)
    out, _, _ = th.process_float(hc, xin)
    assert out.size == ref.size
    assert rel_err(out, ref.ravel()) < 1e-4
    th.free_network(hc)


def _onnx_attr_net():
    """Convolutions with the attributes only ONNX files carry: ending pads that differ from the leading ones, dilation,
    auto_pad (both kinds, stride 2 on an odd size) and a reflect-mode Pad node in front."""
    g = fx.Graph(10)
    g.input_shape = (3, 15, 13)
    x = g.relu(g.conv(0, 3, 8, 3, 1, 0, bias=0.1, pads4=(1, 0, 2, 1)))
    x = g.relu(g.conv(x, 8, 8, 3, 1, 2, bias=0.1, dilation=2))
    x = g.relu(g.conv(x, 8, 16, 3, 2, 0, bias=0.1, auto_pad="SAME_UPPER"))
    x = g.relu(g.conv(x, 16, 16, 3, 1, 0, bias=0.1, pads4=(2, 2, 2, 2), reflect=True))
    g.conv(x, 16, 5, 4, 2, 0, bias=0.1, auto_pad="SAME_LOWER")
    return g


@pytest.mark.parametrize("mode", [0, 1], ids=["fp32", "fp16"])
@pytest.mark.parametrize("honour", [False, True], ids=["ignored_as_by_the_reference", "honoured"])
def test_onnx_only_convolution_attributes(th, oracle, tmp_path, monkeypatch, mode, honour):
    """By default the ending pads, dilation, auto_pad and reflection padding of an ONNX convolution are ignored exactly as
    the reference ignores them (SpatialConvolution.c:88-109 parses, nothing reads); with THB200_HONOUR_PADS=1 (read when a
    network is converted) the result is what the ONNX model means, checked against a NumPy model of it."""
    g = _onnx_attr_net()
    x = g.make_input(3)
    ref = oracle.run(g, x, honour_pads=honour)
    p = str(tmp_path / "attrs.onnx")
    fx.write_onnx(g, p)
    h = th.load_network(p)
    th.set_stats(h, g.mean, g.std)
    if honour:
        monkeypatch.setenv("THB200_HONOUR_PADS", "1")
    th.lib.THB200_SetPrecision(mode)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    assert hc, th.lib.THB200_LastErrorString()
    th.free_network(h)
    out, ow, oh = th.process_float(hc, x)
    assert out.size == ref.size, (out.size, ref.shape)
    assert (ow, oh) == (ref.shape[3], ref.shape[2])
    assert rel_err(out, ref.ravel()) < TOL[mode]
    th.free_network(hc)


@pytest.mark.parametrize("bgr", [0, 1])
def test_process_images_through_the_space_to_depth_stem(th, oracle, tmp_path, bgr):
    """THProcessImages on a network whose first convolution has stride 2 (fp16): the byte images are normalised and
    regrouped space-to-depth by one kernel, so the stem and its pooling run as for a float batch."""
    import ctypes as C
    g = fx.resnet18(width=0.25, size=64, classes=10)
    g.mean, g.std = np.array([0.45, 0.42, 0.40], np.float32), np.array([0.225, 0.23, 0.22], np.float32)
    hc = _convert(th, g, "py", tmp_path, "r18img", 1)
    rng = np.random.default_rng(23)
    batch = 5
    imgs = [rng.integers(0, 256, (64, 64, 3)).astype(np.uint8) for _ in range(batch)]
    out, _, _ = th.process_images(hc, imgs, bgr=bgr)
    dst = np.empty((batch, 3, 64, 64), np.float32)
    ptrs = (C.POINTER(C.c_ubyte) * batch)(*[i.ctypes.data_as(C.POINTER(C.c_ubyte)) for i in imgs])
    oracle.lib.orc_images_to_float(ptrs, batch, 64, 64, 64 * 3, 3, g.mean.ctypes.data_as(C.POINTER(C.c_float)),
                                   g.std.ctypes.data_as(C.POINTER(C.c_float)), bgr, dst.ctypes.data_as(C.POINTER(C.c_float)))
    plain = fx.Graph()
    plain.nodes, plain.output = g.nodes, g.output   # same weights, identity statistics
    ref = oracle.run(plain, dst)
    assert rel_err(out, ref.ravel()) < TOL[1]
    th.free_network(hc)
