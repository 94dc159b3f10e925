"""The rest of the public surface on the GPU: THForward, struct module.updateOutput, THUseSpatialConvolutionMM and the
th_minmax report -- through the C API, against the CPU oracle."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
os.environ.setdefault("THB200_NO_EXIT", "1")

from thnets_b200 import fixtures as fx  # noqa: E402
from thnets_b200.capi import THNets, THNetworkStruct  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class THFloatTensor(C.Structure):
    """thnets.h:110-120 (CPU build, no LOWP tail)"""
    _fields_ = [("size", C.c_long * 4), ("stride", C.c_long * 4), ("nDimension", C.c_int), ("storage", C.c_void_p),
                ("storageOffset", C.c_long)]


class Network(C.Structure):
    """struct network, thnets.h:403-407"""
    _fields_ = [("nelem", C.c_int), ("engine", C.c_int), ("modules", C.c_void_p)]


MODULE_SIZE, MODULE_UPDATE_OUTPUT, MODULE_OUTPUT = 208, 8, 24     # sizeof / offsetof(struct module), see test_host.py


@pytest.fixture(scope="module")
def th():
    t = THNets()
    lib = t.lib
    lib.THFloatTensor_new.restype = C.c_void_p
    lib.THFloatTensor_resize4d.argtypes = [C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_long]
    lib.THFloatTensor_resize3d.argtypes = [C.c_void_p, C.c_long, C.c_long, C.c_long]
    lib.THFloatTensor_data.restype = C.POINTER(C.c_float)
    lib.THFloatTensor_data.argtypes = [C.c_void_p]
    lib.THFloatTensor_free.argtypes = [C.c_void_p]
    lib.THFloatTensor_nElement.restype = C.c_long
    lib.THFloatTensor_nElement.argtypes = [C.c_void_p]
    lib.THForward.restype = C.c_void_p
    lib.THForward.argtypes = [C.c_void_p, C.c_void_p]
    return t


def rel_err(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(ref, np.float64)).max() / max(np.abs(ref).max(), 1e-30))


def _tensor(lib, x):
    t = lib.THFloatTensor_new()
    if x.ndim == 4:
        lib.THFloatTensor_resize4d(t, *x.shape)
    else:
        lib.THFloatTensor_resize3d(t, *x.shape)
    C.memmove(lib.THFloatTensor_data(t), np.ascontiguousarray(x, np.float32).ctypes.data, x.size * 4)
    return t


def _read(lib, tptr):
    t = THFloatTensor.from_address(tptr)
    shape = tuple(t.size[i] for i in range(t.nDimension))
    n = lib.THFloatTensor_nElement(tptr)
    return np.ctypeslib.as_array(lib.THFloatTensor_data(tptr), shape=(n,)).copy().reshape(shape)


def test_thforward_takes_a_tensor_and_skips_the_normalisation(th, oracle, tmp_path):
    """THForward (thapi.c:237-242) runs the network on a tensor as it is: no mean / std normalisation, rank 3 or 4."""
    g = fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128)
    d = str(tmp_path / "alex")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    plain = fx.Graph()
    plain.nodes, plain.output = g.nodes, g.output          # same weights, identity statistics
    for batch in (2, 1):
        x = g.make_input(batch)
        t = _tensor(th.lib, x)
        out = th.lib.THForward(h, t)
        assert out, th.lib.THB200_LastErrorString()
        got = _read(th.lib, out)
        ref = oracle.run(plain, x)
        assert got.size == ref.size
        assert rel_err(got.ravel(), ref.ravel()) < 1e-4
        th.lib.THFloatTensor_free(t)
    th.free_network(h)


def test_module_update_output_runs_one_module_and_keeps_its_engine(th, oracle, tmp_path):
    """struct module.updateOutput (thnets.h:292-336; external code calls it directly, examples/thnets-tf.cc:113-138): one
    module on the device, host tensor in, module->output out.  The second call on the same record reuses the converted
    module (no new weight upload); results match the oracle's operator."""
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    d = str(tmp_path / "vgg")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    net = Network.from_address(THNetworkStruct.from_address(h).net)
    assert net.nelem >= 3
    x = np.random.default_rng(1).standard_normal((2, 3, 32, 32)).astype(np.float32)
    proto = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_void_p)
    cur_t, cur = _tensor(th.lib, x), x
    l0 = th.lib.THB200_KernelLaunches()
    for i in range(3):                                      # conv, ReLU, conv
        m = net.modules + i * MODULE_SIZE
        fn = proto(C.c_void_p.from_address(m + MODULE_UPDATE_OUTPUT).value)
        for _ in range(2):                                  # the second call reuses the engine kept for the record
            out = fn(m, cur_t)
            assert out == C.c_void_p.from_address(m + MODULE_OUTPUT).value
        node = g.nodes[i + 1]
        ts = [t for _, t in node.tensors]
        ref = oracle.conv2d(cur, ts[0], ts[1], node.attrs["stride"], node.attrs["padding"]) if node.op == "conv" \
            else oracle.threshold(cur, 0.0, 0.0)
        got = _read(th.lib, out)
        assert got.shape == ref.shape
        assert rel_err(got, ref) < 1e-4
        cur_t, cur = out, got
    assert th.lib.THB200_KernelLaunches() - l0 > 0
    th.free_network(h)


def test_use_spatial_convolution_mm_keeps_the_result(th, oracle, tmp_path):
    """THUseSpatialConvolutionMM(net, 0 / 1 / 2) chooses between the reference's CPU convolution algorithms
    (thapi.c:692-728); every choice is the same implicit GEMM here, and the call answers 0."""
    g = fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128)
    d = str(tmp_path / "alex")
    fx.write_torch7(g, d)
    x = g.make_input(2)
    ref = oracle.run(g, x).ravel()
    for choice in (0, 1, 2):
        h = th.load_network(d)
        # 0 asks for the direct algorithm, which the reference refuses for padded convolutions (thapi.c:709-713): -3
        assert th.lib.THUseSpatialConvolutionMM(h, choice) == (0 if choice else -3)
        out, _, _ = th.process_float(h, x)
        assert rel_err(out, ref) < 1e-4
        th.free_network(h)


def test_th_minmax_prints_every_layers_range(tmp_path):
    """th_minmax = 1 (thapi.c:141-154, :197-202): one "Layer N output: min=..., max=..." line per launch -- what a caller
    reads to choose the lowp range.  Run in a child process (the report goes to stdout)."""
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    d = str(tmp_path / "vgg")
    fx.write_torch7(g, d)
    code = f"""
import sys, ctypes as C
sys.path.insert(0, {ROOT!r})
from thnets_b200.capi import THNets
from thnets_b200 import fixtures as fx
th = THNets()
C.c_int.in_dll(th.lib, "th_minmax").value = 1
h = th.load_network({d!r})
g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
out, _, _ = th.process_float(h, g.make_input(2))
sys.stdout.flush()
print("LOGITS", float(out.min()), float(out.max()))
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=dict(os.environ, THB200_NO_EXIT="1"))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("Layer ")]
    assert len(lines) >= 16, r.stdout
    lo, hi = [float(v) for v in r.stdout.splitlines()[-1].split()[1:]]
    last = lines[-1]
    mn = float(last.split("min=")[1].split(",")[0])
    mx = float(last.split("max=")[1])
    assert abs(mn - lo) < 1e-4 * max(1, abs(lo)) and abs(mx - hi) < 1e-4 * max(1, abs(hi))


def test_a_wait_that_runs_out_becomes_an_error_and_the_network_recovers(th, oracle, tmp_path, monkeypatch):
    """The host side of the give-up path: THProcessFloat reports the status word of a kernel whose wait ran out as an
    error (count 0, a message), and the same network computes the right result on the next call."""
    g = fx.resnet50(width=0.125, size=64, classes=10)
    x = g.make_input(3)
    p = str(tmp_path / "r50.net")
    fx.write_pymodel(g, p)
    h = th.load_network(p)
    th.set_stats(h, g.mean, g.std)
    th.lib.THB200_SetPrecision(1)
    hc = th.lib.THCreateCudaNetwork(h)
    th.lib.THB200_SetPrecision(0)
    th.free_network(h)
    th.lib.thb_conv_reload_knobs.restype = None
    monkeypatch.setenv("THB200_TEST_WITHHOLD", "1")
    monkeypatch.setenv("THB200_WAIT_LIMIT_CYCLES", "20000000")
    th.lib.thb_conv_reload_knobs()
    try:
        res = C.POINTER(C.c_float)()
        ow, oh = C.c_int(), C.c_int()
        buf = np.array(x, copy=True)
        n = th.lib.THProcessFloat(hc, buf.ctypes.data_as(C.c_void_p), 3, 64, 64, 3, C.byref(res), C.byref(ow), C.byref(oh))
        assert n == 0
        assert b"timed out" in th.lib.THB200_LastErrorString()
    finally:
        monkeypatch.undo()
        th.lib.thb_conv_reload_knobs()
    out, _, _ = th.process_float(hc, x)
    assert rel_err(out, oracle.run(g, x).ravel()) < 1e-2
    th.free_network(hc)
