"""Host-side logic that needs no GPU: loaders, graph lowering, THMakeSpatial, error conventions,
struct ABI, and that the shared library exports every symbol its headers declare.
No compute entry point is called here."""
import ctypes as C
import os
import re
import shutil
import subprocess

import numpy as np
import pytest

from thnets_b200 import fixtures as fx
from thnets_b200.capi import DEFAULT_LIB, THNets, THNetworkStruct

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
os.environ.setdefault("THB200_NO_EXIT", "1")

pytestmark = pytest.mark.skipif(not os.path.exists(DEFAULT_LIB), reason="libthnets.so not built")


@pytest.fixture(scope="module")
def th():
    return THNets()


def describe(th, h):
    buf = C.create_string_buffer(1 << 18)
    n = th.lib.THB200_DescribeNetwork(h, buf, len(buf))
    assert n > 0, buf.value
    return [line for line in buf.value.decode().split("\n") if line]


def test_every_declared_symbol_is_exported():
    lib = C.CDLL(DEFAULT_LIB)
    names = set()
    for hdr in ("thnets.h", "thb200_kernels.h"):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b((?:TH|thb_|THB200_)\w+|loadtorch|freeobject|freenetwork|Module2Network|loadpytorch|"
                                r"freepynet|th_seconds)\s*\(", text))
    names -= {"THB_"}
    assert len(names) > 60
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing
    for var in ("th_debug", "th_profile", "th_minmax", "th_convtot", "th_convflops"):
        C.c_int.in_dll(lib, var)
    # ... and nothing but the documented ABI: the planner, the loaders' helpers and the launch internals stay local
    exported = set(subprocess.check_output(["nm", "-D", "--defined-only", DEFAULT_LIB], text=True).split()[2::3])
    internal = [n for n in exported if n.startswith(("thb_engine_", "thb_model_", "thb_t7_", "thb_lowp_", "thb_host_")) or n.startswith("_Z")]
    assert not internal, internal
    assert exported <= names | {"th_debug", "th_profile", "th_minmax", "th_convtot", "th_convflops", "loadonnx"}, exported - names


EXPECTED_ABI = {
    "sizeof(THFloatTensor)": 88, "sizeof(THFloatStorage)": 16, "sizeof(struct module)": 208, "sizeof(struct network)": 16,
    "sizeof(THNETWORK)": 72, "sizeof(struct thobject)": 24, "sizeof(struct pyelement)": 248,
    "offsetof(struct module, updateOutput)": 8, "offsetof(struct module, output)": 24,
    "offsetof(struct module, SpatialConvolution)": 128, "offsetof(struct module, SpatialConvolution.nOutputPlane)": 180,
    "offsetof(struct module, SpatialBatchNormalization.eps)": 160, "offsetof(THNETWORK, net)": 16,
    "offsetof(THNETWORK, mean)": 48, "offsetof(THNETWORK, std)": 60, "offsetof(struct network, modules)": 8,
    "offsetof(THFloatTensor, storage)": 72, "MT_CSubTable": 22, "MT_Transpose": 36, "ENGINE_LOWP": 4,
}


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_struct_layout_matches_the_reference_header(tmp_path):
    """sizes / offsets measured on the reference's own thnets.h (CPU build, x86-64) are pinned above; when the
    reference tree is present the two headers are also compared directly."""
    def probe(include):
        exe = str(tmp_path / ("abi_" + str(abs(hash(include)))))
        subprocess.check_call(["gcc", "-I", include, "-o", exe, os.path.join(ROOT, "tests", "abi_probe.c")])
        out = subprocess.check_output([exe], text=True)
        return dict((k, int(v)) for k, v in (line.rsplit("=", 1) for line in out.split("\n") if line))
    mine = probe(os.path.join(ROOT, "include"))
    for k, v in EXPECTED_ABI.items():
        assert mine[k] == v, (k, mine[k], v)
    from oracle.oracle import reference_root
    if reference_root():
        assert probe(reference_root()) == mine


def test_torch7_loader_and_lowering(th, tmp_path):
    g = fx.alexnet_owt(width=0.25, size=224, classes=50, fc=128)
    d = str(tmp_path / "alex")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    s = THNetworkStruct.from_address(h)
    assert s.net and not s.pynet
    assert np.allclose(list(s.mean), 0.45) and np.allclose(list(s.std), 0.225)   # stat.t7
    lines = describe(th, h)
    ops = [line.split()[1] for line in lines]
    assert ops == ["input", "conv", "act", "maxpool", "conv", "act", "maxpool", "conv", "act", "conv", "act", "conv", "act",
                   "maxpool", "view", "linear", "act", "linear", "act", "linear", "softmax"]
    assert "3->16 k11x11 s4,4 p2,2 bias=1" in lines[1]
    assert lines[-1].endswith("<- output")
    th.free_network(h)


def test_torch7_containers_and_caddtable_signs(th, tmp_path):
    """nn.Sequential { conv, ConcatTable { Sequential{conv,bn}, Identity }, CAddTable, ReLU, Concat{conv|conv}, JoinTable-free }"""
    rng = np.random.default_rng(0)
    conv = lambda ci, co, k, p: ("nn.SpatialConvolutionMM", dict(  # noqa: E731
        padW=p, padH=p, dW=1, dH=1, kW=k, kH=k, nInputPlane=ci, nOutputPlane=co,
        weight=rng.standard_normal((co, ci * k * k)).astype(np.float32), bias=rng.standard_normal(co).astype(np.float32)))
    bn = ("nn.SpatialBatchNormalization", dict(running_mean=np.zeros(8, np.float32), running_var=np.ones(8, np.float32),
                                               weight=np.ones(8, np.float32), bias=np.zeros(8, np.float32), eps=1e-5))
    spec = ("nn.Sequential", [
        conv(3, 8, 3, 1),
        ("nn.ConcatTable", [("nn.Sequential", [conv(8, 8, 3, 1), bn]), ("nn.Identity", {})]),
        ("nn.CAddTable", {}),
        ("nn.ReLU", dict(threshold=0.0, val=0.0, inplace=False)),
        ("nn.Concat", [conv(8, 8, 1, 0), conv(8, 16, 1, 0)], dict(dimension=2)),
    ])
    d = str(tmp_path / "branchy")
    fx.write_torch7(spec, d)
    h = th.load_network(d)
    lines = describe(th, h)
    ops = [line.split()[1] for line in lines]
    assert ops == ["input", "conv", "conv", "bn", "alias", "combine", "act", "conv", "conv", "concat"]
    comb = lines[5]
    assert "in=3,4" in comb and "+1 -1" in comb       # two-input CAddTable: first minus second
    assert "dim=1" in lines[9]
    th.free_network(h)


def test_pytorch_dump_loader_shares_referenced_nodes(th, tmp_path):
    g = fx.resnet18(width=0.25, size=64, classes=10)
    p = str(tmp_path / "r18.net")
    fx.write_pymodel(g, p)
    h = th.load_network(p)
    s = THNetworkStruct.from_address(h)
    assert s.pynet and not s.net                        # as in the reference, no struct network on this route
    lines = describe(th, h)
    combines = [line for line in lines if " combine " in line]
    assert len(combines) == 8 and all("+1 -1" in c for c in combines)
    # the shortcut of the first block is the max-pool output, consumed twice (second time by reference)
    assert "in=9,4" in combines[0]
    assert sum(" conv " in line for line in lines) == 20
    th.free_network(h)
    # a directory holding pymodel.net loads the same way
    d = tmp_path / "dir"
    d.mkdir()
    shutil.copy(p, d / "pymodel.net")
    h = th.load_network(str(d))
    assert len(describe(th, h)) == len(lines)
    th.free_network(h)


def test_onnx_reader_builds_the_same_graph(th, tmp_path):
    """The protobuf-free ONNX reader (onnx.cc:572-834 without protoc): batch normalisations are absorbed into their
    convolutions, a bias written as Add-of-a-constant and a padding written as a Pad node fold back, shared tensors are
    referenced, and what comes out is the node tree of the PyTorch-dump route."""
    g = fx.resnet18(width=0.25, size=64, classes=10)
    ref_lines = None
    for variant in ({}, {"bias_as_add": True, "pad_nodes": True}):
        p = str(tmp_path / "r18.onnx")
        fx.write_onnx(g, p, **variant)
        h = th.load_network(p)
        s = THNetworkStruct.from_address(h)
        assert s.pynet and not s.net
        lines = describe(th, h)
        assert sum(" conv " in line for line in lines) == 20
        assert not any(" bn " in line for line in lines)           # absorb_bn (onnx.cc:472-570)
        combines = [line for line in lines if " combine " in line]
        assert len(combines) == 8 and all("+1 -1" in c for c in combines)   # ONNX Add is CAddTable too (onnx.cc:46)
        assert sum("p3,3" in line for line in lines) == 1          # the stem's padding, Pad node or attribute
        if ref_lines is None:
            ref_lines = lines
        assert len(lines) == len(ref_lines)
        th.free_network(h)
    # VGG (biases everywhere) and the encoder-decoder (ConvTranspose, Concat)
    for build in (lambda: fx.vgg16(width=0.125, size=32, classes=10, fc=64), lambda: fx.segnet(width=0.25, size=32, classes=5)):
        g2 = build()
        p = str(tmp_path / "m.onnx")
        fx.write_onnx(g2, p, bias_as_add=True)
        h = th.load_network(p)
        lines = describe(th, h)
        assert sum((" conv " in line) or (" deconv " in line) or (" linear " in line) for line in lines) == \
            sum(n.op in ("conv", "deconv", "linear") for n in g2.nodes)
        th.free_network(h)


def test_onnx_reader_rejects_what_it_cannot_read(th, tmp_path):
    bad = tmp_path / "bad.onnx"
    bad.write_bytes(b"\x3a\x05hello")                   # field 7 (graph) holding garbage
    assert not th.lib.THLoadNetwork(str(bad).encode())
    # an operator outside the supported set is an error, not a silent Dropout
    g = fx.Graph(0)
    g.input_shape = (3, 8, 8)
    x = g.conv(0, 3, 4, 3, 1, 1)
    g.softmax(x)
    p = str(tmp_path / "ok.onnx")
    fx.write_onnx(g, p)
    raw = open(p, "rb").read()
    assert raw.count(b"Softmax") == 1
    open(p, "wb").write(raw.replace(b"Softmax", b"Softmin"))
    assert not th.lib.THLoadNetwork(p.encode())
    assert b"Unsupported node type Softmin" in th.lib.THB200_LastErrorString()


def test_make_spatial_rewrites_the_classifier(th, tmp_path):
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    d = str(tmp_path / "vgg")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    before = describe(th, h)
    assert any(" view " in x for x in before) and sum(" linear " in x for x in before) == 3
    th.make_spatial(h, 32)
    after = describe(th, h)
    assert not any(" view " in x or " linear " in x for x in after)
    convs = [x for x in after if " conv " in x]
    assert len(convs) == 16
    assert "64->64 k1x1" in convs[-3] and "64->64 k1x1" in convs[-2] and "64->10 k1x1" in convs[-1]   # 32/2^5 = 1
    th.free_network(h)
    # a 64x64 classifier: the first Linear becomes a 2x2 convolution
    g = fx.vgg16(width=0.125, size=64, classes=10, fc=64)
    d = str(tmp_path / "vgg64")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    th.make_spatial(h, 64)
    assert "k2x2" in [x for x in describe(th, h) if " conv " in x][-3]
    th.free_network(h)


def test_error_conventions(th, tmp_path):
    lib = th.lib
    assert not lib.THLoadNetwork(str(tmp_path / "missing").encode())
    assert lib.THLastError() == -1                       # ERR_OPENFILE
    d = tmp_path / "corrupt"
    d.mkdir()
    (d / "model.net").write_bytes(b"\x09\x00\x00\x00garbage")
    assert not lib.THLoadNetwork(str(d).encode())
    assert lib.THLastError() == -4                       # ERR_CORRUPTED
    (d / "model.net").write_bytes(b"\x01\x00\x00\x00" + b"\x00" * 8)   # a bare number, not a module
    assert not lib.THLoadNetwork(str(d).encode())
    assert lib.THLastError() == -5                       # ERR_WRONGOBJECT
    (d / "model.net").write_bytes(b"\x04\x00")
    assert not lib.THLoadNetwork(str(d).encode())
    assert lib.THLastError() == -2                       # ERR_READFILE
    assert lib.THOpenCLHalfFloat(1) == -3 and not lib.THCreateOpenCLNetwork(None)
    assert lib.THCudaHalfFloat(1) == 0 and lib.THCudaHalfFloat(0) == 0


def test_unsupported_module_is_reported(th, tmp_path):
    spec = ("nn.Sequential", [("nn.SpatialConvolutionMM", dict(
        padW=0, padH=0, dW=1, dH=1, kW=1, kH=1, nInputPlane=3, nOutputPlane=4,
        weight=np.zeros((4, 3), np.float32), bias=np.zeros(4, np.float32))), ("nn.SpatialSubtractiveNormalization", {})])
    d = str(tmp_path / "ls")
    fx.write_torch7(spec, d)
    # unknown module types are fatal in the reference's loader (thload.c:777-778): run in a child process
    code = ("import os, sys; sys.path.insert(0, %r); from thnets_b200.capi import THNets; THNets().lib.THLoadNetwork(%r)"
            % (ROOT, d.encode()))
    r = subprocess.run([os.sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode != 0 and "Unknown module type nn.SpatialSubtractiveNormalization" in r.stderr


def test_batch_slicing(th):
    off, cnt = C.c_int(), C.c_int()
    for n in (1, 7, 256, 250):
        for g in (1, 2, 4, 8):
            covered = []
            for r in range(g):
                th.lib.THB200_SliceBatch(n, g, r, C.byref(off), C.byref(cnt))
                covered += list(range(off.value, off.value + cnt.value))
                assert cnt.value in (n // g, n // g + 1)
            assert covered == list(range(n))


def test_onnx_reader_leaky_and_prelu(th, tmp_path):
    """ONNX LeakyRelu becomes a Threshold record with the node's alpha (onnx.cc:36, Threshold.c:30-35), PRelu a PReLU with
    one slope per plane taken from the second input (onnx.cc:35, PReLU.c:21-29); both lower to activations."""
    g = fx.prelu_net(onnx_form=True)
    p = str(tmp_path / "prelu.onnx")
    fx.write_onnx(g, p)
    h = th.load_network(p)
    assert h, th.lib.THB200_LastErrorString()
    lines = describe(th, h)
    kinds = [ln.split("kind=")[1].split()[0] for ln in lines if " act " in ln]
    assert kinds == ["3", "2", "3"], lines            # PReLU, leaky, PReLU
    th.free_network(h)


def test_onnx_reader_whole_map_average(th, tmp_path):
    """GlobalAveragePool and ReduceMean over axes (2, 3) both become an average pooling with kernel 0 -- the whole map
    (onnx.cc:49-50, SpatialAveragePooling.c:47-67, :116-119) -- which the planner sizes to its input, so the launch is the
    one an AveragePool with the map's extent gets; ReduceMean over other axes is refused as by the reference."""
    g = fx.resnet18(width=0.125, size=32, classes=5)
    lines = {}
    for how in (None, "GlobalAveragePool", "ReduceMean"):
        p = str(tmp_path / ("r18_%s.onnx" % how))
        fx.write_onnx(g, p, global_pool=how)
        h = th.load_network(p)
        assert h, th.lib.THB200_LastErrorString()
        lines[how] = describe(th, h)
        th.free_network(h)
    pools = {how: [ln for ln in ls if " avgpool " in ln] for how, ls in lines.items()}
    assert len(pools[None]) == 1 and " k1x1 " in pools[None][0]            # a 32 x 32 input leaves a 1 x 1 map
    assert pools["GlobalAveragePool"] == pools["ReduceMean"] and " k0x0 s1,1 p0,0" in pools["ReduceMean"][0]
    strip = lambda ls: [ln for ln in ls if " avgpool " not in ln]
    assert strip(lines[None]) == strip(lines["ReduceMean"]) == strip(lines["GlobalAveragePool"])
    p = str(tmp_path / "r18_bad.onnx")
    fx.write_onnx(g, p, global_pool=("ReduceMean", [1]))
    assert not th.lib.THLoadNetwork(p.encode())
    assert b"ReduceMean along channel" in th.lib.THB200_LastErrorString()


def test_reshape_lowering(th, tmp_path):
    """nn.Reshape to three dimensions lowers to an operator of its own with the target map; to one dimension it is a View"""
    g = fx.reshape_net()
    d = str(tmp_path / "reshape")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    lines = describe(th, h)
    assert any(" reshape in=5 3x5x4" in ln for ln in lines), lines
    assert lines[-1].startswith("7 conv in=6 3->6") and lines[-1].endswith("<- output")
    th.free_network(h)


def test_sub_batch_slicing(th):
    """Pipelined sub-batches cover a GPU's slice once, in order, none empty; up to four of them grow from first to last
    (the first copy is short, each later copy ends under the kernels ahead of it)."""
    off, cnt = C.c_int(), C.c_int()
    for n in (1, 5, 16, 31, 32, 64, 250, 256):
        for s in (1, 2, 3, 4):
            if s > n:
                continue
            covered, sizes = [], []
            for c in range(s):
                th.lib.THB200_SliceSubBatches(n, s, c, C.byref(off), C.byref(cnt))
                assert cnt.value >= 1
                covered += list(range(off.value, off.value + cnt.value))
                sizes.append(cnt.value)
            assert covered == list(range(n)), (n, s, sizes)
            if n >= 8 * s:
                assert sizes == sorted(sizes), (n, s, sizes)
    th.lib.THB200_SliceSubBatches(256, 2, 0, C.byref(off), C.byref(cnt))
    assert (off.value, cnt.value) == (0, 96)
    th.lib.THB200_SliceSubBatches(256, 4, 3, C.byref(off), C.byref(cnt))
    assert (off.value, cnt.value) == (176, 80)


def test_fixture_writers_round_trip_through_the_reference_formats(tmp_path):
    """the .t7 writer emits objects with strictly increasing indices and float tensors with 1-based offsets"""
    g = fx.vgg16(width=0.125, size=32, classes=10, fc=64)
    d = str(tmp_path / "vgg")
    fx.write_torch7(g, d)
    raw = open(os.path.join(d, "model.net"), "rb").read()
    assert raw[:4] == (4).to_bytes(4, "little") and b"nn.Sequential" in raw[:64] and b"torch.FloatStorage" in raw
    p = str(tmp_path / "m.net")
    fx.write_pymodel(g, p)
    assert open(p, "rb").read(24) == b"PyTorch Graph Dump 1.00\0"


def test_static_scratch_entry_validates_before_any_launch():
    """thb_conv_u8_fwd_static must answer a descriptor its channel-sum pass cannot digest with an error code, before any
    CUDA call: every case below returns without touching a device (this test runs where there is none)."""
    from thnets_b200 import kernels_abi as K
    lib = K.load()
    lib.thb_conv_u8_fwd_static.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    fake = C.c_void_p(1 << 20)          # never dereferenced: each call is refused first

    def desc(**kw):
        d = K.ConvDesc()
        d.dtype = K.THB_U8
        d.N, d.H, d.W, d.Cin, d.Cout, d.in_ld = 2, 8, 8, 24, 16, 32
        d.w = d.kinfo = d.tmap = d.wsat = d.status = 1 << 20
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    ARG, UNSUP = -4, -1
    cases = [(desc(dtype=K.THB_F16), fake, ARG), (desc(N=-2, H=-8), fake, ARG), (desc(N=0), fake, ARG),
             (desc(Cin=0), fake, ARG), (desc(in_ld=24), fake, ARG), (desc(in_ld=16), fake, ARG),
             (desc(), C.c_void_p((1 << 20) + 4), ARG), (desc(wsat=None), fake, ARG), (desc(status=None), fake, ARG),
             (desc(tmap=None), fake, ARG), (desc(in_row_pitch=12, in_pad_left=1), fake, UNSUP),
             (desc(N=64, H=512, W=512), fake, ARG)]
    for d, x, want in cases:
        assert lib.thb_conv_u8_fwd_static(C.byref(d), x, fake, None) == want
    assert lib.thb_conv_u8_fwd_static(None, fake, fake, None) == ARG


def test_split_plan_is_for_launches_that_leave_the_machine_idle():
    """thb_conv_splitk_plan (host arithmetic only; without a device it assumes 148 SMs): a handful of tiles with a long
    reduction is split so that the units fill the machine, with at least four K blocks per part and a bounded scratch;
    launches of a wave or more, short reductions, narrow tiles, the uint8 type and two-operand convolutions are not."""
    from thnets_b200 import kernels_abi as K
    lib = K.load()
    lib.thb_conv_splitk_plan.argtypes = [C.c_void_p, C.POINTER(C.c_size_t)]

    def plan(n, cin, hw, cout, k, dtype=K.THB_F16, **kw):
        d = K.ConvDesc()
        d.dtype = dtype
        d.N, d.H, d.W, d.Cin, d.Cout = n, hw, hw, cin, cout
        d.kH = d.kW = k
        d.dH = d.dW = 1
        d.padH = d.padW = k // 2
        d.oH = d.oW = hw
        d.in_ld = cin
        assert lib.thb_conv_geometry(C.byref(d)) == 0
        for key, v in kw.items():
            setattr(d, key, v)
        nbytes = C.c_size_t(0)
        return lib.thb_conv_splitk_plan(C.byref(d), C.byref(nbytes)), nbytes.value, d

    s, nbytes, d = plan(1, 512, 7, 512, 3)                 # 1 pixel tile x 4 column tiles, 72 K blocks
    assert 2 <= s <= 8 and d.Ktot_pad // 64 // s >= 4
    assert nbytes == s * 49 * d.Cout_pad * 4
    assert plan(32, 25088, 1, 4096, 1, BN=128)[0] >= 2    # a Linear on 32 rows with wide tiles
    assert plan(256, 256, 14, 256, 3)[0] == 1             # 392 tiles: more than a wave
    assert plan(64, 256, 14, 256, 3)[0] == 1              # 196 tiles: the partial sums would cost more than they save
    assert plan(1, 64, 7, 512, 1)[0] == 1                 # one K block
    assert plan(1, 512, 7, 32, 3)[0] == 1                 # 32-column tiles have no split form
    assert plan(1, 512, 7, 512, 3, dtype=K.THB_U8)[0] == 1
    assert plan(1, 512, 7, 512, 3, x2=1 << 20)[0] == 1


def test_tile_width_rules():
    """thb_conv_geometry picks the output-channel width of a tile on the host: the narrowest of 32 / 64 / 128 that holds
    the layer's channels; 256 once the reduction is at least four K blocks long, every SM gets a tile and the padding is
    not increased by it; 64 where wide tiles would leave most SMs without work; 32 for a Linear proper of few rows.  The
    padded extents follow from it; fp32 always works on 64 columns; a width set by the caller is kept."""
    from thnets_b200 import kernels_abi as K
    lib = K.load()

    def geom(n, cin, hw, cout, k, dtype=K.THB_F16, bn=0):
        d = K.ConvDesc()
        d.dtype = dtype
        d.N, d.H, d.W, d.Cin, d.Cout = n, hw, hw, cin, cout
        d.kH = d.kW = k
        d.dH = d.dW = 1
        d.padH = d.padW = k // 2
        d.oH = d.oW = hw
        d.in_ld = cin
        d.BN = bn
        assert lib.thb_conv_geometry(C.byref(d)) == 0
        return d

    assert geom(4, 64, 56, 24, 3).BN == 32
    assert geom(4, 64, 56, 64, 3).BN == 64
    assert geom(4, 64, 56, 128, 1).BN == 128
    assert geom(256, 256, 14, 1024, 1).BN == 256            # 392 pixel tiles, K = 4 blocks
    assert geom(256, 64, 56, 256, 1).BN == 128              # one K block: the epilogue outweighs the reduction
    assert geom(256, 512, 7, 512, 3).BN == 256              # 98 x 2 wide tiles: every SM still gets one
    assert geom(64, 512, 7, 512, 3).BN == 128               # 25 x 2 wide tiles would leave SMs idle
    assert geom(256, 256, 14, 384, 3).BN == 128             # 384 channels pad to 512 on wide tiles
    assert geom(1, 256, 13, 256, 3).BN == 64                # 2 pixel tiles x 2: narrower tiles for more SMs
    d = geom(256, 2048, 1, 1000, 1)
    assert d.BN == 32 and d.Cout_pad == 1024                # a Linear on 256 rows
    assert geom(256, 256, 14, 1024, 1, bn=128).BN == 128    # the caller's choice stands
    d = geom(4, 3, 224, 64, 3, dtype=K.THB_F32)
    assert d.BN == 64 and d.Cin_pad == 4 and d.Ktot_pad == 48
    d = geom(4, 100, 14, 130, 3, dtype=K.THB_U8)
    assert d.Cin_pad == 112 and d.Ktot_pad == 1024 and d.Cout_pad % d.BN == 0 and d.Cout_pad >= 130
    bad = K.ConvDesc()
    bad.dtype = K.THB_F16
    assert lib.thb_conv_geometry(C.byref(bad)) != 0          # no kernel extent


def test_patch_kernel_eligibility_rules():
    """thb_conv_patch_supported / thb_conv_maxpool_supported decide on the host which convolutions the patch kernel takes:
    16-bit types, stride 1, at most 64 output channels on 64-column tiles, 16 or 64 stored input channels, kernels up to
    8 x 8 whose weights fit in shared memory; a fused residual needs +-1 for the convolution's own term and has no pooled
    form; pooling windows of 2 or 3 with stride 2."""
    from thnets_b200 import kernels_abi as K
    lib = K.load()
    lib.thb_conv_patch_supported.argtypes = [C.c_void_p]
    lib.thb_conv_maxpool_supported.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]

    def desc(cin=64, cout=64, k=3, stride=1, hw=56, dtype=K.THB_F16, **kw):
        d = K.ConvDesc()
        d.dtype = dtype
        d.N, d.H, d.W, d.Cin, d.Cout = 4, hw, hw, cin, cout
        d.kH = d.kW = k
        d.dH = d.dW = stride
        d.padH = d.padW = k // 2
        d.oH = d.oW = (hw + 2 * (k // 2) - k) // stride + 1
        d.in_ld = max(cin, 8)
        d.BN = 64 if cout <= 64 else 0
        assert lib.thb_conv_geometry(C.byref(d)) == 0
        for key, v in kw.items():
            setattr(d, key, v)
        return d

    ok = lambda d: lib.thb_conv_patch_supported(C.byref(d))
    assert ok(desc()) == 1
    assert ok(desc(cin=16, cout=24, k=5)) == 1
    assert ok(desc(dtype=K.THB_BF16)) == 1
    assert ok(desc(res=1 << 20, res_ld=64, self_coef=1.0, res_coef=-1.0)) == 1
    assert ok(desc(res=1 << 20, res_ld=64, self_coef=0.5, res_coef=1.0)) == 0
    assert ok(desc(res=(1 << 20) + 8, res_ld=64, self_coef=1.0, res_coef=1.0)) == 0
    assert ok(desc(cout=128)) == 0
    assert ok(desc(stride=2)) == 0
    assert ok(desc(cin=32)) == 0
    assert ok(desc(dtype=K.THB_U8, cin=64)) == 0
    assert ok(desc(cin=64, k=7)) == 0                      # 49 x 64 x 128 bytes of weights do not fit
    d = desc()
    assert lib.thb_conv_maxpool_supported(C.byref(d), 3, 2, 1) == 1
    assert lib.thb_conv_maxpool_supported(C.byref(d), 2, 2, 0) == 1
    assert lib.thb_conv_maxpool_supported(C.byref(d), 3, 1, 1) == 0
    assert lib.thb_conv_maxpool_supported(C.byref(d), 4, 2, 0) == 0
    assert lib.thb_conv_maxpool_supported(C.byref(desc(res=1 << 20, res_ld=64, self_coef=1.0, res_coef=1.0)), 3, 2, 1) == 0


def test_loaders_accept_the_remaining_operators(th, tmp_path):
    """SpatialZeroPadding / SpatialMaxUnpooling (with its reference to the pooling module) / LogSoftMax / Normalize from
    Torch7 files, Cmax / Slice from a graph dump, Upsample / Max / Slice / LogSoftmax from ONNX: loaded and lowered."""
    g = fx.unpool_net()
    d = str(tmp_path / "unpool")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    lines = describe(th, h)
    assert any("unpool" in l.lower() for l in lines) and any("pad" in l.lower() for l in lines), lines
    th.free_network(h)
    g = fx.normalize_net()
    d = str(tmp_path / "norm")
    fx.write_torch7(g, d)
    h = th.load_network(d)
    assert len(describe(th, h)) >= 5
    th.free_network(h)
    g = fx.cmax_slice_net()
    p = str(tmp_path / "cmax.net")
    fx.write_pymodel(g, p)
    h = th.load_network(p)
    lines = describe(th, h)
    assert any("max" in l.lower() for l in lines) and any("slice" in l.lower() for l in lines), lines
    th.free_network(h)
    g = fx.onnx_ops_net()
    p = str(tmp_path / "ops.onnx")
    fx.write_onnx(g, p)
    h = th.load_network(p)
    lines = describe(th, h)
    assert any("upsample" in l.lower() for l in lines), lines
    th.free_network(h)
