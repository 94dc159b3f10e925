"""Seeded synthetic networks and the two on-disk formats thnets loads them from.

A `Graph` is a small DAG description (conv, deconv, linear, bn, pools, threshold,
view, add, concat, softmax ...) with NumPy weights.  It can be written as

* a "PyTorch Graph Dump 1.00" file (`write_pymodel`), the format parsed by the
  reference's pytorch.c:151-299: the root element is the network OUTPUT, inputs are
  nested depth-first, a tensor with a second consumer is written as a type-7 id
  reference (thexport.py:130-137);
* a Torch7 directory `model.net` + `stat.t7` (`write_torch7`), the binary
  serialisation parsed by thload.c:119-406 (only purely sequential graphs).

The builders at the bottom reproduce the five benchmark architectures with
He-normal weights drawn in layer order (weight, then bias) from
`numpy.random.default_rng(seed)`; `width`/`size` arguments shrink them for tests.
No dataset and no trained weights are involved anywhere.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass, field

import numpy as np


@dataclass
class Node:
    op: str
    inputs: list
    attrs: dict = field(default_factory=dict)
    tensors: list = field(default_factory=list)  # [(name, ndarray)], '' = positional


class Graph:
    """DAG under construction; node 0 is always the network input."""

    def __init__(self, seed=0, mean=(0.0, 0.0, 0.0), std=(1.0, 1.0, 1.0)):
        self.rng = np.random.default_rng(seed)
        self.nodes = [Node("input", [])]
        self.output = 0
        self.mean = np.asarray(mean, np.float32)
        self.std = np.asarray(std, np.float32)
        self.input_shape = None  # (C, H, W)
        self.input_dist = "normal"

    # ---- helpers -------------------------------------------------------------
    def _add(self, op, inputs, attrs=None, tensors=None):
        self.nodes.append(Node(op, list(inputs), attrs or {}, tensors or []))
        self.output = len(self.nodes) - 1
        return self.output

    def he(self, shape, fan_in):
        return (self.rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    # ---- layers --------------------------------------------------------------
    def conv(self, x, cin, cout, k, stride=1, pad=0, bias="zero", pads4=None, dilation=None, auto_pad=None, reflect=False):
        """pads4 (top, left, bottom, right), dilation, auto_pad ("SAME_UPPER" / "SAME_LOWER") and reflect (the padding
        comes from a reflect-mode Pad node) exist in ONNX files only: the reference parses and ignores them."""
        kh, kw = (k, k) if isinstance(k, int) else k
        w = self.he((cout, cin, kh, kw), cin * kh * kw)
        t = [("", w)]
        b = self._bias(bias, cout)
        if b is not None:
            t.append(("", b))
        attrs = dict(stride=(stride, stride), padding=(pad, pad))
        if pads4 is not None:
            attrs["pads4"] = tuple(int(v) for v in pads4)
            attrs["padding"] = (int(pads4[0]), int(pads4[1]))
        if dilation is not None:
            attrs["dilation"] = (int(dilation), int(dilation))
        if auto_pad is not None:
            attrs["auto_pad"] = auto_pad
        if reflect:
            attrs["reflect"] = 1
        return self._add("conv", [x], attrs, t)

    def deconv(self, x, cin, cout, k, stride=1, pad=0, adj=0, bias=None):
        w = self.he((cin, cout, k, k), cin * k * k)
        t = [("", w)]
        b = self._bias(bias, cout)
        if b is not None:
            t.append(("", b))
        return self._add("deconv", [x], dict(stride=(stride, stride), padding=(pad, pad),
                                            output_padding=(adj, adj)), t)

    def _bias(self, bias, n):
        if bias is None:
            return None
        if isinstance(bias, str) and bias == "zero":
            return np.zeros(n, np.float32)
        if isinstance(bias, (int, float)):
            return (self.rng.standard_normal(n) * bias).astype(np.float32)
        return np.asarray(bias, np.float32)

    def linear(self, x, cin, cout, bias="zero"):
        w = self.he((cout, cin), cin)
        return self._add("linear", [x], {}, [("", w), ("", self._bias(bias, cout))])

    def bn(self, x, c, eps=1e-5):
        rng = self.rng
        mean = (rng.standard_normal(c) * 0.1).astype(np.float32)
        var = rng.uniform(0.5, 1.5, c).astype(np.float32)
        gamma = rng.uniform(0.8, 1.2, c).astype(np.float32)
        beta = (rng.standard_normal(c) * 0.1).astype(np.float32)
        return self._add("bn", [x], dict(eps=float(eps)),
                         [("", gamma), ("", beta), ("running_mean", mean), ("running_var", var)])

    def relu(self, x, threshold=0.0, value=0.0):
        return self._add("threshold", [x], dict(threshold=float(threshold), value=float(value), inplace=0))

    def leaky(self, x, alpha):
        """x >= 0 ? x : alpha * x -- a Threshold record with `alpha` set (Threshold.c:55-57), which only an ONNX LeakyRelu makes"""
        return self._add("threshold", [x], dict(threshold=0.0, value=0.0, inplace=0, alpha=float(alpha)))

    def prelu(self, x, channels, shared=False):
        """nn.PReLU: one slope per channel, or one for all (nOutputPlane = 0)"""
        w = (0.05 + 0.4 * self.rng.random(1 if shared else channels)).astype(np.float32)
        return self._add("prelu", [x], dict(planes=0 if shared else int(channels)), [("weight", w)])

    def maxpool(self, x, k, stride, pad=0, ceil_mode=0):
        return self._add("maxpool", [x], dict(kernel_size=(k, k), stride=(stride, stride),
                                             padding=(pad, pad), ceil_mode=int(ceil_mode)))

    def avgpool(self, x, k, stride=None, pad=0, ceil_mode=0):
        stride = stride or k
        return self._add("avgpool", [x], dict(kernel_size=(k, k), stride=(stride, stride),
                                             padding=(pad, pad), ceil_mode=int(ceil_mode)))

    def view(self, x, n):
        return self._add("view", [x], dict(sizes=(-1, int(n))))

    def reshape(self, x, c, h, w):
        """nn.Reshape(c, h, w): the vector of every image becomes a [c, h, w] map"""
        return self._add("reshape", [x], dict(sizes=(int(c), int(h), int(w))))

    def dropout(self, x):
        return self._add("dropout", [x])

    def softmax(self, x):
        return self._add("softmax", [x])

    def sigmoid(self, x):
        return self._add("sigmoid", [x])

    def tanh(self, x):
        return self._add("tanh", [x])

    def upsample(self, x):
        return self._add("upsample", [x])

    def zeropad(self, x, pad_l, pad_r, pad_t, pad_b):
        return self._add("zeropad", [x], dict(pad_l=int(pad_l), pad_r=int(pad_r), pad_t=int(pad_t), pad_b=int(pad_b)))

    def slice(self, x, axis, start, stop):
        return self._add("slice", [x], dict(axis=int(axis), start=int(start), stop=int(stop)))

    def cmax(self, xs):
        return self._add("cmax", list(xs))

    def logsoftmax(self, x):
        return self._add("logsoftmax", [x])

    def l2normalize(self, x):
        return self._add("l2normalize", [x])

    def unpool(self, x, pool_node):
        """SpatialMaxUnpooling of x against the max pooling that is node `pool_node` of this graph."""
        return self._add("unpool", [x], dict(pool=int(pool_node)))

    def add(self, a, b):
        """Reference semantics for two inputs: a - b (CAddTable.c:59-69)."""
        return self._add("add", [a, b])

    def concat(self, xs, dim=1):
        return self._add("concat", list(xs), dict(dim=int(dim)))

    # ---- misc ----------------------------------------------------------------
    def make_input(self, batch, seed=1234):
        rng = np.random.default_rng(seed)
        c, h, w = self.input_shape
        if self.input_dist == "uniform":
            return rng.random((batch, c, h, w), dtype=np.float32)
        return rng.standard_normal((batch, c, h, w)).astype(np.float32)

    def is_sequential(self):
        return all(n.inputs == [i - 1] for i, n in enumerate(self.nodes) if i > 0) and \
            self.output == len(self.nodes) - 1


# ============================================================================
# "PyTorch Graph Dump 1.00" writer
# ============================================================================
_PYNAME = {
    "conv": "ConvNd", "deconv": "ConvTransposedNd", "linear": "Linear", "bn": "BatchNorm",
    "maxpool": "MaxPool2d", "avgpool": "AvgPool2d", "threshold": "Threshold", "dropout": "Dropout",
    "softmax": "Softmax", "view": "View", "add": "Add", "concat": "Concat", "slice": "Slice", "cmax": "Cmax",
}


def _w_str(f, s):
    f.write(s.encode("ascii") + b"\0")


def _w_tensor(f, name, arr):
    arr = np.ascontiguousarray(arr, np.float32)
    f.write(b"\x03")
    _w_str(f, name)
    f.write(struct.pack("<i", arr.ndim))
    f.write(struct.pack("<%di" % arr.ndim, *arr.shape))
    f.write(struct.pack("<q", arr.size))
    f.write(arr.tobytes())


def write_pymodel(graph: Graph, path: str):
    """Serialise `graph` depth-first from its output node."""
    emitted = set()
    with open(path, "wb") as f:
        f.write(b"PyTorch Graph Dump 1.00\0")

        def emit(i):
            node = graph.nodes[i]
            if node.op == "input":
                f.write(b"\x01")
                return
            if i in emitted:
                f.write(b"\x07" + struct.pack("<i", i))
                return
            emitted.add(i)
            if node.op not in _PYNAME or node.attrs.get("alpha"):
                raise ValueError("no graph-dump form for " + node.op)
            f.write(b"\x02" + struct.pack("<i", i))
            _w_str(f, "torch.nn.fn." + _PYNAME[node.op])
            attrs = node.attrs
            if node.op == "slice":
                # Slice.c:3-14: the dump carries index = {from, to} and no axis (dimension 0 of the tensor)
                if attrs["axis"] != 0:
                    raise ValueError("the graph-dump Slice cuts dimension 0 only")
                attrs = {"index": (attrs["start"], attrs["stop"])}
            for k, v in attrs.items():
                if k in ("pads4", "dilation", "auto_pad", "reflect"):
                    continue
                if isinstance(v, tuple):
                    f.write(b"\x06")
                    _w_str(f, k)
                    f.write(struct.pack("<i", len(v)) + struct.pack("<%di" % len(v), *v))
                elif isinstance(v, float):
                    f.write(b"\x05")
                    _w_str(f, k)
                    f.write(struct.pack("<f", v))
                else:
                    f.write(b"\x04")
                    _w_str(f, k)
                    f.write(struct.pack("<i", int(v)))
            for j in node.inputs:
                emit(j)
            for name, arr in node.tensors:
                _w_tensor(f, name, arr)
            f.write(b"\x00")

        emit(graph.output)


# ============================================================================
# Torch7 writer (sequential graphs; containers for the branchy test nets)
# ============================================================================
class _T7:
    def __init__(self, f):
        self.f = f
        self.idx = 1

    def i32(self, v):
        self.f.write(struct.pack("<i", v))

    def i64(self, v):
        self.f.write(struct.pack("<q", v))

    def string_raw(self, s):
        b = s.encode("ascii")
        self.i32(len(b))
        self.f.write(b)

    def number(self, v):
        self.i32(1)
        self.f.write(struct.pack("<d", float(v)))

    def string(self, s):
        self.i32(2)
        self.string_raw(s)

    def boolean(self, v):
        self.i32(5)
        self.i32(1 if v else 0)

    def nil(self):
        self.i32(0)

    def tensor(self, arr):
        if arr is None:
            # a tensor object without storage (what Torch writes for an absent bias)
            self.i32(4)
            self.i32(self.idx)
            self.idx += 1
            self.string_raw("V 1")
            self.string_raw("torch.FloatTensor")
            self.i32(0)
            self.i64(1)
            self.nil()
            return
        arr = np.ascontiguousarray(arr, np.float32)
        self.i32(4)
        self.i32(self.idx)
        self.idx += 1
        self.string_raw("V 1")
        self.string_raw("torch.FloatTensor")
        self.i32(arr.ndim)
        for s in arr.shape:
            self.i64(s)
        stride = 1
        strides = []
        for s in reversed(arr.shape):
            strides.append(stride)
            stride *= s
        for s in reversed(strides):
            self.i64(s)
        self.i64(1)  # storageOffset, 1-based
        self.i32(4)
        self.i32(self.idx)
        self.idx += 1
        self.string_raw("V 1")
        self.string_raw("torch.FloatStorage")
        self.i64(arr.size)
        self.f.write(arr.tobytes())

    def long_storage(self, values):
        """a torch.LongStorage object (8-byte elements): what nn.Reshape keeps its sizes in"""
        self.i32(4)
        self.i32(self.idx)
        self.idx += 1
        self.string_raw("V 1")
        self.string_raw("torch.LongStorage")
        self.i64(len(values))
        for v in values:
            self.i64(int(v))

    def table(self, items):
        """items: list of (key, writer-callable); string or number keys."""
        self.i32(3)
        self.i32(self.idx)
        self.idx += 1
        self.i32(len(items))
        for k, w in items:
            if isinstance(k, str):
                self.string(k)
            else:
                self.number(k)
            w()

    def module(self, name, items):
        self.i32(4)
        idx = self.idx
        self.i32(self.idx)
        self.idx += 1
        self.string_raw("V 1")
        self.string_raw(name)
        self.table(items)
        return idx

    def reference(self, idx):
        """an object written earlier, by its index (how Torch serialises a second mention of the same object)"""
        self.i32(4)
        self.i32(idx)


def _t7_module(t: _T7, spec):
    """spec = (torch class name, {field: value}) or (container name, [children], {fields})."""
    name = spec[0]
    if name in ("nn.Sequential", "nn.Concat", "nn.ConcatTable"):
        children = spec[1]
        extra = spec[2] if len(spec) > 2 else {}
        items = [("modules", lambda: t.table([(i + 1, (lambda c=c: _t7_module(t, c)))
                                              for i, c in enumerate(children)]))]
        for k, v in extra.items():
            items.append((k, (lambda v=v: t.number(v))))
        t.module(name, items)
        return
    items = []
    if not hasattr(t, "written"):
        t.written = {}
    for k, v in spec[1].items():
        if isinstance(v, np.ndarray) or v is None:
            items.append((k, (lambda v=v: t.tensor(v))))
        elif isinstance(v, bool):
            items.append((k, (lambda v=v: t.boolean(v))))
        elif isinstance(v, tuple) and v and v[0] == "longs":
            items.append((k, (lambda v=v: t.long_storage(v[1]))))
        elif isinstance(v, tuple) and v and v[0] == "ref":
            items.append((k, (lambda v=v: t.reference(t.written[id(v[1])]))))   # a module spec written earlier
        else:
            items.append((k, (lambda v=v: t.number(v))))
    t.written[id(spec)] = t.module(name, items)


def graph_to_t7_spec(graph: Graph):
    """Nested Torch7 module spec of a purely sequential graph."""
    if not graph.is_sequential():
        raise ValueError("only sequential graphs map onto a flat nn.Sequential")
    mods = []
    spec_of = {}
    for ni, node in enumerate(graph.nodes[1:], start=1):
        a = node.attrs
        ts = [arr for _, arr in node.tensors]
        if node.op == "conv":
            w = ts[0]
            mods.append(("nn.SpatialConvolutionMM", dict(
                padW=a["padding"][1], padH=a["padding"][0], dW=a["stride"][1], dH=a["stride"][0],
                kW=w.shape[3], kH=w.shape[2], nInputPlane=w.shape[1], nOutputPlane=w.shape[0],
                weight=w.reshape(w.shape[0], -1), bias=ts[1] if len(ts) > 1 else None)))
        elif node.op == "linear":
            mods.append(("nn.Linear", dict(weight=ts[0], bias=ts[1])))
        elif node.op == "threshold":
            if a.get("alpha"):
                raise ValueError("no Torch7 mapping for a leaky threshold")
            mods.append(("nn.Threshold", dict(threshold=a["threshold"], val=a["value"], inplace=False)))
        elif node.op == "prelu":
            mods.append(("nn.PReLU", dict(nOutputPlane=a["planes"], weight=ts[0])))
        elif node.op == "maxpool":
            mods.append(("nn.SpatialMaxPooling", dict(
                padW=a["padding"][1], padH=a["padding"][0], dW=a["stride"][1], dH=a["stride"][0],
                kW=a["kernel_size"][1], kH=a["kernel_size"][0], ceil_mode=a["ceil_mode"])))
        elif node.op == "avgpool":
            mods.append(("nn.SpatialAveragePooling", dict(
                padW=a["padding"][1], padH=a["padding"][0], dW=a["stride"][1], dH=a["stride"][0],
                kW=a["kernel_size"][1], kH=a["kernel_size"][0], ceil_mode=a["ceil_mode"],
                count_include_pad=0)))
        elif node.op == "view":
            mods.append(("nn.View", dict(numElements=a["sizes"][1])))
        elif node.op == "reshape":
            # as nn.Reshape writes itself: `size`, `batchsize` with a placeholder in front, no batchMode (nil)
            sz = list(a["sizes"])
            mods.append(("nn.Reshape", dict(nelement=int(np.prod(sz)), size=("longs", sz), batchsize=("longs", [-1] + sz))))
        elif node.op == "dropout":
            mods.append(("nn.Dropout", dict(p=0.5, v2=True, inplace=False)))
        elif node.op == "softmax":
            mods.append(("nn.SoftMax", {}))
        elif node.op == "bn":
            mods.append(("nn.SpatialBatchNormalization", dict(
                running_mean=ts[2], running_var=ts[3], weight=ts[0], bias=ts[1], eps=a["eps"])))
        elif node.op == "deconv":
            w = ts[0]
            mods.append(("nn.SpatialFullConvolution", dict(
                padW=a["padding"][1], padH=a["padding"][0], dW=a["stride"][1], dH=a["stride"][0],
                adjW=a["output_padding"][1], adjH=a["output_padding"][0], kW=w.shape[3], kH=w.shape[2],
                nInputPlane=w.shape[0], nOutputPlane=w.shape[1], weight=w,
                bias=ts[1] if len(ts) > 1 else None)))
        elif node.op == "zeropad":
            mods.append(("nn.SpatialZeroPadding", dict(pad_l=a["pad_l"], pad_r=a["pad_r"], pad_t=a["pad_t"], pad_b=a["pad_b"])))
        elif node.op == "l2normalize":
            mods.append(("nn.Normalize", {}))
        elif node.op == "logsoftmax":
            mods.append(("nn.LogSoftMax", {}))
        elif node.op == "unpool":
            mods.append(("nn.SpatialMaxUnpooling", dict(pooling=("ref", spec_of[a["pool"]]))))
        else:
            raise ValueError("no Torch7 mapping for " + node.op)
        spec_of[ni] = mods[-1]
    return ("nn.Sequential", mods)


def write_torch7(spec_or_graph, dirpath: str, mean=None, std=None):
    """Write `dirpath/model.net` (+ `stat.t7` when mean/std are given)."""
    os.makedirs(dirpath, exist_ok=True)
    if isinstance(spec_or_graph, Graph):
        g = spec_or_graph
        spec = graph_to_t7_spec(g)
        if mean is None and (np.any(g.mean != 0) or np.any(g.std != 1)):
            mean, std = g.mean, g.std
    else:
        spec = spec_or_graph
    with open(os.path.join(dirpath, "model.net"), "wb") as f:
        _t7_module(_T7(f), spec)
    if mean is not None:
        with open(os.path.join(dirpath, "stat.t7"), "wb") as f:
            t = _T7(f)
            t.table([("mean", lambda: t.tensor(np.asarray(mean, np.float32))),
                     ("std", lambda: t.tensor(np.asarray(std, np.float32)))])


# ============================================================================
# The benchmark architectures (seeded, synthetic)
# ============================================================================
def alexnet_owt(seed=0, width=1.0, size=224, classes=1000, fc=4096):
    """AlexNet "one weird trick": profilealexnetowt.lua:8-31 minus Dropout, plus SoftMax."""
    g = Graph(seed, mean=(0.45,) * 3, std=(0.225,) * 3)
    g.input_shape, g.input_dist = (3, size, size), "uniform"
    c = [max(8, int(round(v * width))) for v in (64, 192, 384, 256, 256)]
    s = size
    x = g.relu(g.conv(0, 3, c[0], 11, 4, 2)); s = (s + 4 - 11) // 4 + 1
    x = g.maxpool(x, 3, 2); s = (s - 3) // 2 + 1
    x = g.relu(g.conv(x, c[0], c[1], 5, 1, 2))
    x = g.maxpool(x, 3, 2); s = (s - 3) // 2 + 1
    x = g.relu(g.conv(x, c[1], c[2], 3, 1, 1))
    x = g.relu(g.conv(x, c[2], c[3], 3, 1, 1))
    x = g.relu(g.conv(x, c[3], c[4], 3, 1, 1))
    x = g.maxpool(x, 3, 2); s = (s - 3) // 2 + 1
    n = c[4] * s * s
    x = g.view(x, n)
    x = g.relu(g.linear(x, n, fc))
    x = g.relu(g.linear(x, fc, fc))
    x = g.linear(x, fc, classes)
    g.softmax(x)
    return g


def vgg16(seed=2, width=1.0, size=224, classes=1000, fc=4096, bias_std=0.01):
    """VGG-16; biases are non-zero because an all-zero bias is undefined in the lowp scheme."""
    g = Graph(seed)
    g.input_shape, g.input_dist = (3, size, size), "uniform"
    cfg = [(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]
    x, cin, s = 0, 3, size
    for ch, reps in cfg:
        ch = max(8, int(round(ch * width)))
        for _ in range(reps):
            x = g.relu(g.conv(x, cin, ch, 3, 1, 1, bias=bias_std))
            cin = ch
        x = g.maxpool(x, 2, 2); s //= 2
    n = cin * s * s
    x = g.view(x, n)
    x = g.relu(g.linear(x, n, fc, bias=bias_std))
    x = g.relu(g.linear(x, fc, fc, bias=bias_std))
    g.linear(x, fc, classes, bias=bias_std)
    g.fc_spatial = s  # size to pass to THMakeSpatial's first Linear
    return g


def _basic_block(g, x, cin, cout, stride):
    y = g.relu(g.bn(g.conv(x, cin, cout, 3, stride, 1, bias=None), cout))
    y = g.bn(g.conv(y, cout, cout, 3, 1, 1, bias=None), cout)
    sc = x
    if stride != 1 or cin != cout:
        sc = g.bn(g.conv(x, cin, cout, 1, stride, 0, bias=None), cout)
    return g.relu(g.add(y, sc))


def _bottleneck(g, x, cin, mid, stride):
    cout = mid * 4
    y = g.relu(g.bn(g.conv(x, cin, mid, 1, 1, 0, bias=None), mid))
    y = g.relu(g.bn(g.conv(y, mid, mid, 3, stride, 1, bias=None), mid))
    y = g.bn(g.conv(y, mid, cout, 1, 1, 0, bias=None), cout)
    sc = x
    if stride != 1 or cin != cout:
        sc = g.bn(g.conv(x, cin, cout, 1, stride, 0, bias=None), cout)
    return g.relu(g.add(y, sc))


def _resnet(seed, blocks, bottleneck, width, size, classes, fc_bias="zero"):
    g = Graph(seed)
    g.input_shape, g.input_dist = (3, size, size), "normal"
    base = max(8, int(round(64 * width)))
    x = g.relu(g.bn(g.conv(0, 3, base, 7, 2, 3, bias=None), base))
    x = g.maxpool(x, 3, 2, 1)
    s = ((size + 6 - 7) // 2 + 1 + 2 - 3) // 2 + 1
    cin = base
    for stage, reps in enumerate(blocks):
        mid = base * (2 ** stage)
        for r in range(reps):
            stride = 2 if (r == 0 and stage > 0) else 1
            if bottleneck:
                x = _bottleneck(g, x, cin, mid, stride)
                cin = mid * 4
            else:
                x = _basic_block(g, x, cin, mid, stride)
                cin = mid
            if stride == 2:
                s = (s + 2 - 3) // 2 + 1
    x = g.avgpool(x, s, s)
    x = g.view(x, cin)
    g.linear(x, cin, classes, bias=fc_bias)
    return g


def resnet18(seed=1, width=1.0, size=224, classes=1000, fc_bias="zero"):
    """fc_bias: "zero", or the standard deviation of a random bias (the uint8 engine cannot quantise an all-zero one)."""
    return _resnet(seed, [2, 2, 2, 2], False, width, size, classes, fc_bias)


def resnet50(seed=4, width=1.0, size=224, classes=1000, fc_bias="zero"):
    return _resnet(seed, [3, 4, 6, 3], True, width, size, classes, fc_bias)


def segnet(seed=3, width=1.0, size=512, classes=21, deconv_bias=None):
    """Encoder-decoder with transposed convolutions and channel-concat skips."""
    g = Graph(seed)
    g.input_shape, g.input_dist = (3, size, size), "normal"
    ch = [max(4, int(round(v * width))) for v in (32, 64, 128, 256)]
    x, cin, skips = 0, 3, []
    for c in ch:
        x = g.relu(g.bn(g.conv(x, cin, c, 3, 1, 1, bias=None), c))
        skips.append((x, c))
        x = g.maxpool(x, 2, 2)
        cin = c
    dec = [ch[3] // 2, ch[2] // 2, ch[1] // 2, ch[0] // 2]
    for i, dc in enumerate(dec):
        x = g.deconv(x, cin, dc, 4, 2, 1, 0, bias=deconv_bias)
        sx, sc = skips[3 - i]
        x = g.concat([x, sx], 1)
        cin = dc + sc
    g.conv(x, cin, classes, 1, 1, 0)
    return g


def unpool_net(seed=5, size=16, classes=6, zeropad=True):
    """Sequential Torch7-style network through the operators outside the benchmark configurations: zero padding (with a
    crop), max pooling and the unpooling that undoes it, LogSoftMax."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.relu(g.conv(0, 3, 8, 3, 1, 1, bias=0.1))
    if zeropad:
        x = g.zeropad(x, 2, -1, 1, 0)                # left 2, right crop 1, top 1: (size+1) x (size+1), square
    else:
        size -= 1
    p = g.maxpool(x, 2, 2, 0, 1)
    x = g.relu(g.conv(p, 8, 8, 3, 1, 1, bias=0.1))
    x = g.unpool(x, p)
    x = g.conv(x, 8, 4, 3, 1, 0, bias=0.1)
    n = 4 * (size - 1) * (size - 1)
    x = g.view(x, n)
    x = g.linear(x, n, classes, bias=0.1)
    g.logsoftmax(x)
    return g


def reshape_net(seed=11, size=10, maps=(3, 5, 4)):
    """conv -> View -> Linear -> Reshape(c, h, w) -> conv: a vector per image turned back into a map (Torch7 route)."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.relu(g.conv(0, 3, 4, 3, 2, 1, bias=0.1))
    n = 4 * (size // 2) * (size // 2)
    x = g.view(x, n)
    c, h, w = maps
    x = g.relu(g.linear(x, n, c * h * w, bias=0.1))
    x = g.reshape(x, c, h, w)
    g.conv(x, c, 6, 3, 1, 1, bias=0.1)
    return g


def prelu_net(seed=12, size=12, onnx_form=False):
    """conv -> PReLU (a slope per channel) -> conv -> PReLU with one shared slope (Torch7) or a leaky threshold (an ONNX
    LeakyRelu) -> max pooling -> View -> Linear -> PReLU per feature on the 2-D (batch) or 1-D (one image) tensor -> Linear."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.prelu(g.conv(0, 3, 8, 3, 1, 1, bias=0.1), 8)
    x = g.conv(x, 8, 12, 3, 1, 1, bias=0.1)
    x = g.leaky(x, 0.2) if onnx_form else g.prelu(x, 12, shared=True)
    x = g.maxpool(x, 2, 2)
    n = 12 * (size // 2) * (size // 2)
    x = g.view(x, n)
    x = g.prelu(g.linear(x, n, 16, bias=0.1), 16)
    g.linear(x, 16, 5, bias=0.1)
    return g


def normalize_net(seed=6, size=12, feat=10):
    """conv -> View -> Linear -> Normalize (rows of a 2-D tensor for a batch, the whole tensor for one image)."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.relu(g.conv(0, 3, 6, 3, 2, 1, bias=0.1))
    n = 6 * (size // 2) * (size // 2)
    x = g.view(x, n)
    x = g.linear(x, n, feat, bias=0.1)
    g.l2normalize(x)
    return g


def cmax_slice_net(seed=7, size=10, batch_slice=(1, 3)):
    """Graph-dump style network: two convolution branches meet in an elementwise maximum, then a Slice, which on this
    route always cuts dimension 0 (the batch of a 4-D tensor)."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.relu(g.conv(0, 3, 8, 3, 1, 1, bias=0.1))
    a = g.conv(x, 8, 12, 3, 1, 1, bias=0.1)
    b = g.conv(x, 8, 12, 1, 1, 0, bias=0.1)
    m = g.cmax([a, b])
    m = g.slice(m, 0, batch_slice[0], batch_slice[1])
    g.conv(m, 12, 5, 3, 1, 1, bias=0.1)
    return g


def onnx_ops_net(seed=8, size=8):
    """ONNX-only operators: Upsample (2x), Max, Slice along channels / rows / columns, LogSoftmax."""
    g = Graph(seed)
    g.input_shape = (3, size, size)
    x = g.relu(g.conv(0, 3, 12, 3, 1, 1, bias=0.1))
    u = g.upsample(g.maxpool(x, 2, 2))
    m = g.cmax([x, u])
    m = g.slice(m, 1, 3, 11)          # channels 3..10 (not aligned to a 16-byte group)
    m = g.slice(m, 2, 1, size - 1)    # rows
    m = g.slice(m, 3, 0, size - 2)    # columns
    x = g.conv(m, 8, 6, 3, 1, 1, bias=0.1)
    x = g.view(x, 6 * (size - 2) * (size - 2))
    x = g.linear(x, 6 * (size - 2) * (size - 2), 7, bias=0.1)
    g.logsoftmax(x)
    return g


BUILDERS = {"alexnet_owt": alexnet_owt, "resnet18": resnet18, "vgg16": vgg16, "segnet": segnet,
            "resnet50": resnet50}

# algorithmic GFLOP per image at full size (2 * MACs of conv / deconv / linear layers)
GFLOP_PER_IMAGE = {"alexnet_owt": 1.428, "resnet18": 3.628, "vgg16": 30.94, "segnet": 18.97,
                   "resnet50": 8.178}


# ---------------------------------------------------------------------------------------------- ONNX
def _pb_varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _pb_len(field, payload):
    return _pb_varint(field << 3 | 2) + _pb_varint(len(payload)) + payload


def _pb_int(field, v):
    return _pb_varint(field << 3) + _pb_varint(int(v))


def _onnx_tensor(name, a):
    """TensorProto: dims = 1, data_type = 2, name = 8, raw_data = 9 (float32 -> 1, int64 -> 7)."""
    a = np.ascontiguousarray(a)
    dt = 7 if a.dtype == np.int64 else 1
    if dt == 1:
        a = a.astype(np.float32)
    return b"".join(_pb_int(1, d) for d in a.shape) + _pb_int(2, dt) + _pb_len(8, name.encode()) + _pb_len(9, a.tobytes())


def _onnx_attr(name, v):
    """AttributeProto: name = 1, f = 2, i = 3, s = 4, ints = 8 (one by one), type = 20."""
    out = _pb_len(1, name.encode())
    if isinstance(v, float):
        return out + _pb_varint(2 << 3 | 5) + struct.pack("<f", v) + _pb_int(20, 1)
    if isinstance(v, int):
        return out + _pb_int(3, v) + _pb_int(20, 2)
    if isinstance(v, str):
        return out + _pb_len(4, v.encode()) + _pb_int(20, 3)
    if len(v) and isinstance(v[0], float):
        return out + _pb_len(7, struct.pack("<%df" % len(v), *v)) + _pb_int(20, 6)   # floats, packed
    return out + b"".join(_pb_int(8, i) for i in v) + _pb_int(20, 7)


def write_onnx(graph: Graph, path: str, bias_as_add=False, pad_nodes=False, global_pool=None):
    """Serialise `graph` as an ONNX ModelProto with a hand-written protobuf encoder (no onnx package needed).

    conv -> Conv, deconv -> ConvTranspose, linear -> Gemm(transB=1), bn -> BatchNormalization, threshold(0, 0) -> Relu,
    maxpool -> MaxPool, avgpool -> AveragePool, view -> Flatten, add -> Add, concat -> Concat, softmax -> Softmax,
    dropout -> Dropout.  bias_as_add writes a convolution's bias as a separate Add of a constant; pad_nodes writes its
    padding as a Pad node in front of it (two shapes the reference's loader folds back, onnx.cc:605-700).  global_pool
    ("GlobalAveragePool", "ReduceMean" or ("ReduceMean", axes)) writes every average pooling as that operator over the
    whole map -- for graphs whose average poolings cover their whole input.
    """
    nodes, inits = [], []

    def node(op, ins, out, **attrs):
        body = b"".join(_pb_len(1, i.encode()) for i in ins) + _pb_len(2, out.encode()) + _pb_len(3, ("n_" + out).encode())
        body += _pb_len(4, op.encode()) + b"".join(_pb_len(5, _onnx_attr(k, v)) for k, v in attrs.items())
        nodes.append(_pb_len(1, body))

    def init(name, a):
        inits.append(_pb_len(5, _onnx_tensor(name, a)))
        return name

    name = {0: "input"}
    for i, nd in enumerate(graph.nodes):
        if i == 0:
            continue
        a, ts = nd.attrs, [t for _, t in nd.tensors]
        ins, out = [name[j] for j in nd.inputs], "v%d" % i
        name[i] = out
        if nd.op in ("conv", "deconv"):
            src, pads = ins[0], list(a.get("pads4", list(a["padding"]) * 2))
            if (a.get("reflect") or pad_nodes) and nd.op == "conv" and any(pads):
                node("Pad", [src], out + "_pad", mode="reflect" if a.get("reflect") else "constant",
                     pads=[0, 0, pads[0], pads[1], 0, 0, pads[2], pads[3]])
                src, pads = out + "_pad", [0, 0, 0, 0]
            cin = [src, init(out + "_w", ts[0])]
            split_bias = bias_as_add and len(ts) > 1
            if len(ts) > 1 and not split_bias:
                cin.append(init(out + "_b", ts[1]))
            extra = dict(output_padding=list(a["output_padding"])) if nd.op == "deconv" else {}
            if "dilation" in a:
                extra["dilations"] = list(a["dilation"])
            if "auto_pad" in a:
                extra["auto_pad"] = a["auto_pad"]
            node("Conv" if nd.op == "conv" else "ConvTranspose", cin, out + "_c" if split_bias else out,
                 kernel_shape=list(ts[0].shape[2:]), strides=list(a["stride"]), pads=pads, **extra)
            if split_bias:
                node("Add", [out + "_c", init(out + "_b", ts[1])], out)
        elif nd.op == "linear":
            node("Gemm", [ins[0], init(out + "_w", ts[0]), init(out + "_b", ts[1])], out, alpha=1.0, beta=1.0, transB=1)
        elif nd.op == "bn":
            node("BatchNormalization", [ins[0]] + [init("%s_%d" % (out, k), t) for k, t in enumerate(ts)], out, epsilon=float(a["eps"]))
        elif nd.op == "threshold":
            if a["threshold"] != 0 or a["value"] != 0:
                raise ValueError("only ReLU maps onto ONNX here")
            if a.get("alpha"):
                node("LeakyRelu", ins, out, alpha=float(a["alpha"]))
            else:
                node("Relu", ins, out)
        elif nd.op == "prelu":
            if not a["planes"]:
                raise ValueError("one shared slope has no ONNX form the reference accepts (PReLU.c:21-29 takes the tensor's length as the plane count)")
            node("PRelu", [ins[0], init(out + "_slope", ts[0].reshape(-1, 1, 1))], out)
        elif nd.op == "avgpool" and global_pool:
            if global_pool == "GlobalAveragePool":
                node("GlobalAveragePool", ins, out)
            else:
                axes = global_pool[1] if isinstance(global_pool, tuple) else [2, 3]
                node("ReduceMean", ins, out, axes=list(axes), keepdims=1)
        elif nd.op in ("maxpool", "avgpool"):
            extra = dict(ceil_mode=int(a["ceil_mode"])) if a["ceil_mode"] else {}
            node("MaxPool" if nd.op == "maxpool" else "AveragePool", ins, out, kernel_shape=list(a["kernel_size"]),
                 strides=list(a["stride"]), pads=list(a["padding"]) * 2, **extra)
        elif nd.op == "view":
            node("Flatten", ins, out, axis=1)
        elif nd.op == "dropout":
            node("Dropout", ins, out)
        elif nd.op == "softmax":
            node("Softmax", ins, out, axis=1)
        elif nd.op in ("sigmoid", "tanh"):
            node(nd.op.capitalize(), ins, out)
        elif nd.op == "add":
            node("Add", ins, out)
        elif nd.op == "concat":
            node("Concat", ins, out, axis=int(a["dim"]))
        elif nd.op == "upsample":
            node("Upsample", ins, out, mode="nearest", scales=[1.0, 1.0, 2.0, 2.0])
        elif nd.op == "cmax":
            node("Max", ins, out)
        elif nd.op == "slice":
            node("Slice", ins, out, axes=[int(a["axis"])], starts=[int(a["start"])], ends=[int(a["stop"])])
        elif nd.op == "logsoftmax":
            node("LogSoftmax", ins, out, axis=1)
        else:
            raise ValueError("no ONNX form for " + nd.op)
    value_info = lambda n: _pb_len(1, n.encode())
    g = b"".join(nodes) + _pb_len(2, b"thnets_b200_fixture") + b"".join(inits)
    g += _pb_len(11, value_info("input")) + _pb_len(12, value_info(name[graph.output]))
    model = _pb_int(1, 3) + _pb_len(2, b"thnets_b200") + _pb_len(7, g)
    with open(path, "wb") as f:
        f.write(model)
