#!/usr/bin/env python
"""Generates tests/golden/*.npz from the UNMODIFIED reference CPU build (oracle/_ref/).

The reference ships no tests and no known-answer vectors, so its own outputs on seeded synthetic
fixtures are the golden data: this script builds each fixture (thnets_b200.fixtures, fixed seeds),
runs it through the reference's public API (THLoadNetwork / THProcessFloat, and THMakeSpatial +
THCreateLowpNetwork for the uint8 route at batch 1, first forward) and stores the outputs.  The
inputs are regenerated from their seeds by the tests, so only outputs are stored.

Run where the reference tree exists:   python tests/golden/make_golden.py
(needs `make -C oracle ref reflowp`).  Records which build flavour and thread count produced the data.
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ.setdefault("OMP_NUM_THREADS", "4")

from oracle.oracle import REF_DIR, ref_lib  # noqa: E402
from thnets_b200 import fixtures as fx  # noqa: E402
from thnets_b200.capi import THNets  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (builder kwargs, batch, file format); keep in step with tests/test_oracle.py
FP32_CASES = {
    "alexnet_owt": ("alexnet_owt", dict(width=0.25, size=224, classes=50, fc=128), 1, "t7"),
    "resnet18": ("resnet18", dict(width=0.25, size=64, classes=10), 4, "py"),
    "resnet50": ("resnet50", dict(width=0.125, size=64, classes=10), 4, "py"),
    "segnet": ("segnet", dict(width=0.5, size=32, classes=21), 4, "py"),
    "segnet_bias": ("segnet", dict(width=0.5, size=32, classes=5, deconv_bias=0.1), 4, "py"),
    "vgg16": ("vgg16", dict(width=0.125, size=32, classes=10, fc=64), 4, "t7"),
}
LOWP_CASES = {
    "vgg16_r8": (dict(width=0.125, size=32, classes=10, fc=64), 8.0),
    "vgg16_r20": (dict(width=0.25, size=64, classes=10, fc=64), 20.0),
    "vgg16_r4": (dict(width=0.25, size=32, classes=10, fc=64), 4.0),
}


def main():
    lib = ref_lib()
    assert lib, "build the reference first: make -C oracle ref reflowp"
    ref = THNets(lib)
    out = {"_flavour": os.path.basename(lib), "_threads": os.environ["OMP_NUM_THREADS"]}
    with tempfile.TemporaryDirectory() as tmp:
        for name, (builder, kw, batch, kind) in FP32_CASES.items():
            g = getattr(fx, builder)(**kw)
            x = g.make_input(batch)
            if kind == "t7":
                path = os.path.join(tmp, name)
                fx.write_torch7(g, path)
            else:
                path = os.path.join(tmp, name + ".net")
                fx.write_pymodel(g, path)
            h = ref.load_network(path)
            ref.set_stats(h, g.mean, g.std)
            y, ow, oh = ref.process_float(h, x)
            out[name] = y
            out[name + "_wh"] = np.array([ow, oh])
            ref.free_network(h)
        np.savez_compressed(os.path.join(HERE, "fp32_networks.npz"), **out)

        lowp = THNets(os.path.join(REF_DIR, "libthnets_ref_lowp.so"))
        out = {}
        for name, (kw, rng) in LOWP_CASES.items():
            g = fx.vgg16(**kw)
            x = g.make_input(1)
            path = os.path.join(tmp, name)
            fx.write_torch7(g, path)
            h = lowp.load_network(path)
            lowp.make_spatial(h, kw["size"])
            hl = lowp.create_lowp_network(h, rng)
            y, _, _ = lowp.process_float(hl, x)   # batch 1, first forward: the only state the reference gets right
            out[name] = y
        np.savez_compressed(os.path.join(HERE, "lowp_networks.npz"), **out)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
