"""Seeded parity cases shared by the golden-vector generator and the tests.

Every tensor comes from numpy's PCG64 with a seed derived from the case name, so the
generator (run where the reference checkout exists) and the tests (run anywhere) see the
same inputs.  Layouts are the oracle's: activations [n, C, H, W], conv weights
[Cin, Cout, kh, kw], fully connected weights [Nin, Nout] (rows in (y, x, z) order).
"""
import zlib

import numpy as np


def rng(name):
    return np.random.Generator(np.random.PCG64(zlib.crc32(name.encode())))


def conv_case(name, n, cin, cout, h, w, k, bias=True, scale_in=1.0):
    g = rng(name)
    x = (g.standard_normal((n, cin, h, w)) * scale_in).astype(np.float32)
    wt = (g.standard_normal((cin, cout, k, k)) * np.sqrt(2.0 / (k * k * cin))).astype(np.float32)
    b = (g.standard_normal(cout) * 0.1).astype(np.float32) if bias else None
    return x, wt, b


def fc_case(name, n, c, h, w, nout, bias=True):
    g = rng(name)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((c * h * w, nout)) * np.sqrt(2.0 / (c * h * w))).astype(np.float32)
    b = (g.standard_normal(nout) * 0.1).astype(np.float32) if bias else None
    return x, wt, b


def act_case(name, n, c, h, w, scale=1.0):
    return (rng(name).standard_normal((n, c, h, w)) * scale).astype(np.float32)


# name -> (kind, kwargs): the reference-kernel leg can run every one of these shapes
GOLDEN_CASES = {
    "wino_3to8_10x7": ("wino", dict(n=1, cin=3, cout=8, h=7, w=10, act=1, bias=True)),
    "wino_16to16_12x12": ("wino", dict(n=1, cin=16, cout=16, h=12, w=12, act=1, bias=True)),
    "wino_8to32_9x11_linear": ("wino", dict(n=1, cin=8, cout=32, h=11, w=9, act=0, bias=True)),
    "wino_32to8_8x8_nobias": ("wino", dict(n=1, cin=32, cout=8, h=8, w=8, act=1, bias=False)),
    "c1x1_16to24_10x7": ("c1x1", dict(n=1, cin=16, cout=24, h=7, w=10, act=1, bias=True)),
    "c1x1_64to16_20x20_linear": ("c1x1", dict(n=1, cin=64, cout=16, h=20, w=20, act=0, bias=True)),
    "fc_3x2x8_to_20": ("fc", dict(n=1, c=8, h=2, w=3, nout=20, act=1, bias=True)),
    "fc_4x4x16_to_64_linear": ("fc", dict(n=1, c=16, h=4, w=4, nout=64, act=0, bias=True)),
    "pool_max3s2_13x11x5": ("pool", dict(n=1, c=5, h=11, w=13, k=3, stride=2, kind=0)),
    "pool_avg2s2_9x7x4": ("pool", dict(n=1, c=4, h=7, w=9, k=2, stride=2, kind=1)),
    "pool_avg14s14_14x14x6": ("pool", dict(n=1, c=6, h=14, w=14, k=14, stride=14, kind=1)),
    "softmax_1000": ("softmax", dict(n=1, c=1000, h=1, w=1, scale=3.0)),
    "ew1_all": ("ew1", dict(n=1, c=3, h=5, w=7)),
    "ew2_all": ("ew2", dict(n=1, c=3, h=5, w=7)),
    "slice_crop": ("slice", dict(n=1, c=6, h=9, w=8)),
}


def make_inputs(name):
    kind, kw = GOLDEN_CASES[name]
    if kind == "wino":
        return conv_case(name, kw["n"], kw["cin"], kw["cout"], kw["h"], kw["w"], 3, kw["bias"])
    if kind == "c1x1":
        return conv_case(name, kw["n"], kw["cin"], kw["cout"], kw["h"], kw["w"], 1, kw["bias"])
    if kind == "fc":
        return fc_case(name, kw["n"], kw["c"], kw["h"], kw["w"], kw["nout"], kw["bias"])
    if kind == "softmax":
        return (act_case(name, kw["n"], kw["c"], kw["h"], kw["w"], kw["scale"]),)
    if kind == "ew2":
        g = rng(name)
        a = (np.abs(g.standard_normal((kw["n"], kw["c"], kw["h"], kw["w"]))) + 0.5).astype(np.float32)
        b = (np.abs(g.standard_normal((kw["n"], kw["c"], kw["h"], kw["w"]))) + 0.5).astype(np.float32)
        return a, b
    if kind == "ew1":
        return ((np.abs(act_case(name, kw["n"], kw["c"], kw["h"], kw["w"])) + 0.5).astype(np.float32),)
    return (act_case(name, kw["n"], kw["c"], kw["h"], kw["w"]),)


EW1_OPS = [(0, 1.5), (1, 0.25), (2, -3.0), (3, 7.0), (4, 0.0), (5, 0.0), (6, 0.0), (7, 2.5), (8, 1.7)]
EW2_OPS = [0, 1, 2, 3, 4]
