"""Synthetic networks of the benchmark configurations, built through the Python mirror of the
reference's interface.  Weights are seeded He-normal, biases zero (or small), as the benchmark
configurations prescribe; the last fully connected layer is scaled so that logits stay far below
the overflow point of the reference's max-less softmax."""
import numpy as np

import deepracin_b200 as dr
from cases import rng

VGG16_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def he(g, shape, fan_in):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(np.sqrt(2.0 / fan_in)))


def vgg16(graph, size=224, cfg=VGG16_CFG, fc_dims=(4096, 4096, 1000), seed="vgg16", width_div=1, softmax=True):
    """VGG-16: 13 3x3 convs + ReLU, 5 max-pools 2x2/2, FC 25088->4096->4096->1000, softmax.
    width_div shrinks the channel counts (tests); size is the input side length."""
    g = rng(seed)
    x = dr.feed_node(graph, [size, size, 3])
    node, cin, s = x, 3, size
    for v in cfg:
        if v == "M":
            node = dr.Pooling(node, "max", [1, 2, 2, 1], [1, 2, 2, 1])
            s = (s + 1) // 2
        else:
            cout = max(v // width_div, 4)
            node = dr.Conv2d(node, [3, 3, cin, cout], [1, 1, 1, 1], "relu", he(g, (3, 3, cin, cout), 9 * cin), np.zeros(cout, np.float32))
            cin = cout
    nin = s * s * cin
    for i, nout in enumerate(fc_dims):
        nout = max(nout // width_div, 8) if i < len(fc_dims) - 1 else nout
        last = i == len(fc_dims) - 1
        w = he(g, (nin, nout), nin)
        if last:
            w *= np.float32(0.05)
        node = dr.Fully_Connected(node, [nin, nout], "linear" if last else "relu", w, np.zeros(nout, np.float32))
        nin = nout
    if softmax:
        node = dr.Softmax(node)
    return x, node


def fire(graph, g, node, cin, squeeze, expand):
    sq = dr.Conv2d(node, [1, 1, cin, squeeze], [1, 1, 1, 1], "relu", he(g, (1, 1, cin, squeeze), cin), np.zeros(squeeze, np.float32))
    e1 = dr.Conv2d(sq, [1, 1, squeeze, expand], [1, 1, 1, 1], "relu", he(g, (1, 1, squeeze, expand), squeeze), np.zeros(expand, np.float32))
    e3 = dr.Conv2d(sq, [3, 3, squeeze, expand], [1, 1, 1, 1], "relu", he(g, (3, 3, squeeze, expand), 9 * squeeze), np.zeros(expand, np.float32))
    return dr.Concat([e1, e3], 2), 2 * expand


def squeezenet11(graph, size=224, classes=1000, seed="squeezenet", preamble=True):
    """SqueezeNet v1.1 in the form the reference's example graph has it: mean-subtract / BGR preamble
    (3 x Slice -> SubS -> Concat), conv1 3x3 stride 1 + average pool 2x2/2 (the reference's strided direct
    convolution is unusable), max pools 3x3/2, 8 Fire modules, conv10 1x1, global average pool, softmax."""
    g = rng(seed)
    x = dr.feed_node(graph, [size, size, 3])
    node = x
    if preamble:
        means = [123.68, 116.779, 103.939]
        chans = [dr.Sub_Scalar(dr.Slice(x, (0, 0, c), (size, size, 1)), means[c]) for c in range(3)]
        node = dr.Concat([chans[2], chans[1], chans[0]], 2)
    node = dr.Conv2d(node, [3, 3, 3, 64], [1, 1, 1, 1], "relu", he(g, (3, 3, 3, 64), 27), np.zeros(64, np.float32))
    node = dr.Pooling(node, "average", [1, 2, 2, 1], [1, 2, 2, 1])
    node = dr.Pooling(node, "max", [1, 3, 3, 1], [1, 2, 2, 1])
    cin = 64
    for i, (s, e) in enumerate([(16, 64), (16, 64), (32, 128), (32, 128), (48, 192), (48, 192), (64, 256), (64, 256)]):
        node, cin = fire(graph, g, node, cin, s, e)
        if i in (1, 3):
            node = dr.Pooling(node, "max", [1, 3, 3, 1], [1, 2, 2, 1])
    node = dr.Conv2d(node, [1, 1, cin, classes], [1, 1, 1, 1], "relu", he(g, (1, 1, cin, classes), cin) * np.float32(0.3), np.zeros(classes, np.float32))
    last = size // 16
    node = dr.Pooling(node, "average", [1, last, last, 1], [1, last, last, 1])
    node = dr.Softmax(node)
    return x, node


def synthetic_images(name, n, size):
    """uniform[0,255] minus 128 per channel, [n, size, size, 3] (HWC)"""
    g = rng(name)
    return (g.random((n, size, size, 3), dtype=np.float32) * np.float32(255.0) - np.float32(128.0))
