"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

No dataset or checkpoint is involved: activations are N(0,1) (or U(0,1)), weights are uniform integers in
[-127,127], per-output-channel weight scales are U(0.001,0.01), bias is N(0,0.1).  The activation scale is
symmetric per tensor: quantize_scale = 127 / max|x|, replicated once per sample as the operator requires.
"""
import numpy as np


def conv_layer(name, n, c, h, w, o, k, stride=1, pad=0, dilation=1, act="relu", leaky=0.0):
    return dict(name=name, n=n, c=c, h=h, w=w, o=o, kh=k, kw=k, stride=stride, pad=pad, dilation=dilation, act=act,
                leaky=leaky)


def out_hw(layer):
    def dim(x, k):
        return (x + 2 * layer["pad"] - (layer["dilation"] * (k - 1) + 1)) // layer["stride"] + 1
    return dim(layer["h"], layer["kh"]), dim(layer["w"], layer["kw"])


def layer_ops(layer):
    """2 * N * O * OH * OW * C * KH * KW (real, unpadded extents)."""
    oh, ow = out_hw(layer)
    return 2 * layer["n"] * layer["o"] * oh * ow * layer["c"] * layer["kh"] * layer["kw"]


def layer_bytes(layer, out_bytes_per_elem=4):
    """Algorithmic HBM bytes of conv2d_quantized: int8 input + int8 weights + scales/bias + output."""
    oh, ow = out_hw(layer)
    return (layer["n"] * layer["c"] * layer["h"] * layer["w"] + layer["o"] * layer["c"] * layer["kh"] * layer["kw"]
            + 8 * layer["o"] + layer["n"] * layer["o"] * oh * ow * out_bytes_per_elem)


# single layer, batch 1 (runs on the reference's CPU path as is)
CONFIG0 = [conv_layer("3x3_64_64_56", 1, 64, 56, 56, 64, 3, 1, 1)]

# shape sweep at batch 32
CONFIG1 = [
    conv_layer("1x1_256_1024_14", 32, 256, 14, 14, 1024, 1, 1, 0),
    conv_layer("3x3_128_128_28", 32, 128, 28, 28, 128, 3, 1, 1),
    conv_layer("3x3s2_256_512_28", 32, 256, 28, 28, 512, 3, 2, 1),
    conv_layer("1x1_2048_512_7", 32, 2048, 7, 7, 512, 1, 1, 0),
    conv_layer("7x7s2_3_64_224", 32, 3, 224, 224, 64, 7, 2, 3),
]


def with_batch(layers, n):
    return [dict(l, n=n) for l in layers]


def make_layer_data(layer, seed=0, dist="normal"):
    """Returns dict(x fp32 NCHW, qscale float32, w int8 OIHW, dq fp32[O], bias fp32[O])."""
    rng = np.random.default_rng(seed)
    shape = (layer["n"], layer["c"], layer["h"], layer["w"])
    if dist == "normal":
        x = rng.standard_normal(shape, dtype=np.float32)
    else:
        x = rng.random(shape, dtype=np.float32)
    qscale = np.float32(127.0) / np.float32(np.abs(x).max())
    w = rng.integers(-127, 128, size=(layer["o"], layer["c"], layer["kh"], layer["kw"]), dtype=np.int8)
    sw = rng.uniform(0.001, 0.01, size=layer["o"]).astype(np.float32)
    dq = (sw / qscale).astype(np.float32)          # weight scale x activation step, one fp32 division
    bias = (rng.standard_normal(layer["o"]) * 0.1).astype(np.float32)
    return dict(x=x, qscale=qscale, w=w, dq=dq, bias=bias)
