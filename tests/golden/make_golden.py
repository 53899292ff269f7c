"""Generates tests/golden/*.npz from the reference's own compiled CPU operators.

Run in a container that has the reference tree (it builds oracle/_ref from the sources where they lie):
    python tests/golden/make_golden.py
Each file holds the inputs and the outputs of quantize / conv2d_quantized / add_bias / relu / leaky_relu as
the reference computes them with one computing thread on an x86-64 AVX2 build.  The fixtures are small on
purpose; they pin the rounding rules, the padding rules and the operator order.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

QUANT_CASES = [
    # (name, shape, number of scales)
    ("q_one_scale_tail0", (1, 2, 4, 4), 1),
    ("q_one_scale_tail3", (1, 3, 5, 5), 1),
    ("q_one_scale_tail7", (1, 1, 3, 13), 1),
    ("q_short", (1, 5), 1),
    ("q_batch4", (4, 3, 5, 7), 4),
    ("q_batch3_ragged", (3, 7), 3),
    ("q_weights_per_channel", (6, 4, 3, 3), 6),
]

# quantize of FLOAT64 tensors: (name, shape, number of scales)
QUANT64_CASES = [
    ("d_one_scale", (1, 3, 5, 5), 1),
    ("d_batch4", (4, 3, 5, 7), 4),
]

# pooling2d, type max: (name, N, C, H, W, k, stride, pad(t,b,l,r))
POOL_CASES = [
    ("p_k3s2_p1_ceil", 2, 3, 12, 12, 3, 2, (1, 1, 1, 1)),      # ceil mode adds a last window: 12 -> 7
    ("p_k3s2_p1_0", 1, 4, 12, 14, 3, 2, (1, 0, 1, 0)),         # how a floor-mode pool reaches TenniS: 12 -> 6
    ("p_k2s2", 2, 2, 9, 7, 2, 2, (0, 0, 0, 0)),                # odd extents, clipped last window
    ("p_k3s1_p1", 1, 2, 6, 5, 3, 1, (1, 1, 1, 1)),
]

CONV_CASES = [
    # name, N, C, H, W, O, KH, KW, pad(t,b,l,r), stride, dilation, padding_value, act, leaky
    ("c_3x3_p1", 1, 8, 9, 9, 5, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0, "relu", 0.0),
    ("c_7x7_s2_p3_c3", 2, 3, 15, 17, 6, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), 0.0, "relu", 0.0),
    ("c_1x1", 2, 16, 7, 7, 12, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 0.0, "none", 0.0),
    ("c_1x1_s2", 1, 6, 8, 8, 4, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1), 0.0, "leaky_relu", 0.1),
    ("c_asym_pad_dil2", 1, 4, 10, 12, 6, 3, 3, (2, 0, 1, 3), (2, 1), (2, 2), 0.0, "leaky_relu", 0.1),
    ("c_pad_value", 1, 5, 6, 6, 3, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 3.0, "relu", 0.0),
    ("c_64ch", 2, 64, 6, 6, 16, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0, "relu", 0.0),
    ("c_maxmag", 1, 32, 5, 5, 4, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0, "none", 0.0),
]


def tie_values(rng, shape):
    """Random values with exact .5 ties, clamps and negatives sprinkled in."""
    x = (rng.standard_normal(shape) * 60).astype(np.float32)
    flat = x.reshape(-1)
    special = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, -127.5, -128.5, 300.0, -300.0, 0.49999997,
                        -0.49999997], dtype=np.float32)
    idx = rng.permutation(flat.size)[:min(flat.size, special.size)]
    flat[idx] = special[:idx.size]
    flat[-1] = 2.5  # a tie in the scalar tail of the one-scale path
    return x


def main():
    orc.build()
    ref = orc.Reference()
    rng = np.random.default_rng(20240)
    for name, shape, nscales in QUANT_CASES:
        x = tie_values(rng, shape)
        scales = np.ones(nscales, dtype=np.float32)
        if nscales > 1:
            scales[1:] = rng.uniform(0.5, 2.0, size=nscales - 1).astype(np.float32)
        y = ref.quantize(x, scales)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x, scales=scales, y=y)
    for (name, N, C, H, W, O, KH, KW, pad, stride, dil, pv, act, leaky) in CONV_CASES:
        if name == "c_maxmag":
            x = np.full((N, C, H, W), -128, dtype=np.int8)
            w = np.full((O, C, KH, KW), -127, dtype=np.int8)
            w[1::2] = 127
        else:
            x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
            w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
        dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
        bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
        y_conv = ref.conv2d_quantized(x, w, pad, stride, dil, dq, pv)
        y_bias = ref.add_bias(y_conv, bias)
        y_act = ref.activation(y_bias, act, leaky)
        amax = float(np.abs(y_act).max())
        rq = np.full(N, np.float32(127.0) / np.float32(amax if amax > 0 else 1.0), dtype=np.float32)
        y_q = ref.quantize(y_act, rq)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x, w=w, dq=dq, bias=bias, pad=np.array(pad),
                            stride=np.array(stride), dilation=np.array(dil), padding_value=np.float32(pv),
                            act=np.array(act), leaky=np.float32(leaky), y_conv=y_conv, y_bias=y_bias, y_act=y_act,
                            rq=rq, y_q=y_q)
    for name, shape, nscales in QUANT64_CASES:
        x = tie_values(rng, shape).astype(np.float64)
        x.reshape(-1)[1] = 0.49999999999999994     # just below a tie in double
        x.reshape(-1)[2] = 3e9                      # beyond int32: -128
        scales = np.ones(nscales, dtype=np.float32)
        if nscales > 1:
            scales[1:] = rng.uniform(0.5, 2.0, size=nscales - 1).astype(np.float32)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x, scales=scales, y=ref.quantize_f64(x, scales))
    for name, N, C, H, W, k, stride, pad in POOL_CASES:
        x = rng.standard_normal((N, C, H, W)).astype(np.float32)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x, k=np.int32(k), stride=np.int32(stride), pad=np.array(pad),
                            y=ref.max_pooling2d(x, k, stride, pad))
    print("wrote", len(QUANT_CASES) + len(CONV_CASES) + len(QUANT64_CASES) + len(POOL_CASES), "fixtures to", HERE)


if __name__ == "__main__":
    main()
