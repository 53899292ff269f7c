"""Seeded random sweep over convolution geometries (sizes, paddings, strides, dilations, channel counts that are not
multiples of anything) through both kernels and every plan mode the heuristics pick, against the CPU checker: int32
accumulators and requantized int8 bit for bit, fp32 up to the sign of zero."""
import numpy as np
import pytest

from test_gpu_conv import check_case

pytestmark = pytest.mark.gpu


def random_case(seed):
    rng = np.random.default_rng(1000 + seed)
    N = int(rng.integers(1, 4))
    C = int(rng.choice([1, 3, 4, 8, 13, 16, 17, 24, 64, 72, 128, 160]))
    KH, KW = (int(v) for v in rng.choice([1, 2, 3, 5, 7], size=2))
    if seed % 3 == 0:
        KW = KH
    dh, dw = (int(v) for v in rng.choice([1, 1, 1, 2], size=2))
    sh, sw = (int(v) for v in rng.choice([1, 1, 2, 3], size=2))
    pad = tuple(int(v) for v in rng.integers(0, 4, size=4))
    H = int(rng.integers((KH - 1) * dh + 1, (KH - 1) * dh + 34))
    W = int(rng.integers((KW - 1) * dw + 1, (KW - 1) * dw + 34))
    O = int(rng.choice([1, 5, 16, 31, 32, 64, 65, 96, 128, 130, 200, 256, 300]))
    x = rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, (O, C, KH, KW), dtype=np.int8)
    dq = (rng.random(O).astype(np.float32) + 0.25) * np.float32(2e-4)
    bias = rng.standard_normal(O).astype(np.float32) if seed % 4 else None
    act, leaky = [("relu", 0.0), ("leaky_relu", 0.1), ("none", 0.0)][seed % 3]
    rq = (rng.random(N).astype(np.float32) + 0.5) * np.float32(30.0) if N > 1 else np.array([17.0], np.float32)
    return x, w, pad, (sh, sw), (dh, dw), dq, bias, act, leaky, rq


@pytest.mark.parametrize("seed", range(48))
def test_random_geometry(checker, port, seed):
    x, w, pad, stride, dil, dq, bias, act, leaky, rq = random_case(seed)
    kernel = 0 if seed % 5 else 1          # mostly the plan's own choice (tcgen05 where it applies); every fifth: direct
    layouts = [dict(), dict(x_layout="nhwc", i8_layout="nhwc"), dict(x_layout="nhwc", i8_layout="nhwc", f32_layout="nhwc")]
    check_case(checker, port, x, w, pad, stride, dil, dq, bias, act, leaky, 0.0, kernel, rq=rq, **layouts[seed % 3])
