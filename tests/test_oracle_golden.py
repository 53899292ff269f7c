"""The C restatement (oracle/oracle.c) against the fixtures generated from the reference's compiled operators,
and against those operators live where they were built."""
import numpy as np
import pytest

from conftest import golden_cases, load_golden, same_bits


@pytest.mark.parametrize("name", golden_cases("q_"))
def test_quantize_golden(port, name):
    g = load_golden(name)
    assert np.array_equal(port.quantize(g["x"], g["scales"]), g["y"])


@pytest.mark.parametrize("name", golden_cases("c_"))
def test_conv_golden(port, name):
    g = load_golden(name)
    y = port.conv2d_quantized(g["x"], g["w"], g["pad"], g["stride"], g["dilation"], g["dq"], float(g["padding_value"]))
    assert same_bits(y, g["y_conv"])
    yb = port.add_bias(y, g["bias"])
    assert same_bits(yb, g["y_bias"])
    ya = port.activation(yb, str(g["act"]), float(g["leaky"]))
    assert same_bits(ya, g["y_act"])
    assert np.array_equal(port.quantize(ya, g["rq"]), g["y_q"])


@pytest.mark.parametrize("name", golden_cases("d_"))
def test_quantize_fp64_golden(port, name):
    g = load_golden(name)
    assert np.array_equal(port.quantize_f64(g["x"], g["scales"]), g["y"])


@pytest.mark.parametrize("name", golden_cases("p_"))
def test_max_pooling_golden(port, name):
    g = load_golden(name)
    y = port.max_pooling2d(g["x"], int(g["k"]), int(g["stride"]), g["pad"])
    assert y.shape == g["y"].shape and np.array_equal(y, g["y"])


def test_pooling_extent_is_ceil_mode(port):
    # the ResNet stem pool: 112, k3, s2 -- padding 1 on both sides gives 57 under the reference's ceil rule,
    # {1, 0} gives the familiar 56
    x = np.zeros((1, 1, 112, 112), np.float32)
    assert port.max_pooling2d(x, 3, 2, (1, 1, 1, 1)).shape == (1, 1, 57, 57)
    assert port.max_pooling2d(x, 3, 2, (1, 0, 1, 0)).shape == (1, 1, 56, 56)
    with pytest.raises(ValueError):      # a window that lies wholly in the padding
        port.max_pooling2d(np.zeros((1, 1, 4, 4), np.float32), 2, 2, (0, 2, 0, 2))


def test_fp64_rounds_half_away_everywhere(port):
    x = np.array([[0.5, 2.5, 126.5, -0.5, -2.5, 1.5, 3.5, -1.5, 0.5, 2.5, 126.5, 3e9, np.nan]], dtype=np.float64)
    assert port.quantize_f64(x, [1.0]).tolist() == [[1, 3, 127, -1, -3, 2, 4, -2, 1, 3, 127, -128, -128]]


def test_known_rounding_answers(port):
    # one scale: the 8-wide body rounds half-to-even, the tail half-away-from-zero
    x = np.array([[0.5, 2.5, 126.5, -0.5, -2.5, 1.5, 3.5, -1.5, 0.5, 2.5, 126.5]], dtype=np.float32)
    assert port.quantize(x, [1.0]).tolist() == [[0, 2, 126, 0, -2, 2, 4, -2, 1, 3, 127]]
    # several scales: half-away everywhere
    x2 = np.stack([x[0], x[0]])
    assert port.quantize(x2, [1.0, 1.0])[0].tolist() == [1, 3, 127, -1, -3, 2, 4, -2, 1, 3, 127]
    # clamp and the x86 "integer indefinite" result of out-of-range products
    x3 = np.array([[200.0, -200.0, 3e9, -3e9, np.nan, np.inf, 127.4, -128.4]], dtype=np.float32)
    assert port.quantize(x3, [1.0]).tolist() == [[127, -128, -128, -128, -128, -128, 127, -128]]


def test_max_magnitude_accumulators(port):
    x = np.full((1, 512, 3, 3), -128, dtype=np.int8)
    w = np.full((2, 512, 3, 3), -127, dtype=np.int8)
    w[1] = 127
    y, acc = port.conv2d_quantized(x, w, (1, 1, 1, 1), (1, 1), (1, 1), np.ones(2, np.float32), return_acc=True)
    assert acc[0, 0, 1, 1] == 512 * 9 * 128 * 127 and acc[0, 1, 1, 1] == -512 * 9 * 128 * 127
    assert y[0, 0, 1, 1] == np.float32(512 * 9 * 128 * 127)


def test_port_matches_reference_live(port, reference):
    rng = np.random.default_rng(7)
    for count, nscales in [(1, 1), (9, 1), (64, 1), (1003, 1), (30, 3), (31, 4), (7, 7)]:
        x = (rng.standard_normal((nscales, count // nscales if nscales > 1 and count % nscales == 0 else count)) * 50).astype(np.float32)
        x = x[:nscales]
        s = rng.uniform(0.5, 2.0, size=nscales).astype(np.float32)
        assert np.array_equal(port.quantize(x, s), reference.quantize(x, s))
    for count, nscales in [(9, 1), (1003, 1), (30, 3), (31, 4)]:
        x = (rng.standard_normal((nscales, count)) * 50)
        x[0, :4] = [0.5, 2.5, -0.5, 1e12]
        s = rng.uniform(0.5, 2.0, size=nscales).astype(np.float32)
        assert np.array_equal(port.quantize_f64(x, s), reference.quantize_f64(x, s))
    for (shape, k, st, pad) in [((2, 3, 112, 112), 3, 2, (1, 1, 1, 1)), ((1, 2, 13, 9), 3, 2, (1, 0, 0, 1)), ((1, 1, 8, 8), 2, 2, (0, 0, 0, 0)),
                                ((1, 2, 7, 7), 3, 1, (1, 1, 1, 1)), ((1, 2, 10, 11), 5, 3, (2, 2, 2, 2))]:
        x = rng.standard_normal(shape).astype(np.float32)
        a, b = port.max_pooling2d(x, k, st, pad), reference.max_pooling2d(x, k, st, pad)
        assert a.shape == b.shape and np.array_equal(a, b), (shape, k, st, pad)
    cases = [(2, 5, 8, 8, 7, 3, 2, (1, 1, 0, 1), (1, 2), (1, 1)), (1, 6, 6, 6, 3, 1, 1, (1, 1, 1, 1), (1, 1), (3, 3)),
             (1, 3, 12, 12, 4, 5, 5, (2, 2, 2, 2), (3, 3), (1, 1))]
    for (N, C, H, W, O, KH, KW, pad, st, dl) in cases:
        x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
        w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
        dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
        for pv in (0.0, -2.7):
            assert same_bits(port.conv2d_quantized(x, w, pad, st, dl, dq, pv), reference.conv2d_quantized(x, w, pad, st, dl, dq, pv))
