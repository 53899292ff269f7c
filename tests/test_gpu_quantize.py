"""Parity of the CUDA quantize / staging kernels with the CPU checker, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden, same_bits

pytestmark = pytest.mark.gpu


def gpu_quantize(x, scales):
    from tennis_b200 import ops
    q = ops.Quantize()
    q.set("quantize_scale", np.asarray(scales, np.float32))
    q.init()
    return q.run([torch.from_numpy(np.ascontiguousarray(x)).cuda()]).cpu().numpy()


def ties(rng, shape, spread=60.0):
    x = (rng.standard_normal(shape) * spread).astype(np.float32)
    flat = x.reshape(-1)
    special = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, -127.5, -128.5, 300.0, -300.0, 3e9, -3e9,
                        np.nan, np.inf, -np.inf, 0.49999997], dtype=np.float32)
    idx = rng.permutation(flat.size)[:min(flat.size, special.size)]
    flat[idx] = special[:idx.size]
    return x


@pytest.mark.parametrize("name", golden_cases("q_"))
def test_quantize_golden(name):
    g = load_golden(name)
    assert np.array_equal(gpu_quantize(g["x"], g["scales"]), g["y"])


@pytest.mark.parametrize("name", golden_cases("d_"))
def test_quantize_fp64_golden(name):
    g = load_golden(name)
    assert np.array_equal(gpu_quantize(g["x"], g["scales"]), g["y"])


@pytest.mark.parametrize("shape", [(1, 1), (1, 9), (1, 17), (1, 1003), (3, 7), (4, 3, 5, 5), (200, 4, 3, 3), (2, 100003)])
def test_fp64_input(checker, shape):
    """FLOAT64 tensors take the reference's generic branch: a double product, half-away rounding for every element."""
    rng = np.random.default_rng(sum(shape))
    x = ties(rng, shape).astype(np.float64)
    x.reshape(-1)[0] = 0.49999999999999994     # below a tie in double, a tie once narrowed to fp32
    x.reshape(-1)[-1] = 2.5000000000000004
    s = rng.uniform(0.5, 2.0, size=shape[0]).astype(np.float32)
    s[0] = 1.0
    assert np.array_equal(gpu_quantize(x, s), checker.quantize_f64(x, s))
    # misaligned view: the element-at-a-time kernel
    from tennis_b200 import _lib, ops
    flat = torch.from_numpy(x.reshape(-1)).cuda()
    if flat.numel() > 40:
        y = torch.zeros(flat.numel(), dtype=torch.int8, device="cuda")
        _lib.check(_lib.load().tsb_quantize_f64_i8(ops._ptr(flat[1:]), ops._ptr(y[1:]), flat.numel() - 1, _lib.float_array([1.0]), 1,
                                                   ops._stream_ptr()))
        assert np.array_equal(y[1:].cpu().numpy(), checker.quantize_f64(x.reshape(1, -1)[:, 1:], [1.0])[0])


@pytest.mark.parametrize("count", [1, 7, 8, 9, 15, 16, 17, 24, 31, 32, 33, 255, 1000, 1003, 4099, 100003])
def test_one_scale_tails_and_ties(checker, count):
    rng = np.random.default_rng(count)
    x = ties(rng, (1, count))
    x[0, -1] = 2.5
    for s in (1.0, 0.37, 2.0):
        assert np.array_equal(gpu_quantize(x, [s]), checker.quantize(x, [s])), (count, s)


@pytest.mark.parametrize("shape", [(2, 5), (3, 7), (4, 3, 5, 5), (5, 3), (7, 1, 1, 3), (64, 3, 16, 16), (3, 1000)])
def test_scale_groups(checker, shape):
    rng = np.random.default_rng(sum(shape))
    x = ties(rng, shape)
    s = rng.uniform(0.5, 2.0, size=shape[0]).astype(np.float32)
    s[0] = 1.0
    assert np.array_equal(gpu_quantize(x, s), checker.quantize(x, s))


def test_many_scales_go_through_device_table(checker):
    rng = np.random.default_rng(5)
    x = ties(rng, (200, 4, 3, 3))
    s = rng.uniform(0.5, 2.0, size=200).astype(np.float32)
    assert np.array_equal(gpu_quantize(x, s), checker.quantize(x, s))


def test_misaligned_views(checker):
    from tennis_b200 import _lib, ops
    rng = np.random.default_rng(11)
    base = ties(rng, (1, 4099))
    xb = torch.from_numpy(base).cuda()
    for off in (1, 3, 4):
        x = xb[:, off:off + 4000]
        y_store = torch.zeros(4100, dtype=torch.int8, device="cuda")
        y = y_store[off:off + 4000]
        _lib.check(_lib.load().tsb_quantize_f32_i8(ops._ptr(x), ops._ptr(y), 4000,
                                                   _lib.float_array([1.0]), 1, ops._stream_ptr()))
        want = checker.quantize(base[:, off:off + 4000], [1.0])
        assert np.array_equal(y.cpu().numpy(), want[0])
        assert int(y_store[:off].abs().sum()) == 0 and int(y_store[off + 4000:].abs().sum()) == 0


def test_empty_tensor_is_a_no_op():
    from tennis_b200 import _lib, ops
    x = torch.zeros(16, device="cuda")
    y = torch.full((16,), 7, dtype=torch.int8, device="cuda")
    _lib.check(_lib.load().tsb_quantize_f32_i8(ops._ptr(x), ops._ptr(y), 0, _lib.float_array([1.0]), 1, ops._stream_ptr()))
    assert int(y.sum()) == 7 * 16


@pytest.mark.parametrize("shape,nscales", [((1, 3, 5, 7), 1), ((2, 64, 9, 9), 2), ((3, 70, 8, 8), 3), ((2, 17, 4, 4), 2),
                                           ((1, 130, 13, 5), 1), ((4, 256, 14, 14), 4)])
def test_quantize_to_nhwc_matches_flat_quantize(checker, shape, nscales):
    from tennis_b200 import ops
    rng = np.random.default_rng(shape[1])
    x = ties(rng, shape)
    s = rng.uniform(0.5, 2.0, size=nscales).astype(np.float32)
    want = checker.quantize(x, s)
    y = ops.quantize_nchw_to_nhwc(torch.from_numpy(x).cuda(), list(s))
    cp = ops.padded_channels(shape[1])
    assert tuple(y.shape) == (shape[0], shape[2], shape[3], cp)
    got = y.cpu().numpy()
    assert np.array_equal(got[..., :shape[1]].transpose(0, 3, 1, 2), want)
    assert not got[..., shape[1]:].any()
    # and the int8 repack both ways
    xq = torch.from_numpy(want).cuda()
    assert np.array_equal(ops.repack_nchw_to_nhwc(xq).cpu().numpy(), got)
    assert np.array_equal(ops.repack_nhwc_to_nchw(y, shape[1]).cpu().numpy(), want)


def test_elementwise_epilogue_operators(checker):
    from tennis_b200 import ops
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 5, 7, 9)).astype(np.float32)
    x.reshape(-1)[:4] = [0.0, -0.0, 1e-30, -1e-30]
    b = rng.standard_normal(5).astype(np.float32)
    xd, bd = torch.from_numpy(x).cuda(), torch.from_numpy(b).cuda()
    assert same_bits(ops.add_bias(xd, bd).cpu().numpy(), checker.add_bias(x, b))
    assert same_bits(ops.relu(xd).cpu().numpy(), checker.relu(x))
    assert same_bits(ops.leaky_relu(xd, 0.1).cpu().numpy(), checker.leaky_relu(x, 0.1))


def test_full_size_properties():
    """Configuration-size input (64 x 3 x 224 x 224): idempotence of the grid against the value domain --
    every output equals the quantization of its own input element computed independently in torch fp32
    for non-tie values, and the NHWC staging is a permutation of the flat result."""
    from tennis_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((64, 3, 224, 224), device="cuda", generator=g)
    s = float(127.0 / x.abs().max())
    q = ops.Quantize()
    q.set("quantize_scale", np.full(64, s, np.float32))
    q.init()
    y = q.run([x])
    v = x * s
    frac = (v - torch.floor(v)).abs()
    safe = (frac - 0.5).abs() > 1e-3
    want = torch.clamp(torch.round(v), -128, 127).to(torch.int8)
    assert bool((y[safe] == want[safe]).all())
    assert int(y.max()) == 127 or int(y.min()) == -127
    yn = ops.quantize_nchw_to_nhwc(x, [s] * 64)
    assert bool((yn[..., :3].permute(0, 3, 1, 2) == y).all()) and not bool(yn[..., 3:].any())
