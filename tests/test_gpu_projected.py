"""The expansion convolution of a residual block with its projection shortcut inside the same launch
(tsb_conv2d_i8_run_projected), against the CPU checker's operator chain
    add(add_bias(conv2d_quantized(x, w)), add_bias(conv2d_quantized(x_shortcut, w_shortcut))) -> activation -> quantize
int8 bit for bit, fp32 bit for bit up to the sign of zero."""
import numpy as np
import pytest
import torch

from conftest import same_bits

pytestmark = pytest.mark.gpu

ACT = {"none": 0, "relu": 1, "leaky_relu": 2}


def run_projected(x, w, xs, ws, stride_s, dq, bias, dqs, bias_s, act, leaky, rq, res_after=False, tile_channels=0,
                  want_f32=True, kernel_main=(1, 1), pad_main=(0, 0, 0, 0)):
    from tennis_b200 import ops
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    main = ops.ConvPlan(x.shape, w.shape, pad_main, (1, 1), (1, 1), 0.0, 2, dev)
    main.set_weights(t(w))
    short = ops.ConvPlan(xs.shape, ws.shape, (0, 0, 0, 0), stride_s, (1, 1), 0.0, 2, dev)
    short.set_weights(t(ws))
    N, O, OH, OW = main.out_shape
    assert short.out_shape == main.out_shape
    xin, xsin = ops.repack_nchw_to_nhwc(t(x)), ops.repack_nchw_to_nhwc(t(xs))
    out_f32 = torch.full((N, OH, OW, O), float("nan"), dtype=torch.float32, device=dev) if want_f32 else None
    out_i8 = torch.full((N, OH, OW, ops.padded_channels(O)), 99, dtype=torch.int8, device=dev) if rq is not None else None
    main.run_projected(xin, short, xsin, t(dq), t(dqs), bias=None if bias is None else t(bias),
                       shortcut_bias=None if bias_s is None else t(bias_s), activation=ACT[act], leaky=leaky,
                       out_f32=out_f32, out_i8=out_i8, requant_scales=None if rq is None else list(rq),
                       residual_after_activation=res_after, tile_channels=tile_channels)
    main.status()
    torch.cuda.synchronize()
    r = {}
    if want_f32:
        r["f32"] = out_f32.cpu().numpy().transpose(0, 3, 1, 2)
    if out_i8 is not None:
        q = out_i8.cpu().numpy()
        assert not q[..., O:].any(), "padding channels of the NHWC int8 output must be zero"
        r["i8"] = q[..., :O].transpose(0, 3, 1, 2)
    return r


def expected(checker, x, w, xs, ws, stride_s, dq, bias, dqs, bias_s, act, leaky, rq, res_after, pad_main=(0, 0, 0, 0)):
    y = checker.conv2d_quantized(x, w, pad_main, (1, 1), (1, 1), dq, 0.0)
    if bias is not None:
        y = checker.add_bias(y, bias)
    s = checker.conv2d_quantized(xs, ws, (0, 0, 0, 0), stride_s, (1, 1), dqs, 0.0)
    if bias_s is not None:
        s = checker.add_bias(s, bias_s)
    if not res_after:
        y = (y + s).astype(np.float32)
    y = checker.activation(y, act, leaky)
    if res_after:
        y = (y + s).astype(np.float32)
    return y, (checker.quantize(y, rq) if rq is not None else None)


def make(rng, N, C, Cs, H, W, O, stride, kmain=1):
    x = rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, (O, C, kmain, kmain), dtype=np.int8)
    xs = rng.integers(-128, 128, (N, Cs, (H - 1) * stride + 1 + (stride - 1) * (N % 2), (W - 1) * stride + 1), dtype=np.int8)
    ws = rng.integers(-127, 128, (O, Cs, 1, 1), dtype=np.int8)
    dq = (rng.random(O).astype(np.float32) + 0.5) * 1e-3
    dqs = (rng.random(O).astype(np.float32) + 0.5) * 1e-3
    bias = rng.standard_normal(O).astype(np.float32)
    bias_s = rng.standard_normal(O).astype(np.float32)
    return x, w, xs, ws, dq, dqs, bias, bias_s


# N, C (main), C (shortcut), H, W (output grid), O, shortcut stride, tile_channels
CASES = [
    (2, 64, 64, 14, 14, 256, 1, 0),        # ResNet stage 1: both 1x1 over the same pixels
    (2, 64, 64, 14, 14, 256, 1, 128),
    (3, 128, 256, 9, 7, 512, 2, 0),        # a stride-2 projection, two channel tiles, ragged pixel tile
    (3, 128, 256, 9, 7, 512, 2, 128),
    (2, 64, 192, 5, 5, 200, 2, 0),         # K blocks of 64 on one side, O not a multiple of 32
    (2, 512, 1024, 7, 7, 2048, 2, 0),      # stage 4: streamed weights, eight channel tiles
    (5, 256, 128, 12, 12, 128, 1, 0),      # at most 128 output channels
    (40, 64, 64, 28, 28, 256, 1, 0),       # more tiles than SMs: resident weights, several tiles per CTA
    (40, 64, 64, 28, 28, 256, 1, 128),
]


@pytest.mark.parametrize("case", CASES)
def test_projected_shortcut_matches_the_operator_chain(checker, case):
    N, C, Cs, H, W, O, stride, tile = case
    rng = np.random.default_rng(sum(case))
    x, w, xs, ws, dq, dqs, bias, bias_s = make(rng, N, C, Cs, H, W, O, stride)
    rq = (rng.random(N).astype(np.float32) + 0.5) * 20.0
    want_f, want_q = expected(checker, x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, "relu", 0.0, rq, False)
    got = run_projected(x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, "relu", 0.0, rq, tile_channels=tile)
    assert same_bits(got["f32"], want_f), "fp32 output differs"
    assert np.array_equal(got["i8"], want_q), "requantized int8 output differs"


@pytest.mark.parametrize("variant", ["after_leaky", "no_bias", "i8_only", "f32_only", "3x3_main"])
def test_projected_shortcut_variants(checker, variant):
    rng = np.random.default_rng(11)
    N, C, Cs, H, W, O, stride = 3, 64, 128, 10, 10, 256, 2
    kmain = 3 if variant == "3x3_main" else 1
    pad = (1, 1, 1, 1) if kmain == 3 else (0, 0, 0, 0)
    x, w, xs, ws, dq, dqs, bias, bias_s = make(rng, N, C, Cs, H, W, O, stride, kmain)
    rq = np.array([9.0, 11.0, 13.0], np.float32)    # one scale per image (a single scale takes the operator's other rounding)
    act, leaky, after = ("leaky_relu", 0.1, True) if variant == "after_leaky" else ("relu", 0.0, False)
    if variant == "no_bias":
        bias = bias_s = None
    if variant == "f32_only":
        rq = None
    want_f, want_q = expected(checker, x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, act, leaky, rq, after, pad)
    got = run_projected(x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, act, leaky, rq, res_after=after,
                        want_f32=variant != "i8_only", pad_main=pad)
    if variant != "i8_only":
        assert same_bits(got["f32"], want_f)
    if rq is not None:
        assert np.array_equal(got["i8"], want_q)


def test_projected_shortcut_values_beyond_int32_take_the_exact_path(checker):
    """Requantized values beyond the int32 range (they quantize to -128 in the reference) leave the tile path."""
    rng = np.random.default_rng(5)
    N, C, Cs, H, W, O, stride = 2, 64, 64, 6, 6, 256, 1
    x, w, xs, ws, dq, dqs, bias, bias_s = make(rng, N, C, Cs, H, W, O, stride)
    bias_s[::7] = 3e9
    rq = np.array([4.0, 5.0], np.float32)
    want_f, want_q = expected(checker, x, w, xs, ws, (1, 1), dq, bias, dqs, bias_s, "relu", 0.0, rq, False)
    got = run_projected(x, w, xs, ws, (1, 1), dq, bias, dqs, bias_s, "relu", 0.0, rq)
    assert same_bits(got["f32"], want_f)
    assert np.array_equal(got["i8"], want_q)


def test_projected_shortcut_refuses_what_it_cannot_run():
    from tennis_b200 import ops
    from tennis_b200._lib import TsbError
    dev = torch.device("cuda")
    main = ops.ConvPlan((1, 64, 8, 8), (256, 64, 1, 1), (0, 0, 0, 0), (1, 1), (1, 1), 0.0, 2, dev)
    main.set_weights(torch.zeros((256, 64, 1, 1), dtype=torch.int8, device=dev))
    bad = ops.ConvPlan((1, 64, 8, 8), (256, 64, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 0.0, 2, dev)   # not 1x1
    bad.set_weights(torch.zeros((256, 64, 3, 3), dtype=torch.int8, device=dev))
    x = torch.zeros((1, 8, 8, 64), dtype=torch.int8, device=dev)
    dq = torch.ones(256, device=dev)
    out = torch.empty((1, 8, 8, 256), device=dev)
    with pytest.raises(TsbError) as e:
        main.run_projected(x, bad, x, dq, dq, out_f32=out)
    assert "1x1" in str(e.value)


@pytest.mark.parametrize("seed", range(16))
def test_projected_shortcut_random_geometry(checker, seed):
    rng = np.random.default_rng(500 + seed)
    N = int(rng.integers(2, 5))
    C, Cs = int(rng.choice([64, 128, 192, 256])), int(rng.choice([64, 128, 192, 320]))
    H, W = int(rng.integers(3, 21)), int(rng.integers(3, 21))
    O = int(rng.choice([64, 100, 128, 256, 260, 512]))
    stride = int(rng.integers(1, 4))
    tile = int(rng.choice([0, 128, 256]))
    x, w, xs, ws, dq, dqs, bias, bias_s = make(rng, N, C, Cs, H, W, O, stride)
    if seed % 4 == 0:
        bias_s = None
    rq = (rng.random(N).astype(np.float32) + 0.5) * 25.0
    act, leaky, after = [("relu", 0.0, False), ("leaky_relu", 0.1, True), ("none", 0.0, False)][seed % 3]
    want_f, want_q = expected(checker, x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, act, leaky, rq, after)
    got = run_projected(x, w, xs, ws, (stride, stride), dq, bias, dqs, bias_s, act, leaky, rq, res_after=after, tile_channels=tile)
    assert same_bits(got["f32"], want_f)
    assert np.array_equal(got["i8"], want_q)


# N, C_first, C_rest, H, W, O, tile_channels
CONCAT_CASES = [
    (2, 64, 64, 12, 12, 64, 0),
    (2, 64, 64, 12, 12, 128, 256),
    (3, 128, 128, 9, 7, 256, 0),
    (2, 256, 256, 6, 6, 512, 0),
    (2, 64, 192, 5, 5, 200, 0),
    (40, 64, 64, 28, 28, 128, 0),          # several tiles per CTA
]


@pytest.mark.parametrize("case", CONCAT_CASES)
def test_convolution_over_a_concatenation_without_the_concatenation(checker, case):
    """tsb_conv2d_i8_run_concat against concat -> conv2d_quantized -> add_bias -> leaky_relu -> quantize of the checker."""
    from tennis_b200 import ops
    N, C1, C2, H, W, O, tile = case
    rng = np.random.default_rng(sum(case))
    x1 = rng.integers(-128, 128, (N, C1, H, W), dtype=np.int8)
    x2 = rng.integers(-128, 128, (N, C2, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, (O, C1 + C2, 1, 1), dtype=np.int8)
    dq = (rng.random(O).astype(np.float32) + 0.5) * 1e-3
    bias = rng.standard_normal(O).astype(np.float32)
    rq = (rng.random(N).astype(np.float32) + 0.5) * 20.0
    y = checker.conv2d_quantized(np.concatenate([x1, x2], axis=1), w, (0, 0, 0, 0), (1, 1), (1, 1), dq, 0.0)
    y = checker.activation(checker.add_bias(y, bias), "leaky_relu", 0.1)
    want_q = checker.quantize(y, rq)

    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    first = ops.ConvPlan(x1.shape, (O, C1, 1, 1), (0, 0, 0, 0), (1, 1), (1, 1), 0.0, 2, dev)
    first.set_weights(t(w[:, :C1]))
    rest = ops.ConvPlan(x2.shape, (O, C2, 1, 1), (0, 0, 0, 0), (1, 1), (1, 1), 0.0, 2, dev)
    rest.set_weights(t(w[:, C1:]))
    out_f32 = torch.full((N, H, W, O), float("nan"), dtype=torch.float32, device=dev)
    out_i8 = torch.full((N, H, W, ops.padded_channels(O)), 99, dtype=torch.int8, device=dev)
    rest.run_concat(ops.repack_nchw_to_nhwc(t(x2)), first, ops.repack_nchw_to_nhwc(t(x1)), t(dq), bias=t(bias), activation=2,
                    leaky=0.1, out_f32=out_f32, out_i8=out_i8, requant_scales=list(rq), tile_channels=tile)
    rest.status()
    torch.cuda.synchronize()
    assert same_bits(out_f32.cpu().numpy().transpose(0, 3, 1, 2), y)
    q = out_i8.cpu().numpy()
    assert not q[..., O:].any()
    assert np.array_equal(q[..., :O].transpose(0, 3, 1, 2), want_q)
