"""Parity of the CUDA convolution kernels (tcgen05 implicit GEMM and the direct kernel) with the CPU checker,
through the C ABI: int32 accumulators and int8 outputs bit-exact, fp32 outputs bit-exact up to the sign of
zero (the stated bar is 1e-5 relative; every step is a single correctly rounded fp32 operation, so the
tests ask for equality)."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden, same_bits

pytestmark = pytest.mark.gpu

ACT = {"none": 0, "relu": 1, "leaky_relu": 2}


def run_gpu(x, w, pad, stride, dil, dq, bias=None, act="none", leaky=0.0, padding_value=0.0, kernel=0,
            x_layout="nchw", residual=None, rq=None, i8_layout="nchw", f32_layout="nchw", want_acc=True, want_f32=True,
            res_after=False, tune=None):
    """x int8 NCHW numpy.  Returns dict(kernel, acc, f32, i8) as NCHW numpy arrays."""
    from tennis_b200 import _lib, ops
    dev = torch.device("cuda")
    xd = torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    wd = torch.from_numpy(np.ascontiguousarray(w)).to(dev)
    # tune: overrides of the plan heuristics (tsb_conv_desc.mma_orientation / raw_row_mode / patch_mode), 0 = automatic
    plan = ops.ConvPlan(x.shape, w.shape, pad, stride, dil, padding_value, kernel, dev, **(tune or {}))
    plan.set_weights(wd)
    N, O, OH, OW = plan.out_shape
    if x_layout == "nhwc":
        xin, xl = ops.repack_nchw_to_nhwc(xd), _lib.LAYOUT_NHWC_PAD
    else:
        xin, xl = xd, _lib.LAYOUT_NCHW
    out_acc = torch.full((N, O, OH, OW), -7, dtype=torch.int32, device=dev) if want_acc else None
    f32_nhwc = f32_layout == "nhwc"
    out_f32 = torch.full((N, OH, OW, O) if f32_nhwc else (N, O, OH, OW), float("nan"), dtype=torch.float32, device=dev) if want_f32 else None
    res = None
    if residual is not None:
        r = np.ascontiguousarray(residual.transpose(0, 2, 3, 1)) if f32_nhwc else residual
        res = torch.from_numpy(r).to(dev)
    out_i8 = None
    if rq is not None:
        cp = ops.padded_channels(O)
        out_i8 = torch.full((N, OH, OW, cp) if i8_layout == "nhwc" else (N, O, OH, OW), 99, dtype=torch.int8, device=dev)
    plan.run(xin, xl, torch.from_numpy(dq).to(dev), bias=None if bias is None else torch.from_numpy(bias).to(dev),
             residual=res, activation=ACT[act], leaky=leaky, out_f32=out_f32,
             out_f32_layout=_lib.LAYOUT_NHWC_PAD if f32_nhwc else _lib.LAYOUT_NCHW, out_i8=out_i8,
             out_i8_layout=_lib.LAYOUT_NHWC_PAD if i8_layout == "nhwc" else _lib.LAYOUT_NCHW,
             requant_scales=None if rq is None else list(rq), out_acc=out_acc, residual_after_activation=res_after)
    plan.status()
    torch.cuda.synchronize()
    r = dict(kernel=plan.kernel)
    r["acc"] = out_acc.cpu().numpy() if want_acc else None
    if want_f32:
        f = out_f32.cpu().numpy()
        r["f32"] = f.transpose(0, 3, 1, 2) if f32_nhwc else f
    if out_i8 is not None:
        q = out_i8.cpu().numpy()
        if i8_layout == "nhwc":
            assert not q[..., O:].any(), "padding channels of the NHWC int8 output must be zero"
            q = q[..., :O].transpose(0, 3, 1, 2)
        r["i8"] = q
    return r


def check_case(checker, port, x, w, pad, stride, dil, dq, bias, act, leaky, pv, kernel, **kw):
    want = checker.conv2d_quantized(x, w, pad, stride, dil, dq, pv)
    _, want_acc = port.conv2d_quantized(x, w, pad, stride, dil, dq, pv, return_acc=True)
    yb = checker.add_bias(want, bias) if bias is not None else want
    residual = kw.get("residual")
    if residual is not None and not kw.get("res_after"):
        yb = (yb + residual).astype(np.float32)
    ya = checker.activation(yb, act, leaky)
    if residual is not None and kw.get("res_after"):
        ya = (ya + residual).astype(np.float32)
    got = run_gpu(x, w, pad, stride, dil, dq, bias, act, leaky, pv, kernel, **kw)
    if kw.get("want_acc", True):
        assert np.array_equal(got["acc"], want_acc), "int32 accumulators differ"
    assert same_bits(got["f32"], ya), "fp32 output differs"
    if kw.get("rq") is not None:
        assert np.array_equal(got["i8"], checker.quantize(ya, kw["rq"])), "requantized int8 output differs"
    return got


@pytest.mark.parametrize("kernel", [1, 0])
@pytest.mark.parametrize("name", golden_cases("c_"))
def test_conv_golden(name, kernel):
    """Fixtures produced by the reference's compiled operators."""
    g = load_golden(name)
    got = run_gpu(g["x"], g["w"], g["pad"], g["stride"], g["dilation"], g["dq"], g["bias"], str(g["act"]),
                  float(g["leaky"]), float(g["padding_value"]), kernel, rq=g["rq"])
    assert same_bits(got["f32"], g["y_act"])
    assert np.array_equal(got["i8"], g["y_q"])
    plain = run_gpu(g["x"], g["w"], g["pad"], g["stride"], g["dilation"], g["dq"], None, "none", 0.0,
                    float(g["padding_value"]), kernel)
    assert same_bits(plain["f32"], g["y_conv"])


# N, C, H, W, O, KH, KW, pad(t,b,l,r), stride, dilation
TC_CASES = [
    (1, 64, 8, 8, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),
    (2, 64, 9, 11, 40, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),          # O not a multiple of 8/16, odd extents
    (3, 128, 7, 7, 64, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),          # 1x1, K block of 128
    (2, 128, 14, 14, 256, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),       # stride 2
    (1, 64, 15, 13, 96, 3, 3, (2, 0, 1, 3), (2, 1), (2, 2)),         # asymmetric padding, dilation, mixed stride
    (2, 70, 10, 10, 130, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),        # channels padded 70 -> 128
    (1, 192, 6, 6, 300, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1)),         # 1x1 stride 2, two N tiles
    (5, 64, 12, 12, 64, 5, 5, (2, 2, 2, 2), (1, 1), (1, 1)),         # 5x5, several M tiles crossing images
    (2, 256, 5, 5, 512, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),         # deep K, wide N
    (1, 64, 3, 3, 16, 3, 3, (0, 0, 0, 0), (1, 1), (1, 1)),           # single output pixel
    (1, 64, 40, 40, 64, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),         # 7x7 stride 2
    # at most 16 input channels: the filter row is folded into the K dimension
    (2, 3, 15, 17, 6, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),           # stem-like, 8 bytes per pixel
    (1, 3, 20, 20, 8, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),           # stride 1: 16 bytes per pixel
    (2, 8, 12, 12, 16, 5, 5, (2, 2, 2, 2), (2, 2), (1, 1)),
    (1, 16, 9, 9, 10, 3, 3, (1, 1, 1, 1), (1, 1), (2, 2)),           # dilation: 128-byte folded row
    (1, 4, 10, 12, 6, 3, 3, (2, 0, 1, 3), (2, 1), (2, 2)),
    (3, 3, 33, 35, 70, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),          # several M tiles, O not a multiple of 64
    (2, 24, 9, 9, 20, 3, 3, (1, 2, 0, 1), (1, 2), (1, 1)),           # 24 channels padded to 64
]


@pytest.mark.parametrize("case", TC_CASES)
def test_tcgen05_kernel_cases(checker, port, case):
    N, C, H, W, O, KH, KW, pad, stride, dil = case
    rng = np.random.default_rng(N * 1000 + C + O)
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    got = check_case(checker, port, x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2)
    assert got["kernel"] == 2
    # NHWC_PAD input, leaky relu, requantize to NHWC_PAD with one scale per sample
    rq = np.full(N, 0.9, dtype=np.float32)
    check_case(checker, port, x, w, pad, stride, dil, dq, bias, "leaky_relu", 0.1, 0.0, 2, x_layout="nhwc", rq=rq,
               i8_layout="nhwc")


@pytest.mark.parametrize("swap", ["1", "0"])
@pytest.mark.parametrize("case", [
    (2, 64, 20, 20, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),      # several 256-pixel tiles, image boundaries inside chunks
    (3, 128, 9, 9, 40, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),       # O not a multiple of 32
    (1, 64, 7, 7, 128, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),       # fewer pixels than one tile
    (5, 64, 12, 12, 96, 5, 5, (2, 2, 2, 2), (1, 1), (1, 1)),
    (2, 3, 33, 35, 16, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),       # folded input
    (4, 192, 14, 14, 100, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),    # 1x1 with tiled activation loads
])
def test_both_mma_orientations(checker, port, case, swap):
    """Layers with at most 128 output channels can run with channels or with pixels on the MMA's M side; the
    library picks one by a heuristic, the test forces each in turn (tsb_conv_desc.mma_orientation)."""
    tune = dict(mma_orientation=2 if swap == "1" else 1)
    N, C, H, W, O, KH, KW, pad, stride, dil = case
    rng = np.random.default_rng(N * 100 + C + O + int(swap))
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    check_case(checker, port, x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, tune=tune)             # fp32 NCHW fast path
    check_case(checker, port, x, w, pad, stride, dil, dq, None, "leaky_relu", 0.1, 0.0, 2, want_acc=False, tune=tune,
               x_layout="nhwc", rq=np.full(N, 0.7, dtype=np.float32), i8_layout="nhwc", f32_layout="nhwc")  # generic path
    got = run_gpu(x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, x_layout="nhwc", rq=np.full(N, 0.7, dtype=np.float32),
                  i8_layout="nhwc", want_acc=False, want_f32=False, tune=tune)                                # int8 NHWC fast path
    want = checker.quantize(checker.relu(checker.add_bias(checker.conv2d_quantized(x, w, pad, stride, dil, dq), bias)), np.full(N, 0.7, np.float32))
    assert np.array_equal(got["i8"], want)


@pytest.mark.parametrize("case", [
    (2, 3, 20, 235, 64, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),     # stem shape, one tile per output row (115 of 128 pixels)
    (1, 3, 12, 300, 32, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),     # two tiles per output row
    (2, 16, 9, 140, 48, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),     # 16 bytes per pixel, stride 1
    (1, 8, 10, 70, 24, 5, 5, (2, 2, 2, 2), (2, 2), (1, 1)),      # short rows
    (1, 4, 11, 64, 16, 3, 3, (0, 2, 1, 0), (2, 2), (2, 1)),      # asymmetric padding, dilated filter rows
    (3, 3, 33, 35, 16, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),
    (1, 3, 6, 260, 300, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),     # two channel tiles: resident weights are reloaded
    (1, 5, 9, 40, 8, 3, 3, (2, 2, 1, 1), (1, 1), (1, 2)),        # two padding rows above, dilated taps inside a row
    (1, 3, 120, 700, 32, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),    # three segments per output row, 180 tiles on 148 CTAs:
                                                                 # CTAs that start in the middle of a row, shared stages
    (2, 3, 50, 390, 24, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),     # 16 bytes per pixel, four segments, 400 tiles
])
def test_raw_row_mode(checker, port, case):
    """Few input channels with a pixel stride of 16 staged bytes: the kernel copies each staged image row once per
    tile and the MMA reads the overlapping windows through a sliding descriptor.  Forced on here for short rows too."""
    tune = dict(raw_row_mode=2)
    N, C, H, W, O, KH, KW, pad, stride, dil = case
    rng = np.random.default_rng(N * 77 + C + O + W)
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    got = check_case(checker, port, x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, tune=tune)
    assert got["kernel"] == 2
    rq = np.full(N, 0.7, dtype=np.float32)
    check_case(checker, port, x, w, pad, stride, dil, dq, None, "leaky_relu", 0.1, 0.0, 2, want_acc=False, tune=tune,
               x_layout="nhwc", rq=rq, i8_layout="nhwc", f32_layout="nhwc")
    got = run_gpu(x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, x_layout="nhwc", rq=rq, i8_layout="nhwc",
                  want_acc=False, want_f32=False, tune=tune)
    want = checker.quantize(checker.relu(checker.add_bias(checker.conv2d_quantized(x, w, pad, stride, dil, dq), bias)), rq)
    assert np.array_equal(got["i8"], want)


@pytest.mark.parametrize("swap", ["0", "1"])
@pytest.mark.parametrize("case", [
    (2, 64, 20, 20, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),      # image edges inside tiles on both axes
    (1, 128, 56, 56, 128, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),    # many tiles per image, 128-byte channel blocks
    (3, 192, 14, 14, 96, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),     # three 64-byte channel blocks, one tile per image
    (2, 256, 9, 17, 40, 3, 3, (1, 1, 1, 1), (1, 1), (2, 2)),      # dilated taps, ragged channels
    (2, 64, 12, 12, 72, 5, 5, (2, 2, 2, 2), (1, 1), (1, 1)),      # 25 taps
    (1, 64, 10, 30, 32, 3, 1, (1, 1, 0, 0), (1, 1), (1, 1)),      # a column filter
    (2, 64, 11, 13, 64, 2, 3, (0, 1, 2, 0), (1, 1), (1, 1)),      # asymmetric padding, even filter height
])
def test_patch_mode(checker, port, case, swap):
    """Stride-1 filters with several taps: one tensor-map load brings the input patch under an 8-pixel-wide tile and
    every tap reads its window out of it through a shifted shared-memory descriptor.  Forced on here regardless of how
    well the tiles cover the image, in both MMA orientations."""
    tune = dict(patch_mode=2, mma_orientation=2 if swap == "1" else 1)
    N, C, H, W, O, KH, KW, pad, stride, dil = case
    rng = np.random.default_rng(N * 13 + C + O + H)
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    got = check_case(checker, port, x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, tune=tune)    # fp32 NCHW
    assert got["kernel"] == 2
    rq = rng.uniform(0.5, 2.0, size=N).astype(np.float32)
    check_case(checker, port, x, w, pad, stride, dil, dq, None, "leaky_relu", 0.1, 0.0, 2, want_acc=False, tune=tune,
               x_layout="nhwc", rq=rq, i8_layout="nhwc", f32_layout="nhwc")                                # element by element
    got = run_gpu(x, w, pad, stride, dil, dq, bias, "relu", 0.0, 0.0, 2, x_layout="nhwc", rq=rq, i8_layout="nhwc",
                  want_acc=False, want_f32=False, tune=tune)                                               # int8 NHWC
    want = checker.quantize(checker.relu(checker.add_bias(checker.conv2d_quantized(x, w, pad, stride, dil, dq), bias)), rq)
    assert np.array_equal(got["i8"], want)


@pytest.mark.parametrize("swap", [None, "0", "1"])
@pytest.mark.parametrize("case", [
    (5, 64, 7, 7, 256),      # 49 pixels per image: most 32-pixel chunks cross an image boundary
    (3, 128, 14, 14, 160),   # 196 pixels per image
    (4, 64, 5, 5, 64),       # fewer than 32 pixels per image: several boundaries in one chunk
])
def test_residual_tail_pixel_major_with_per_sample_scales(checker, port, case, swap):
    """1x1 convolution + residual + relu with pixel-major fp32 in/out and a fused requantize whose scale differs from
    sample to sample: a chunk of 32 pixels that crosses an image boundary must switch scales at the boundary."""
    tune = dict(mma_orientation=0 if swap is None else (2 if swap == "1" else 1))
    N, C, H, W, O = case
    rng = np.random.default_rng(N * 31 + O)
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, 1, 1), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    residual = rng.standard_normal((N, O, H, W)).astype(np.float32)
    rq = rng.uniform(0.5, 4.0, size=N).astype(np.float32)
    check_case(checker, port, x, w, (0, 0, 0, 0), (1, 1), (1, 1), dq, bias, "relu", 0.0, 0.0, 2, want_acc=False, tune=tune,
               x_layout="nhwc", residual=residual, rq=rq, f32_layout="nhwc", i8_layout="nhwc")
    check_case(checker, port, x, w, (0, 0, 0, 0), (1, 1), (1, 1), dq, bias, "none", 0.0, 0.0, 2, want_acc=False, tune=tune,
               x_layout="nhwc", rq=rq, f32_layout="nchw", i8_layout="nhwc")


@pytest.mark.parametrize("case", [
    (2, 3, 15, 17, 6, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), 0.0),
    (1, 5, 6, 6, 3, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 3.0),
    (2, 24, 9, 9, 20, 3, 3, (1, 2, 0, 1), (1, 2), (1, 1), -2.7),
    (1, 64, 8, 8, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0),
    (1, 600, 4, 4, 9, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0),       # weight tile staged in several channel chunks
])
def test_direct_kernel_cases(checker, port, case):
    N, C, H, W, O, KH, KW, pad, stride, dil, pv = case
    rng = np.random.default_rng(C * 7 + O)
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    rq = np.full(N, 1.3, dtype=np.float32)
    check_case(checker, port, x, w, pad, stride, dil, dq, bias, "relu", 0.0, pv, 1, rq=rq)
    check_case(checker, port, x, w, pad, stride, dil, dq, None, "none", 0.0, pv, 1, x_layout="nhwc", rq=rq, i8_layout="nhwc")


@pytest.mark.parametrize("kernel", [1, 2])
def test_epilogue_variants(checker, port, kernel):
    rng = np.random.default_rng(99)
    N, C, H, W, O = 1, 64, 10, 10, 72
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, 3, 3), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    residual = rng.standard_normal((N, O, H, W)).astype(np.float32)
    args = (x, w, (1, 1, 1, 1), (1, 1), (1, 1), dq)
    # batch 1 + one requantize scale: half-to-even body and half-away tail on the NCHW index (7200 = 900*8, so
    # use a scale that produces ties: outputs are multiples of dq, force exact .5 via a power-of-two scale)
    for f32_layout in ("nchw", "nhwc"):
        for i8_layout in ("nchw", "nhwc"):
            check_case(checker, port, *args, bias, "relu", 0.0, 0.0, kernel, residual=residual, rq=np.array([8.0], np.float32),
                       f32_layout=f32_layout, i8_layout=i8_layout)
    check_case(checker, port, *args, None, "leaky_relu", 0.25, 0.0, kernel, rq=np.array([0.5], np.float32))


@pytest.mark.parametrize("tune", [dict(), dict(mma_orientation=1), dict(mma_orientation=2), dict(patch_mode=1)])
def test_nchw_residual_with_nchw_output(checker, port, tune):
    """What the graph rewrite produces when it folds a shortcut into the convolution: fp32 NCHW residual in, fp32 NCHW
    out, no int8 output -- residual before the activation (ResNet) and after it (Darknet)."""
    rng = np.random.default_rng(11)
    N, C, H, W, O = 2, 64, 13, 11, 160
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    residual = rng.standard_normal((N, O, H, W)).astype(np.float32)
    for k, pad in ((1, (0, 0, 0, 0)), (3, (1, 1, 1, 1))):
        w = rng.integers(-127, 128, size=(O, C, k, k), dtype=np.int8)
        check_case(checker, port, x, w, pad, (1, 1), (1, 1), dq, bias, "relu", 0.0, 0.0, 2, residual=residual, want_acc=False, tune=tune)
        check_case(checker, port, x, w, pad, (1, 1), (1, 1), dq, bias, "leaky_relu", 0.1, 0.0, 2, residual=residual, res_after=True,
                   want_acc=False, x_layout="nhwc", tune=tune)


@pytest.mark.parametrize("kernel", [1, 2])
@pytest.mark.parametrize("swap", [None, "0", "1"])
def test_residual_after_the_activation(checker, port, kernel, swap):
    """A Darknet shortcut: leaky_relu(conv + bias) + residual, every output layout, both kernels and orientations."""
    tune = dict(mma_orientation=0 if swap is None else (2 if swap == "1" else 1))
    rng = np.random.default_rng(7)
    N, C, H, W, O = 2, 64, 12, 12, 96
    x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(O, C, 3, 3), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    residual = rng.standard_normal((N, O, H, W)).astype(np.float32)
    rq = rng.uniform(0.5, 2.0, size=N).astype(np.float32)
    args = (x, w, (1, 1, 1, 1), (1, 1), (1, 1), dq)
    for f32_layout, i8_layout in (("nhwc", "nhwc"), ("nchw", "nhwc"), ("nchw", "nchw")):
        check_case(checker, port, *args, bias, "leaky_relu", 0.1, 0.0, kernel, residual=residual, rq=rq, res_after=True,
                   x_layout="nhwc", f32_layout=f32_layout, i8_layout=i8_layout, want_acc=False, tune=tune)
    w1 = rng.integers(-127, 128, size=(O, C, 1, 1), dtype=np.int8)
    check_case(checker, port, x, w1, (0, 0, 0, 0), (1, 1), (1, 1), dq, bias, "relu", 0.0, 0.0, kernel, residual=residual, rq=rq,
               res_after=True, x_layout="nhwc", f32_layout="nhwc", i8_layout="nhwc", want_acc=False, tune=tune)


def test_concat_of_two_int8_tensors():
    from tennis_b200 import _lib, ops
    lib = _lib.load()
    rng = np.random.default_rng(3)
    for ca, cb in ((64, 64), (128, 64), (32, 48), (20, 7)):
        px = 2 * 5 * 7
        a = np.zeros((px, ops.padded_channels(ca)), dtype=np.int8); a[:, :ca] = rng.integers(-128, 128, size=(px, ca))
        b = np.zeros((px, ops.padded_channels(cb)), dtype=np.int8); b[:, :cb] = rng.integers(-128, 128, size=(px, cb))
        ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        y = torch.full((px, ops.padded_channels(ca + cb)), 99, dtype=torch.int8, device="cuda")
        _lib.check(lib.tsb_concat_i8_nhwc(ad.data_ptr(), ca, bd.data_ptr(), cb, y.data_ptr(), px, ops._stream_ptr()))
        got = y.cpu().numpy()
        assert np.array_equal(got[:, :ca], a[:, :ca]) and np.array_equal(got[:, ca:ca + cb], b[:, :cb])
        assert not got[:, ca + cb:].any()


def test_rounding_ties_in_fused_requantize(checker, port):
    """dq = 0.5 and integer accumulators give outputs that are exact multiples of 0.5: every other value is a tie."""
    rng = np.random.default_rng(1)
    for N in (1, 2):
        x = rng.integers(-3, 4, size=(N, 64, 5, 5), dtype=np.int8)
        w = rng.integers(-1, 2, size=(19, 64, 1, 1), dtype=np.int8)
        dq = np.full(19, 0.5, dtype=np.float32)
        rq = np.full(N, 1.0, dtype=np.float32)
        for kernel in (1, 2):
            got = check_case(checker, port, x, w, (0, 0, 0, 0), (1, 1), (1, 1), dq, None, "none", 0.0, 0.0, kernel, rq=rq)
            assert (np.abs(got["f32"] * 2) % 2 == 1).any(), "the case must contain ties"


def test_operator_mirror_runs_like_the_reference_operator(checker):
    from tennis_b200 import ops
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 64, 12, 12)).astype(np.float32)
    s = np.float32(127.0) / np.abs(x).max()
    w = rng.integers(-127, 128, size=(32, 64, 3, 3), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=32).astype(np.float32)
    q = ops.Quantize()
    q.set("quantize_scale", np.array([s, s], np.float32))
    q.init()
    conv = ops.Conv2DQuantized()
    conv.set("format", "NCHW")
    conv.set("padding", np.array([[0, 0], [0, 0], [1, 1], [1, 1]]))
    conv.set("stride", np.array([1, 1, 1, 1]))
    conv.set("dialations", np.array([1, 1, 1, 1]))
    conv.set("dequantize_scales", dq)
    conv.init()
    xq = q.run([torch.from_numpy(x).cuda()])
    y = conv.run([xq, torch.from_numpy(w).cuda()])
    want_q = checker.quantize(x, [s, s])
    assert np.array_equal(xq.cpu().numpy(), want_q)
    assert same_bits(y.cpu().numpy(), checker.conv2d_quantized(want_q, w, (1, 1, 1, 1), (1, 1), (1, 1), dq))
    y2 = conv.run([xq, torch.from_numpy(w).cuda()])  # second run reuses the plan
    assert torch.equal(y, y2)


@pytest.mark.parametrize("case", [
    (2, 64, 9, 9, 40, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0),      # tensor cores, NHWC_PAD staging
    (2, 3, 15, 17, 6, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), 0.0),      # tensor cores, folded staging, 8 bytes per pixel
    (1, 5, 11, 12, 7, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 0.0),      # folded staging, 16 bytes per pixel
    (3, 70, 6, 6, 9, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 0.0),       # channels padded 70 -> 128
    (2, 5, 6, 6, 3, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 3.0),        # direct kernel (padding_value)
])
def test_quantize_into_the_plan_then_run_staged(checker, case):
    """fp32 input -> tsb_conv2d_i8_quantize_input -> run(TSB_LAYOUT_STAGED) equals quantize + conv2d_quantized."""
    from tennis_b200 import _lib, ops
    N, C, H, W, O, KH, KW, pad, stride, dil, pv = case
    rng = np.random.default_rng(C + 17 * O)
    x = (rng.standard_normal((N, C, H, W)) * 50).astype(np.float32)
    x.reshape(-1)[::7] = np.round(x.reshape(-1)[::7]) + 0.5   # ties
    # values the fast rounding forms must hand to the exact one: NaN, infinities, products beyond int32 (all -128 on the
    # reference's CPU), and plain saturation
    special = np.array([np.nan, np.inf, -np.inf, 3e9, -3e9, 300.0, -300.0, 127.5, -128.5], dtype=np.float32)
    where = rng.permutation(x.size)[:special.size]
    x.reshape(-1)[where] = special
    w = rng.integers(-127, 128, size=(O, C, KH, KW), dtype=np.int8)
    dq = rng.uniform(0.001, 0.01, size=O).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.1).astype(np.float32)
    for scales in ([1.0] * N, list(rng.uniform(0.5, 2.0, size=N))):
        xq = checker.quantize(x, scales)
        want = checker.conv_block(xq, w, pad, stride, dil, dq, bias, act="relu", padding_value=pv)
        plan = ops.ConvPlan(x.shape, w.shape, pad, stride, dil, pv)
        plan.set_weights(torch.from_numpy(w).cuda())
        plan.quantize_input(torch.from_numpy(x).cuda(), [float(v) for v in scales])
        out = torch.empty(plan.out_shape, dtype=torch.float32, device="cuda")
        plan.run(None, _lib.LAYOUT_STAGED, torch.from_numpy(dq).cuda(), bias=torch.from_numpy(bias).cuda(),
                 activation=_lib.ACT_RELU, out_f32=out)
        plan.status()
        assert same_bits(out.cpu().numpy(), want)


def test_host_buffer_entry_point(checker):
    import ctypes
    from tennis_b200 import _lib, ops, workloads
    layer = workloads.conv_layer("t", 2, 64, 10, 10, 48, 3, 1, 1)
    d = workloads.make_layer_data(layer, seed=3)
    plan = ops.ConvPlan((2, 64, 10, 10), (48, 64, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1))
    lib = _lib.load()
    nbytes = lib.tsb_conv2d_host_scratch_bytes(plan.handle)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = np.zeros(plan.out_shape, dtype=np.float32)
    scales = [float(d["qscale"])] * 2
    for resident in (0, 1):
        out[:] = 0
        _lib.check(lib.tsb_conv2d_quantized_host(
            plan.handle, d["x"].ctypes.data, _lib.float_array(scales), 2, d["w"].ctypes.data, d["dq"].ctypes.data,
            d["bias"].ctypes.data, _lib.ACT_RELU, 0.0, out.ctypes.data, scratch.data_ptr(), nbytes, resident,
            ops._stream_ptr()))
        xq = checker.quantize(d["x"], scales)
        want = checker.conv_block(xq, d["w"], (1, 1, 1, 1), (1, 1), (1, 1), d["dq"], d["bias"], act="relu")
        assert same_bits(out, want)


def test_host_buffer_entry_point_async_on_two_streams(checker):
    """Two layers enqueued with the non-waiting host call on two streams; results are read after both streams are
    synchronised."""
    from tennis_b200 import _lib, ops, workloads
    lib = _lib.load()
    jobs = []
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for i, (c, o, k) in enumerate([(64, 48, 3), (128, 96, 1)]):
        layer = workloads.conv_layer("t", 3, c, 12, 12, o, k, 1, k // 2)
        d = workloads.make_layer_data(layer, seed=5 + i)
        plan = ops.ConvPlan((3, c, 12, 12), (o, c, k, k), (k // 2,) * 4, (1, 1), (1, 1))
        nbytes = lib.tsb_conv2d_host_scratch_bytes(plan.handle)
        jobs.append(dict(d=d, plan=plan, nbytes=nbytes, k=k, scratch=torch.empty(nbytes, dtype=torch.uint8, device="cuda"),
                         x=torch.from_numpy(d["x"]).pin_memory(), out=torch.zeros(plan.out_shape, dtype=torch.float32).pin_memory(),
                         scales=_lib.float_array([float(d["qscale"])] * 3)))
    torch.cuda.synchronize()
    for j, st in zip(jobs, streams):
        d = j["d"]
        _lib.check(lib.tsb_conv2d_quantized_host_async(
            j["plan"].handle, j["x"].data_ptr(), j["scales"], 3, d["w"].ctypes.data, d["dq"].ctypes.data, d["bias"].ctypes.data,
            _lib.ACT_RELU, 0.0, j["out"].data_ptr(), j["scratch"].data_ptr(), j["nbytes"], 0, st.cuda_stream))
    for st in streams:
        st.synchronize()
    for j in jobs:
        d = j["d"]
        xq = checker.quantize(d["x"], [float(d["qscale"])] * 3)
        want = checker.conv_block(xq, d["w"], (j["k"] // 2,) * 4, (1, 1), (1, 1), d["dq"], d["bias"], act="relu")
        assert same_bits(j["out"].numpy(), want)


def test_run_without_weights_is_rejected():
    from tennis_b200 import _lib, ops
    plan = ops.ConvPlan((1, 64, 8, 8), (64, 64, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1))
    x = torch.zeros((1, 64, 8, 8), dtype=torch.int8, device="cuda")
    dq = torch.ones(64, device="cuda")
    out = torch.zeros(plan.out_shape, device="cuda")
    with pytest.raises(_lib.TsbError, match="set_weights"):
        plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
    plan.set_weights(torch.zeros((64, 64, 3, 3), dtype=torch.int8, device="cuda"))
    with pytest.raises(_lib.TsbError, match="no output requested"):
        plan.run(x, _lib.LAYOUT_NCHW, dq)
