"""A small bottleneck ResNet (same topology code as the ResNet-50-shaped benchmark network) through the fused int8
path, against the CPU checker running the TenniS operator sequence layer by layer:
quantize -> conv2d_quantized -> add_bias -> [add] -> relu, max pooling on fp32 before the next quantize."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden, same_bits

pytestmark = pytest.mark.gpu


def maxpool_f32(x, k=3, s=2, p=1):
    n, c, h, w = x.shape
    oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    xp = np.full((n, c, h + 2 * p, w + 2 * p), -np.inf, dtype=np.float32)
    xp[:, :, p:p + h, p:p + w] = x
    out = np.full((n, c, oh, ow), -np.inf, dtype=np.float32)
    for i in range(k):
        for j in range(k):
            out = np.maximum(out, xp[:, :, i:i + s * oh:s, j:j + s * ow:s])
    return out


def reference_forward(spec, params, scales, x, chk):
    """The network as a chain of reference operators (oracle/chains.py); the stem pool is also checked against a plain
    numpy floor-mode pooling, which the graph's padding {1,0,1,0} under the ceil-mode extent must equal."""
    from oracle import chains
    return chains.resnet_forward(spec, params, scales, x, chk)


@pytest.mark.parametrize("fuse_projection", [True, False])
def test_small_resnet_matches_the_operator_chain(checker, fuse_projection):
    """fuse_projection: the projection shortcuts inside the launch of the blocks' last convolution, or on their own."""
    from tennis_b200 import nets
    spec = nets.resnet_spec(image=64, widths=(64, 128), blocks=(2, 1), classes=10)
    assert len(spec["convs"]) == 1 + (2 * 3 + 1) + (3 + 1)
    params = nets.make_params(spec, seed=1)
    n = 2
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, 3, 64, 64), dtype=np.float32)
    net = nets.QuantResNet(spec, params, n, fuse_projection=fuse_projection)
    xd = torch.from_numpy(x).cuda()
    scales = net.calibrate(xd)
    logits = net.forward(xd).clone()
    net.status()
    torch.cuda.synchronize()
    outs, last_f32, want_logits = reference_forward(spec, params, scales, x, checker)
    # int8 activations after every block: bit-exact
    k = 0
    for stage in spec["stages"]:
        for b in stage:
            got = net.buffers[b["name"] + ".y.i8"].cpu().numpy()
            o = spec["convs"][b["conv3"]]["o"]
            assert np.array_equal(got[..., :o].transpose(0, 3, 1, 2), outs[k]), b["name"]
            k += 1
    last = net.buffers[spec["stages"][-1][-1]["name"] + ".y.f32"].cpu().numpy().transpose(0, 3, 1, 2)
    assert same_bits(last, last_f32)
    # the two fp32 reductions sum in another order than numpy: rounding-level agreement
    np.testing.assert_allclose(logits.cpu().numpy(), want_logits, rtol=1e-5, atol=1e-5 * np.abs(want_logits).max())

    # the same forward pass captured in a CUDA graph replays to the same bits
    static_x = xd.clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        net.forward(static_x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = net.forward(static_x)
    torch.cuda.current_stream().wait_stream(stream)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, logits)


@pytest.mark.parametrize("name", golden_cases("p_"))
def test_max_pooling_golden(name):
    """pooling2d fixtures made by the reference's operator: quantize(pool(x)) == pool(quantize(x)) for the int8 kernel."""
    from tennis_b200 import _lib, ops
    lib = _lib.load()
    g = load_golden(name)
    x, k, st, pad = g["x"], int(g["k"]), int(g["stride"]), [int(v) for v in g["pad"]]
    n, c, h, w = x.shape
    scale = [float(127.0 / np.abs(x).max())] * n
    xq = ops.quantize_nchw_to_nhwc(torch.from_numpy(x).cuda(), scale)
    oh, ow = g["y"].shape[2:]
    assert (oh, ow) == (lib.tsb_pool_out_dim(h, pad[0], pad[1], k, st), lib.tsb_pool_out_dim(w, pad[2], pad[3], k, st))
    y = torch.zeros((n, oh, ow, xq.shape[3]), dtype=torch.int8, device="cuda")
    _lib.check(lib.tsb_maxpool_i8_nhwc(xq.data_ptr(), y.data_ptr(), n, h, w, c, k, st, *pad, ops._stream_ptr()))
    want = ops.quantize_nchw_to_nhwc(torch.from_numpy(g["y"]).cuda(), scale)
    assert torch.equal(y, want)


def test_full_size_resnet50_first_and_last_image(port):
    """Configuration 2 at its full size (ResNet-50-shaped, batch 64, 224 x 224): the first and the last image of the
    batch against the operator chain run on those two images alone.  Every scale is per sample, so a slice of the batch
    is exact -- as long as the slice keeps more than one sample (a batch of one takes the operator's one-scale rounding)."""
    from tennis_b200 import nets
    spec = nets.resnet_spec()
    params = nets.make_params(spec, seed=0)
    n = 64
    g = torch.Generator(device="cuda").manual_seed(0)
    xd = torch.randn((n, 3, 224, 224), device="cuda", generator=g)
    net = nets.QuantResNet(spec, params, n)
    scales = net.calibrate(xd)
    logits = net.forward(xd).clone()
    net.status()
    torch.cuda.synchronize()
    pick = [0, n - 1]
    outs, last_f32, want_logits = reference_forward(spec, params, scales, xd[pick].cpu().numpy(), port)
    k = 0
    for stage in spec["stages"]:
        for b in stage:
            got = net.buffers[b["name"] + ".y.i8"][pick].cpu().numpy()
            o = spec["convs"][b["conv3"]]["o"]
            assert np.array_equal(got[..., :o].transpose(0, 3, 1, 2), outs[k]), b["name"]
            assert not got[..., o:].any()
            k += 1
    last = net.buffers[spec["stages"][-1][-1]["name"] + ".y.f32"][pick].cpu().numpy().transpose(0, 3, 1, 2)
    assert same_bits(last, last_f32)
    np.testing.assert_allclose(logits[pick].cpu().numpy(), want_logits, rtol=1e-5, atol=1e-5 * np.abs(want_logits).max())


def test_resnet50_topology():
    from tennis_b200 import nets
    spec = nets.resnet_spec()
    assert len(spec["convs"]) == 53 and spec["features"] == 2048 and spec["final_size"] == 7
    assert abs(nets.conv_ops(spec, 1) / 1e9 - 8.2) < 0.4   # ~4.1 GMAC per image


def test_pool_and_inner_product_kernels(checker):
    from tennis_b200 import _lib, ops
    lib = _lib.load()
    rng = np.random.default_rng(2)
    x = rng.integers(-128, 128, size=(2, 9, 11, 64), dtype=np.int8)
    xd = torch.from_numpy(x).cuda()
    # the reference's pooling2d: ceil-mode extent, windows clipped to the image
    for (k, st, pad) in ((3, 2, (1, 1, 1, 1)), (3, 2, (1, 0, 1, 0)), (2, 2, (0, 0, 0, 0)), (3, 1, (1, 1, 1, 1)), (5, 3, (2, 2, 2, 1))):
        want = checker.max_pooling2d(x.transpose(0, 3, 1, 2).astype(np.float32), k, st, pad)
        oh, ow = lib.tsb_pool_out_dim(9, pad[0], pad[1], k, st), lib.tsb_pool_out_dim(11, pad[2], pad[3], k, st)
        assert want.shape == (2, 64, oh, ow)
        y = torch.full((2, oh, ow, 64), 99, dtype=torch.int8, device="cuda")
        _lib.check(lib.tsb_maxpool_i8_nhwc(xd.data_ptr(), y.data_ptr(), 2, 9, 11, 64, k, st, *pad, ops._stream_ptr()))
        assert np.array_equal(y.cpu().numpy(), want.transpose(0, 2, 3, 1).astype(np.int8)), (k, st, pad)
    f = rng.standard_normal((3, 49, 40)).astype(np.float32)
    fd = torch.from_numpy(f).cuda()
    g = torch.empty((3, 40), device="cuda")
    _lib.check(lib.tsb_global_avgpool_f32_nhwc(fd.data_ptr(), g.data_ptr(), 3, 49, 40, ops._stream_ptr()))
    np.testing.assert_allclose(g.cpu().numpy(), f.mean(axis=1), rtol=1e-5, atol=1e-6)
    w = rng.standard_normal((7, 40)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    out = torch.empty((3, 7), device="cuda")
    wd, bd = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    _lib.check(lib.tsb_inner_prod_f32(g.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(), 3, 40, 7, ops._stream_ptr()))
    np.testing.assert_allclose(out.cpu().numpy(), g.cpu().numpy() @ w.T + b, rtol=1e-5, atol=1e-5)
