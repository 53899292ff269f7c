"""A small bottleneck ResNet (same topology code as the ResNet-50-shaped benchmark network) through the fused int8
path, against the CPU checker running the TenniS operator sequence layer by layer:
quantize -> conv2d_quantized -> add_bias -> [add] -> relu, max pooling on fp32 before the next quantize."""
import numpy as np
import pytest
import torch

from conftest import same_bits

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
    """The network as a chain of reference operators.  Returns (int8 block outputs, fp32 last block output, logits)."""
    from tennis_b200 import nets
    n = x.shape[0]
    convs, P = spec["convs"], params["convs"]

    def block(idx, xq, act, residual=None, requant=True):
        c, p = convs[idx], P[idx]
        s_in, s_out = scales["convs"][idx]
        dq = nets.dequantize_scales(p["sw"], scales["bn"][idx], s_in)
        rq = [float(s_out)] * n if requant else None
        return chk.conv_block(xq, p["w"], (c["pad"],) * 4, (c["stride"],) * 2, (1, 1), dq, p["bias"], act=act,
                              residual=residual, requant_scales=rq)

    xq = chk.quantize(x, [float(scales["input"])] * n)
    y, _ = block(0, xq, "relu")
    pooled = maxpool_f32(y)
    x_i8 = chk.quantize(pooled, [float(scales["convs"][0][1])] * n)
    x_f32, outs = None, []
    for stage in spec["stages"]:
        for b in stage:
            _, a = block(b["conv1"], x_i8, "relu")
            _, bb = block(b["conv2"], a, "relu")
            sc = block(b["proj"], x_i8, "none", requant=False) if b["projection"] else x_f32
            x_f32, x_i8 = block(b["conv3"], bb, "relu", residual=sc)
            outs.append(x_i8)
    feat = x_f32.reshape(n, x_f32.shape[1], -1).mean(axis=2, dtype=np.float64).astype(np.float32)
    logits = (feat.astype(np.float64) @ params["fc_w"].T.astype(np.float64) + params["fc_b"]).astype(np.float32)
    return outs, x_f32, logits


def test_small_resnet_matches_the_operator_chain(checker):
    from tennis_b200 import nets
    spec = nets.resnet_spec(image=64, widths=(64, 128), blocks=(2, 1), classes=10)
    assert len(spec["convs"]) == 1 + (2 * 3 + 1) + (3 + 1)
    params = nets.make_params(spec, seed=1)
    n = 2
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, 3, 64, 64), dtype=np.float32)
    net = nets.QuantResNet(spec, params, n)
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
    y = torch.empty((2, 5, 6, 64), dtype=torch.int8, device="cuda")
    _lib.check(lib.tsb_maxpool_i8_nhwc(xd.data_ptr(), y.data_ptr(), 2, 9, 11, 64, 3, 2, 1, ops._stream_ptr()))
    want = maxpool_f32(x.transpose(0, 3, 1, 2).astype(np.float32)).transpose(0, 2, 3, 1).astype(np.int8)
    assert np.array_equal(y.cpu().numpy(), want)
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
