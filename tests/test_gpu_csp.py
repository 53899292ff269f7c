"""A small CSPDarknet-shaped backbone (same topology code as the CSPDarknet53-shaped configuration) through the fused
int8 path, against the CPU checker running the TenniS operator sequence layer by layer:
quantize -> conv2d_quantized -> add_bias -> leaky_relu [-> add] and concat on dim 1 before the next quantize."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference_forward(spec, params, scales, x, chk):
    from oracle import chains
    from tennis_b200 import nets
    return chains.cspdarknet_forward(spec, params, scales, x, chk, leaky=nets.LEAKY)


@pytest.mark.parametrize("fuse_concat", [True, False])
def test_small_cspdarknet_matches_the_operator_chain(checker, fuse_concat):
    """fuse_concat: the transition convolutions read their two halves directly, or an int8 concatenation runs first."""
    from tennis_b200 import nets
    spec = nets.cspdarknet_spec(image=64, widths=(64, 128), blocks=(1, 2))
    assert len(spec["convs"]) == 1 + (5 + 2 * 1) + (5 + 2 * 2)
    params = nets.make_conv_params(spec, seed=4)
    n = 2
    rng = np.random.default_rng(1)
    x = rng.random((n, 3, 64, 64), dtype=np.float32)
    net = nets.QuantCSPDarknet(spec, params, n, fuse_concat=fuse_concat)
    xd = torch.from_numpy(x).cuda()
    scales = net.calibrate(xd)
    out = net.forward(xd).clone()
    net.status()
    torch.cuda.synchronize()
    outs, last = reference_forward(spec, params, scales, x, checker)
    for st in spec["stages"]:
        for b in st["blocks"]:
            got = net.buffers[b["name"] + ".y.i8"].cpu().numpy()
            o = spec["convs"][b["conv2"]]["o"]
            assert np.array_equal(got[..., :o].transpose(0, 3, 1, 2), outs[b["name"]]), b["name"]
        got = net.buffers[st["name"] + ".out.i8"].cpu().numpy()
        assert np.array_equal(got[..., :st["width"]].transpose(0, 3, 1, 2), outs[st["name"]]), st["name"]
    assert np.array_equal(out.cpu().numpy()[..., :spec["features"]].transpose(0, 3, 1, 2), last)

    # replayed from a CUDA graph: same bits
    static_x = xd.clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        net.forward(static_x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            res = net.forward(static_x)
    torch.cuda.current_stream().wait_stream(stream)
    res.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(res, out)


def test_full_size_cspdarknet53_first_and_last_image(port):
    """Configuration 3 at its full size (CSPDarknet53-shaped, batch 16 at 608 x 608): the first and the last image of
    the batch against the operator chain run on those two images alone (per-sample scales make the slice exact)."""
    from tennis_b200 import nets
    spec = nets.cspdarknet_spec()
    params = nets.make_conv_params(spec, seed=0)
    n = 16
    g = torch.Generator(device="cuda").manual_seed(0)
    xd = torch.rand((n, 3, 608, 608), device="cuda", generator=g)
    net = nets.QuantCSPDarknet(spec, params, n)
    scales = net.calibrate(xd)
    out = net.forward(xd).clone()
    net.status()
    torch.cuda.synchronize()
    pick = [0, n - 1]
    outs, last = reference_forward(spec, params, scales, xd[pick].cpu().numpy(), port)
    for st in spec["stages"]:
        for b in st["blocks"]:
            got = net.buffers[b["name"] + ".y.i8"][pick].cpu().numpy()
            o = spec["convs"][b["conv2"]]["o"]
            assert np.array_equal(got[..., :o].transpose(0, 3, 1, 2), outs[b["name"]]), b["name"]
        got = net.buffers[st["name"] + ".out.i8"][pick].cpu().numpy()
        assert np.array_equal(got[..., :st["width"]].transpose(0, 3, 1, 2), outs[st["name"]]), st["name"]
    assert np.array_equal(out[pick].cpu().numpy()[..., :spec["features"]].transpose(0, 3, 1, 2), last)


def test_cspdarknet53_topology():
    from tennis_b200 import nets
    spec = nets.cspdarknet_spec()
    assert len(spec["convs"]) == 72 and spec["final_size"] == 19 and spec["features"] == 1024
    assert sum(1 for c in spec["convs"] if c["k"] == 3) == 1 + 5 + 23
