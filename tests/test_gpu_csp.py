"""A small CSPDarknet-shaped backbone (same topology code as the CSPDarknet53-shaped configuration) through the fused
int8 path, against the CPU checker running the TenniS operator sequence layer by layer:
quantize -> conv2d_quantized -> add_bias -> leaky_relu [-> add] and concat on dim 1 before the next quantize."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference_forward(spec, params, scales, x, chk):
    from tennis_b200 import nets
    n = x.shape[0]
    convs, P = spec["convs"], params["convs"]

    def block(idx, xq, residual=None):
        c, p = convs[idx], P[idx]
        s_in, s_out = scales["convs"][idx]
        dq = nets.dequantize_scales(p["sw"], scales["bn"][idx], s_in)
        return chk.conv_block(xq, p["w"], (c["pad"],) * 4, (c["stride"],) * 2, (1, 1), dq, p["bias"], act="leaky_relu",
                              leaky=nets.LEAKY, residual=residual, requant_scales=[float(s_out)] * n,
                              residual_after_activation=residual is not None)

    outs = {}
    xq = chk.quantize(x, [float(scales["input"])] * n)
    _, cur = block(spec["stem"], xq)
    for st in spec["stages"]:
        _, cur = block(st["down"], cur)
        xb_f, xb_q = block(st["route_b"], cur)
        for b in st["blocks"]:
            _, h = block(b["conv1"], xb_q)
            xb_f, xb_q = block(b["conv2"], h, residual=xb_f)
            outs[b["name"]] = xb_q
        _, post = block(st["post"], xb_q)
        _, ra = block(st["route_a"], cur)
        # concat of the fp32 tensors followed by one quantize == concat of the two int8 tensors (same scale)
        assert scales["convs"][st["post"]][1] == scales["convs"][st["route_a"]][1]
        _, cur = block(st["transition"], np.concatenate([post, ra], axis=1))
        outs[st["name"]] = cur
    return outs, cur


def test_small_cspdarknet_matches_the_operator_chain(checker):
    from tennis_b200 import nets
    spec = nets.cspdarknet_spec(image=64, widths=(64, 128), blocks=(1, 2))
    assert len(spec["convs"]) == 1 + (5 + 2 * 1) + (5 + 2 * 2)
    params = nets.make_conv_params(spec, seed=4)
    n = 2
    rng = np.random.default_rng(1)
    x = rng.random((n, 3, 64, 64), dtype=np.float32)
    net = nets.QuantCSPDarknet(spec, params, n)
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


def test_cspdarknet53_topology():
    from tennis_b200 import nets
    spec = nets.cspdarknet_spec()
    assert len(spec["convs"]) == 72 and spec["final_size"] == 19 and spec["features"] == 1024
    assert sum(1 for c in spec["convs"] if c["k"] == 3) == 1 + 5 + 23
