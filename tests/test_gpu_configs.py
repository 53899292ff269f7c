"""The benchmark configurations at their full sizes: configuration 0 (batch 1) and the batch-32 shape sweep,
checked against the CPU checker where it finishes in seconds and through size-independent properties."""
import numpy as np
import pytest
import torch

from conftest import same_bits

pytestmark = pytest.mark.gpu


def run_layer(layer, d, requant=None):
    from tennis_b200 import _lib, ops
    dev = torch.device("cuda")
    x = torch.from_numpy(d["x"]).to(dev)
    w = torch.from_numpy(d["w"]).to(dev)
    pad = (layer["pad"],) * 4
    plan = ops.ConvPlan(x.shape, w.shape, pad, (layer["stride"],) * 2, (layer["dilation"],) * 2, 0.0, 0, dev)
    plan.set_weights(w)
    scales = [float(d["qscale"])] * layer["n"]
    plan.quantize_input(x, scales)
    xq, xl = None, _lib.LAYOUT_STAGED
    out = torch.empty(plan.out_shape, dtype=torch.float32, device=dev)
    acc = torch.empty(plan.out_shape, dtype=torch.int32, device=dev)
    plan.run(xq, xl, torch.from_numpy(d["dq"]).to(dev), bias=torch.from_numpy(d["bias"]).to(dev),
             activation=_lib.ACT_RELU, out_f32=out, out_acc=acc)
    plan.status()
    torch.cuda.synchronize()
    return plan, out, acc


def test_config0_single_layer(checker):
    from tennis_b200 import workloads
    layer = workloads.CONFIG0[0]
    d = workloads.make_layer_data(layer, seed=0)
    plan, out, _ = run_layer(layer, d)
    xq = checker.quantize(d["x"], [float(d["qscale"])])
    want = checker.conv_block(xq, d["w"], (1, 1, 1, 1), (1, 1), (1, 1), d["dq"], d["bias"], act="relu")
    assert plan.kernel == 2
    assert same_bits(out.cpu().numpy(), want)


@pytest.mark.parametrize("index", range(5))
def test_config1_shape_sweep(port, index):
    from tennis_b200 import workloads
    layer = workloads.CONFIG1[index]
    d = workloads.make_layer_data(layer, seed=0)
    plan, out, acc = run_layer(layer, d)
    scales = [float(d["qscale"])] * layer["n"]
    xq = port.quantize(d["x"], scales)
    pad = (layer["pad"],) * 4
    # the C restatement is exact and runs these sizes in seconds; check a slice of the batch against it
    sl = slice(0, 4)
    want, want_acc = port.conv2d_quantized(xq[sl], d["w"], pad, (layer["stride"],) * 2, (1, 1), d["dq"], return_acc=True)
    want = port.relu(port.add_bias(want, d["bias"]))
    assert np.array_equal(acc[sl].cpu().numpy(), want_acc)
    assert same_bits(out[sl].cpu().numpy(), want)
    # the whole batch: every int32 accumulator against an exact fp64 convolution of the same int8 tensors
    # (all products and sums are integers far below 2^53, so fp64 arithmetic is exact in any order)
    xq_t = torch.from_numpy(xq).cuda().to(torch.float64)
    w_t = torch.from_numpy(d["w"]).cuda().to(torch.float64)
    ref = torch.nn.functional.conv2d(xq_t, w_t, stride=layer["stride"], padding=layer["pad"])
    assert torch.equal(ref, acc.to(torch.float64))
    # and the epilogue over the whole batch, recomputed in torch with separately rounded fp32 steps
    y = acc.to(torch.float32) * torch.from_numpy(d["dq"]).cuda().view(1, -1, 1, 1)
    y = torch.relu(y + torch.from_numpy(d["bias"]).cuda().view(1, -1, 1, 1))
    assert torch.equal(y, out)
