"""The benchmark networks as chains of reference operators.  TEST INFRASTRUCTURE ONLY.

A ResNet-50-shaped or CSPDarknet53-shaped int8 network is, in TenniS operator terms, a sequence of
``quantize -> conv2d_quantized -> add_bias -> [add] -> relu | leaky_relu [-> add]`` with ``pooling2d`` / ``concat``
in between.  These walkers run that sequence layer by layer on a CPU checker (oracle.Port or oracle.Reference) from
the same topology description, parameters and calibrated scales the GPU network uses, so that every intermediate
tensor of the GPU pass can be compared with what the operators would have produced one after another.

Imported by the parity tests and by the parity check of the benchmark's secondary workloads; nothing on the product
path uses it.
"""
import numpy as np


def dequantize_scales(weight_scales, bn, input_scale):
    """Per-channel dequantize scales of a layer: weight scale x folded BatchNorm factor / input quantize scale, fp32."""
    return (weight_scales * np.float32(bn) / np.float32(input_scale)).astype(np.float32)


def resnet_forward(spec, params, scales, x, chk):
    """x: fp32 NCHW numpy batch (more than one sample, so that quantize takes its one-scale-per-sample branch).
    Returns (int8 output of every bottleneck block, fp32 output of the last block, logits)."""
    n = x.shape[0]
    convs, P = spec["convs"], params["convs"]

    def block(idx, xq, act, residual=None, requant=True):
        c, p = convs[idx], P[idx]
        s_in, s_out = scales["convs"][idx]
        dq = dequantize_scales(p["sw"], scales["bn"][idx], s_in)
        rq = [float(s_out)] * n if requant else None
        return chk.conv_block(xq, p["w"], (c["pad"],) * 4, (c["stride"],) * 2, (1, 1), dq, p["bias"], act=act,
                              residual=residual, requant_scales=rq)

    xq = chk.quantize(x, [float(scales["input"])] * n)
    y, _ = block(0, xq, "relu")
    # the stem pool as a TenniS graph carries it: pooling2d 3x3/2 with padding {1,0,1,0} under the ceil-mode extent
    pooled = chk.max_pooling2d(y, 3, 2, (1, 0, 1, 0))
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


def cspdarknet_forward(spec, params, scales, x, chk, leaky=0.1):
    """Returns ({block or stage name: int8 output}, int8 output of the last stage)."""
    n = x.shape[0]
    convs, P = spec["convs"], params["convs"]

    def block(idx, xq, residual=None):
        c, p = convs[idx], P[idx]
        s_in, s_out = scales["convs"][idx]
        dq = dequantize_scales(p["sw"], scales["bn"][idx], s_in)
        return chk.conv_block(xq, p["w"], (c["pad"],) * 4, (c["stride"],) * 2, (1, 1), dq, p["bias"], act="leaky_relu",
                              leaky=leaky, residual=residual, requant_scales=[float(s_out)] * n,
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


def resnet_mismatches(spec, net_buffers, logits, picks, outs, last_f32, want_logits, rtol=1e-5):
    """Counts differing elements between a GPU pass (torch buffers of nets.QuantResNet) and resnet_forward's results for
    the images `picks`.  int8 block outputs: exact; last fp32 tensor: identical bits up to the sign of zero; logits: rtol."""
    bad = 0
    k = 0
    for stage in spec["stages"]:
        for b in stage:
            got = net_buffers[b["name"] + ".y.i8"][picks].cpu().numpy()
            o = spec["convs"][b["conv3"]]["o"]
            bad += int((got[..., :o].transpose(0, 3, 1, 2) != outs[k]).sum()) + int((got[..., o:] != 0).sum())
            k += 1
    last = net_buffers[spec["stages"][-1][-1]["name"] + ".y.f32"][picks].cpu().numpy().transpose(0, 3, 1, 2)
    a, b_ = np.ascontiguousarray(last, np.float32), np.ascontiguousarray(last_f32, np.float32)
    bad += int((~((a.view(np.int32) == b_.view(np.int32)) | ((a == 0) & (b_ == 0)))).sum())
    lg = logits[picks].cpu().numpy()
    bad += int((np.abs(lg - want_logits) > rtol * np.abs(want_logits).max() + rtol * np.abs(want_logits)).sum())
    return bad


def cspdarknet_mismatches(spec, net_buffers, out, picks, outs, last):
    bad = 0
    for st in spec["stages"]:
        for b in st["blocks"]:
            got = net_buffers[b["name"] + ".y.i8"][picks].cpu().numpy()
            o = spec["convs"][b["conv2"]]["o"]
            bad += int((got[..., :o].transpose(0, 3, 1, 2) != outs[b["name"]]).sum())
        got = net_buffers[st["name"] + ".out.i8"][picks].cpu().numpy()
        bad += int((got[..., :st["width"]].transpose(0, 3, 1, 2) != outs[st["name"]]).sum())
    bad += int((out[picks].cpu().numpy()[..., :spec["features"]].transpose(0, 3, 1, 2) != last).sum())
    return bad
