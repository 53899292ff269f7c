"""Quantized bottleneck ResNets (the ResNet-50-shaped int8 network of the benchmark configurations) on the fused path.

A network is a list of convolution specs plus the fixed glue of a bottleneck ResNet: stem 7x7/2 -> max pool 3x3/2 ->
stages of [1x1, 3x3, 1x1(x4)] blocks with a 1x1 projection shortcut on the first block of each stage -> fp32 global
average pool -> fp32 inner product.  BatchNorm is folded into per-channel scale and bias, ReLU is fused, activations
travel between convolutions as int8 NHWC_PAD (requantized in the producing convolution's epilogue with the consumer's
quantize scale), residual adds are fp32.  In TenniS operator terms every convolution is
``quantize -> conv2d_quantized -> add_bias -> [add] -> relu`` and the results are bit-identical to running those
operators one by one.

Weights are synthetic (seeded): int8 uniform in [-127,127], per-channel weight scales U(0.001,0.01), bias N(0,0.1).
Activation scales are calibrated once on a sample batch (127 / max|activation| per tensor).
"""
import numpy as np
import torch

from . import _lib
from ._lib import ACT_NONE, ACT_RELU, LAYOUT_NHWC_PAD, LAYOUT_STAGED, check
from . import ops


def resnet_spec(image=224, widths=(64, 128, 256, 512), blocks=(3, 4, 6, 3), stem_channels=64, classes=1000, expansion=4):
    """Topology of a bottleneck ResNet as plain data.  ResNet-50: the defaults (53 convolutions)."""
    convs = []

    def conv(name, cin, cout, k, stride, pad, size_in):
        size_out = (size_in + 2 * pad - k) // stride + 1
        convs.append(dict(name=name, c=cin, o=cout, k=k, stride=stride, pad=pad, h=size_in, oh=size_out))
        return size_out

    size = conv("stem", 3, stem_channels, 7, 2, 3, image)
    # pooling2d 3x3/2 with padding {top 1, bottom 0, left 1, right 0}: under the reference's ceil-mode extent
    # (include/backend/common_function.h:13-20) that is the usual floor-mode pool with padding 1
    pooled = -(-(size + 1 + 0 - 3) // 2) + 1
    stages = []
    cin, size = stem_channels, pooled
    for si, (width, nblocks) in enumerate(zip(widths, blocks)):
        stage = []
        for bi in range(nblocks):
            stride = 2 if (bi == 0 and si > 0) else 1
            cout = width * expansion
            b = dict(name="s%db%d" % (si + 1, bi + 1), projection=(bi == 0))
            b["conv1"] = len(convs); conv(b["name"] + ".conv1", cin, width, 1, 1, 0, size)
            b["conv2"] = len(convs); size_out = conv(b["name"] + ".conv2", width, width, 3, stride, 1, size)
            b["conv3"] = len(convs); conv(b["name"] + ".conv3", width, cout, 1, 1, 0, size_out)
            if b["projection"]:
                b["proj"] = len(convs); conv(b["name"] + ".proj", cin, cout, 1, stride, 0, size)
            stage.append(b)
            cin, size = cout, size_out
        stages.append(stage)
    return dict(image=image, convs=convs, stages=stages, stem_pooled=pooled, features=cin, classes=classes, final_size=size)


def conv_ops(spec, batch):
    """2 * N * O * OH * OW * C * KH * KW summed over the convolutions."""
    return sum(2 * batch * c["o"] * c["oh"] * c["oh"] * c["c"] * c["k"] * c["k"] for c in spec["convs"])


def make_params(spec, seed=0):
    """Seeded synthetic parameters (numpy).  dq holds the per-channel WEIGHT scales; the dequantize scales of a layer are
    weight scale / input quantize scale, computed once the activation scales are known."""
    rng = np.random.default_rng(seed)
    params = []
    for c in spec["convs"]:
        w = rng.integers(-127, 128, size=(c["o"], c["c"], c["k"], c["k"]), dtype=np.int8)
        sw = rng.uniform(0.001, 0.01, size=c["o"]).astype(np.float32)
        bias = (rng.standard_normal(c["o"]) * 0.1).astype(np.float32)
        params.append(dict(w=w, sw=sw, bias=bias))
    fc_w = (rng.standard_normal((spec["classes"], spec["features"])) * 0.01).astype(np.float32)
    fc_b = (rng.standard_normal(spec["classes"]) * 0.01).astype(np.float32)
    return dict(convs=params, fc_w=fc_w, fc_b=fc_b)


def dequantize_scales(weight_scales, bn, input_scale):
    """Per-channel dequantize scales of a layer: weight scale x folded BatchNorm factor / input quantize scale, in fp32."""
    return (weight_scales * np.float32(bn) / np.float32(input_scale)).astype(np.float32)


class QuantResNet:
    """The network on one GPU: plans, weights and activation buffers are built once; forward() launches only kernels of
    libtennis_b200.so (quantize, convolutions with fused epilogues, max pool, average pool, inner product)."""

    def __init__(self, spec, params, batch, device="cuda", fuse_projection=True):
        self.spec, self.batch, self.dev = spec, batch, torch.device(device)
        # the projection shortcut of a stage's first block runs inside the launch of the block's last convolution
        # (tsb_conv2d_i8_run_projected); False: as a launch of its own whose fp32 output is that convolution's residual
        self.fuse_projection = fuse_projection
        self.lib = _lib.load()
        dev = self.dev
        self.convs = []
        for c, p in zip(spec["convs"], params["convs"]):
            xshape = (batch, c["c"], c["h"], c["h"])
            wshape = (c["o"], c["c"], c["k"], c["k"])
            plan = ops.ConvPlan(xshape, wshape, (c["pad"],) * 4, (c["stride"],) * 2, (1, 1), 0.0, _lib.KERNEL_AUTO, dev)
            plan.set_weights(torch.from_numpy(p["w"]).to(dev))
            self.convs.append(dict(spec=c, plan=plan, sw=p["sw"], bias=torch.from_numpy(p["bias"]).to(dev), dq=None,
                                   in_scale=None, out_scale=None, bn=np.float32(1.0)))
        self.fc_w = torch.from_numpy(params["fc_w"]).to(dev)
        self.fc_b = torch.from_numpy(params["fc_b"]).to(dev)
        self.buffers = {}
        self.calibrated = False
        self.launch_log = None

    # ---- buffers ------------------------------------------------------------------------------------------------
    def _i8(self, key, pixels_hw, channels):
        shape = (self.batch, pixels_hw, pixels_hw, ops.padded_channels(channels))
        if key not in self.buffers:
            self.buffers[key] = torch.zeros(shape, dtype=torch.int8, device=self.dev)
        return self.buffers[key]

    def _f32(self, key, pixels_hw, channels):
        shape = (self.batch, pixels_hw, pixels_hw, channels)
        if key not in self.buffers:
            self.buffers[key] = torch.zeros(shape, dtype=torch.float32, device=self.dev)
        return self.buffers[key]

    # ---- one convolution ----------------------------------------------------------------------------------------
    def _conv(self, idx, x_i8, key, act, want_i8=True, want_f32=False, residual=None, staged=False, leaky=0.0,
              residual_after=False):
        L = self.convs[idx]
        c = L["spec"]
        out_i8 = self._i8(key + ".i8", c["oh"], c["o"]) if want_i8 else None
        out_f32 = self._f32(key + ".f32", c["oh"], c["o"]) if want_f32 else None

        def launch():
            L["plan"].run(None if staged else x_i8, LAYOUT_STAGED if staged else LAYOUT_NHWC_PAD, L["dq"], bias=L["bias"],
                          residual=residual, activation=act, leaky=leaky, out_f32=out_f32, out_f32_layout=LAYOUT_NHWC_PAD,
                          out_i8=out_i8, out_i8_layout=LAYOUT_NHWC_PAD,
                          requant_scales=L["out_scale_arr"] if want_i8 else None, residual_after_activation=residual_after)
        launch()
        if self.launch_log is not None:      # layer_times(): every convolution launch of a pass, replayable
            out_bytes = (out_i8.numel() if want_i8 else 0) + (4 * self.batch * c["oh"] * c["oh"] * c["o"] if want_f32 else 0)
            in_bytes = self.batch * c["h"] * c["h"] * ops.padded_channels(c["c"]) + c["o"] * c["c"] * c["k"] * c["k"] + 8 * c["o"]
            if residual is not None:
                in_bytes += 4 * self.batch * c["oh"] * c["oh"] * c["o"]
            self.launch_log.append(dict(name=c["name"], launch=launch, ops=2 * self.batch * c["o"] * c["oh"] * c["oh"] * c["c"] * c["k"] * c["k"],
                                        bytes=in_bytes + out_bytes, k=c["k"], c=c["c"], o=c["o"], size=c["oh"], stride=c["stride"],
                                        residual=residual is not None, fp32_out=bool(want_f32), int8_out=bool(want_i8)))
        return out_i8, out_f32

    def _conv_projected(self, idx, x_i8, idx_proj, x_proj, key, act):
        """Convolution idx with the projection idx_proj (over x_proj) as its residual, one launch; int8 and fp32 out."""
        L, S = self.convs[idx], self.convs[idx_proj]
        c, cs = L["spec"], S["spec"]
        out_i8 = self._i8(key + ".i8", c["oh"], c["o"])
        out_f32 = self._f32(key + ".f32", c["oh"], c["o"])

        def launch():
            L["plan"].run_projected(x_i8, S["plan"], x_proj, L["dq"], S["dq"], bias=L["bias"], shortcut_bias=S["bias"],
                                    activation=act, out_f32=out_f32, out_i8=out_i8, requant_scales=L["out_scale_arr"])
        launch()
        if self.launch_log is not None:
            px = self.batch * c["oh"] * c["oh"]
            in_bytes = (self.batch * c["h"] * c["h"] * ops.padded_channels(c["c"]) + c["o"] * c["c"] * c["k"] * c["k"] + 8 * c["o"] +
                        self.batch * cs["h"] * cs["h"] * ops.padded_channels(cs["c"]) // (cs["stride"] ** 2) + c["o"] * cs["c"] + 8 * c["o"])
            self.launch_log.append(dict(name=c["name"] + "+proj", launch=launch, ops=2 * px * c["o"] * (c["c"] * c["k"] * c["k"] + cs["c"]),
                                        bytes=in_bytes + out_i8.numel() + 4 * px * c["o"], k=c["k"], c=c["c"] + cs["c"], o=c["o"],
                                        size=c["oh"], stride=c["stride"], residual=False, fp32_out=True, int8_out=True))
        return out_i8, out_f32

    def _calibrate_conv(self, idx, x_i8, key, act, residual=None, staged=False, leaky=0.0, residual_after=False):
        """Fixes the layer's folded-BatchNorm factor (the convolution's own output is brought to a maximum of 4, so that
        activations stay bounded through the network whatever the synthetic weight scales are) and returns the maximum
        magnitude of the layer's fp32 output."""
        L = self.convs[idx]
        c = L["spec"]
        f = self._f32(key + ".cal", c["oh"], c["o"])
        src, layout = (None, LAYOUT_STAGED) if staged else (x_i8, LAYOUT_NHWC_PAD)
        L["plan"].run(src, layout, L["dq"], out_f32=f, out_f32_layout=LAYOUT_NHWC_PAD)
        m0 = float(f.abs().max())
        L["bn"] = np.float32(4.0 / m0) if m0 > 0 else np.float32(1.0)
        self._set_in_scale(idx, L["in_scale"])
        L["plan"].run(src, layout, L["dq"], bias=L["bias"], residual=residual, activation=act, leaky=leaky, out_f32=f,
                      out_f32_layout=LAYOUT_NHWC_PAD, residual_after_activation=residual_after)
        m = float(f.abs().max())
        del self.buffers[key + ".cal"]
        return m

    def _set_in_scale(self, idx, scale):
        L = self.convs[idx]
        L["in_scale"] = np.float32(scale)
        L["dq"] = torch.from_numpy(dequantize_scales(L["sw"], L["bn"], scale)).to(self.dev)

    def _set_out_scale(self, idx, scale):
        L = self.convs[idx]
        L["out_scale"] = np.float32(scale)
        L["out_scale_arr"] = _lib.float_array([float(scale)] * self.batch)

    # ---- calibration: run layer by layer in fp32-out mode, fix 127/max|activation| as the next quantize scale ------
    def calibrate(self, x):
        """x: fp32 NCHW sample batch on the device.  Fixes every activation scale; returns them as a dict."""
        spec = self.spec
        amax = float(x.abs().max())
        self.input_scale = np.float32(127.0) / np.float32(amax if amax > 0 else 1.0)
        self._set_in_scale(0, self.input_scale)

        def out_scale_of(idx, x_i8, key, act, residual=None, staged=False):
            m = self._calibrate_conv(idx, x_i8, key, act, residual=residual, staged=staged)
            return np.float32(127.0) / np.float32(m if m > 0 else 1.0)

        self.input_scale_arr = _lib.float_array([float(self.input_scale)] * self.batch)
        self.convs[0]["plan"].quantize_input(x, self.input_scale_arr)
        self._set_out_scale(0, out_scale_of(0, None, "stem", ACT_RELU, staged=True))
        cur_scale = self.convs[0]["out_scale"]          # scale of the int8 tensor entering the next convolutions
        x_i8 = self._forward_stem(x)
        x_f32 = None
        for stage in spec["stages"]:
            for b in stage:
                i1, i2, i3 = b["conv1"], b["conv2"], b["conv3"]
                self._set_in_scale(i1, cur_scale)
                self._set_out_scale(i1, out_scale_of(i1, x_i8, b["name"] + ".a", ACT_RELU))
                a, _ = self._conv(i1, x_i8, b["name"] + ".a", ACT_RELU)
                self._set_in_scale(i2, self.convs[i1]["out_scale"])
                self._set_out_scale(i2, out_scale_of(i2, a, b["name"] + ".b", ACT_RELU))
                bb, _ = self._conv(i2, a, b["name"] + ".b", ACT_RELU)
                if b["projection"]:
                    ip = b["proj"]
                    self._set_in_scale(ip, cur_scale)
                    out_scale_of(ip, x_i8, b["name"] + ".sc", ACT_NONE)   # fixes the layer's folded-BN factor
                    _, sc = self._conv(ip, x_i8, b["name"] + ".sc", ACT_NONE, want_i8=False, want_f32=True)
                else:
                    sc = x_f32
                self._set_in_scale(i3, self.convs[i2]["out_scale"])
                self._set_out_scale(i3, out_scale_of(i3, bb, b["name"] + ".y", ACT_RELU, residual=sc))
                y_i8, y_f32 = self._conv(i3, bb, b["name"] + ".y", ACT_RELU, want_i8=True, want_f32=True, residual=sc)
                x_i8, x_f32, cur_scale = y_i8, y_f32, self.convs[i3]["out_scale"]
        self.calibrated = True
        torch.cuda.synchronize()
        return dict(input=self.input_scale, convs=[(L["in_scale"], L["out_scale"]) for L in self.convs],
                    bn=[L["bn"] for L in self.convs])

    def _forward_stem(self, x):
        spec = self.spec
        L = self.convs[0]
        L["plan"].quantize_input(x, self.input_scale_arr)
        s_i8, _ = self._conv(0, None, "stem", ACT_RELU, staged=True)
        c = L["spec"]
        pooled = self._i8("stem.pool", spec["stem_pooled"], c["o"])
        check(self.lib.tsb_maxpool_i8_nhwc(s_i8.data_ptr(), pooled.data_ptr(), self.batch, c["oh"], c["oh"], c["o"], 3, 2, 1, 0, 1, 0,
                                           ops._stream_ptr()))
        return pooled

    def forward(self, x):
        """x: fp32 NCHW [batch, 3, image, image] on the device -> fp32 logits [batch, classes]."""
        assert self.calibrated, "call calibrate() first"
        spec = self.spec
        x_i8 = self._forward_stem(x)
        x_f32 = None
        for stage in spec["stages"]:
            for b in stage:
                a, _ = self._conv(b["conv1"], x_i8, b["name"] + ".a", ACT_RELU)
                bb, _ = self._conv(b["conv2"], a, b["name"] + ".b", ACT_RELU)
                if b["projection"] and self.fuse_projection:
                    x_i8, x_f32 = self._conv_projected(b["conv3"], bb, b["proj"], x_i8, b["name"] + ".y", ACT_RELU)
                    continue
                if b["projection"]:
                    _, sc = self._conv(b["proj"], x_i8, b["name"] + ".sc", ACT_NONE, want_i8=False, want_f32=True)
                else:
                    sc = x_f32
                x_i8, x_f32 = self._conv(b["conv3"], bb, b["name"] + ".y", ACT_RELU, want_i8=True, want_f32=True, residual=sc)
        feat = self.buffers.setdefault("feat", torch.empty((self.batch, spec["features"]), dtype=torch.float32, device=self.dev))
        logits = self.buffers.setdefault("logits", torch.empty((self.batch, spec["classes"]), dtype=torch.float32, device=self.dev))
        P = spec["final_size"] * spec["final_size"]
        check(self.lib.tsb_global_avgpool_f32_nhwc(x_f32.data_ptr(), feat.data_ptr(), self.batch, P, spec["features"], ops._stream_ptr()))
        check(self.lib.tsb_inner_prod_f32(feat.data_ptr(), self.fc_w.data_ptr(), self.fc_b.data_ptr(), logits.data_ptr(), self.batch,
                                          spec["features"], spec["classes"], ops._stream_ptr()))
        return logits

    def status(self):
        for L in self.convs:
            L["plan"].status()

    def layer_times(self, x, reps=20):
        """Device time of every convolution launch of one forward pass, each on its own: `reps` back-to-back launches
        replayed from a CUDA graph, inputs as the pass left them (warm L2 for small layers, as inside the pass).
        Returns a list of dicts (name, us, ops, bytes, shape fields)."""
        self.launch_log = []
        try:
            self.forward(x)
        finally:
            log, self.launch_log = self.launch_log, None
        torch.cuda.synchronize()
        out = []
        side = torch.cuda.Stream(device=self.dev)
        for item in log:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                item["launch"]()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(reps):
                        item["launch"]()
            torch.cuda.current_stream().wait_stream(side)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            d = {k: v for k, v in item.items() if k != "launch"}
            d["us"] = a.elapsed_time(b) * 1e3 / reps
            out.append(d)
            del g
        return out


# ---------------------------------------------------------------------------------------------------------------------
# CSPDarknet53-shaped backbone (configuration 3): LeakyReLU(0.1), Darknet shortcuts (fp32 add after the activation),
# cross-stage partial routes joined by a channel concatenation
# ---------------------------------------------------------------------------------------------------------------------
LEAKY = 0.1


def cspdarknet_spec(image=608, widths=(64, 128, 256, 512, 1024), blocks=(1, 2, 8, 8, 4), stem_channels=32):
    """Topology of the CSPDarknet53 backbone as plain data (72 convolutions with the defaults)."""
    convs = []

    def conv(name, cin, cout, k, stride, size_in):
        pad = k // 2
        size_out = (size_in + 2 * pad - k) // stride + 1
        convs.append(dict(name=name, c=cin, o=cout, k=k, stride=stride, pad=pad, h=size_in, oh=size_out))
        return len(convs) - 1, size_out

    stem, size = conv("stem", 3, stem_channels, 3, 1, image)
    stages = []
    cin = stem_channels
    for si, (width, nblocks) in enumerate(zip(widths, blocks)):
        name = "s%d" % (si + 1)
        half = width if si == 0 else width // 2
        inner = width // 2 if si == 0 else half          # bottleneck width of the residual blocks
        st = dict(name=name)
        st["down"], size = conv(name + ".down", cin, width, 3, 2, size)
        st["route_a"], _ = conv(name + ".route_a", width, half, 1, 1, size)
        st["route_b"], _ = conv(name + ".route_b", width, half, 1, 1, size)
        st["blocks"] = []
        for bi in range(nblocks):
            b = dict(name="%sb%d" % (name, bi + 1))
            b["conv1"], _ = conv(b["name"] + ".conv1", half, inner, 1, 1, size)
            b["conv2"], _ = conv(b["name"] + ".conv2", inner, half, 3, 1, size)
            st["blocks"].append(b)
        st["post"], _ = conv(name + ".post", half, half, 1, 1, size)
        st["transition"], _ = conv(name + ".transition", 2 * half, width, 1, 1, size)
        st["half"], st["size"], st["width"] = half, size, width
        stages.append(st)
        cin = width
    return dict(image=image, convs=convs, stem=stem, stages=stages, features=cin, final_size=size)


def make_conv_params(spec, seed=0):
    """Seeded synthetic convolution parameters only (networks without a classifier)."""
    rng = np.random.default_rng(seed)
    params = []
    for c in spec["convs"]:
        w = rng.integers(-127, 128, size=(c["o"], c["c"], c["k"], c["k"]), dtype=np.int8)
        sw = rng.uniform(0.001, 0.01, size=c["o"]).astype(np.float32)
        bias = (rng.standard_normal(c["o"]) * 0.1).astype(np.float32)
        params.append(dict(w=w, sw=sw, bias=bias))
    return dict(convs=params, fc_w=np.zeros((1, 1), np.float32), fc_b=np.zeros(1, np.float32))


class QuantCSPDarknet(QuantResNet):
    """The backbone on one GPU.  Every convolution is, in TenniS operator terms,
    ``quantize -> conv2d_quantized -> add_bias -> leaky_relu [-> add]``; the two routes of a stage are requantized with the
    same scale (that of the transition convolution's input) and joined by tsb_concat_i8_nhwc."""

    def __init__(self, spec, params, batch, device="cuda", fuse_concat=True):
        super().__init__(spec, params, batch, device)
        # the transition convolution of a stage reads its two halves (post, route a) directly, each through a plan over
        # its half of the weight columns (tsb_conv2d_i8_run_concat); False: an int8 concatenation kernel runs first
        self.fuse_concat = fuse_concat
        self.halves = {}
        for st in spec["stages"]:
            idx, half = st["transition"], st["half"]
            c, w = spec["convs"][idx], params["convs"][idx]["w"]
            shape = (batch, half, c["h"], c["h"])
            pair = []
            for part in (w[:, :half], w[:, half:]):
                plan = ops.ConvPlan(shape, (c["o"], half, 1, 1), (0,) * 4, (1, 1), (1, 1), 0.0, _lib.KERNEL_AUTO, self.dev)
                plan.set_weights(torch.from_numpy(np.ascontiguousarray(part)).to(self.dev))
                pair.append(plan)
            self.halves[idx] = pair

    def _conv_concat(self, idx, first, rest, key, act, leaky):
        """Transition idx over concat(first, rest) without the concatenation; int8 out."""
        L = self.convs[idx]
        c = L["spec"]
        p_first, p_rest = self.halves[idx]
        out_i8 = self._i8(key + ".i8", c["oh"], c["o"])

        def launch():
            p_rest.run_concat(rest, p_first, first, L["dq"], bias=L["bias"], activation=act, leaky=leaky, out_i8=out_i8,
                              requant_scales=L["out_scale_arr"])
        launch()
        if self.launch_log is not None:
            px = self.batch * c["oh"] * c["oh"]
            self.launch_log.append(dict(name=c["name"] + "+concat", launch=launch, ops=2 * px * c["o"] * c["c"],
                                        bytes=px * ops.padded_channels(c["c"]) + c["o"] * c["c"] + 8 * c["o"] + out_i8.numel(),
                                        k=1, c=c["c"], o=c["o"], size=c["oh"], stride=1, residual=False, fp32_out=False, int8_out=True))
        return out_i8

    def _concat(self, a, ca, b, cb, key, size):
        out = self._i8(key, size, ca + cb)
        check(self.lib.tsb_concat_i8_nhwc(a.data_ptr(), ca, b.data_ptr(), cb, out.data_ptr(), self.batch * size * size,
                                          ops._stream_ptr()))
        return out

    def _scale(self, m):
        return np.float32(127.0) / np.float32(m if m > 0 else 1.0)

    def _walk(self, x, calibrate):
        """One pass over the network; with calibrate=True every layer's scales are fixed just before it runs."""
        spec = self.spec
        act = _lib.ACT_LEAKY_RELU

        def run(idx, x_i8, key, in_scale, out_scale=None, want_f32=False, residual=None, staged=False, want_i8=True):
            if calibrate:
                self._set_in_scale(idx, in_scale)
                m = self._calibrate_conv(idx, x_i8, key, act, residual=residual, staged=staged, leaky=LEAKY,
                                         residual_after=residual is not None)
                self._set_out_scale(idx, out_scale if out_scale is not None else self._scale(m))
            return self._conv(idx, x_i8, key, act, want_i8=want_i8, want_f32=want_f32, residual=residual, staged=staged,
                              leaky=LEAKY, residual_after=residual is not None)

        def peek_max(idx, x_i8, key, in_scale):
            self._set_in_scale(idx, in_scale)
            return self._calibrate_conv(idx, x_i8, key, act, leaky=LEAKY)

        i0 = spec["stem"]
        if calibrate:
            amax = float(x.abs().max())
            self.input_scale = np.float32(127.0) / np.float32(amax if amax > 0 else 1.0)
            self.input_scale_arr = _lib.float_array([float(self.input_scale)] * self.batch)
        self.convs[i0]["plan"].quantize_input(x, self.input_scale_arr)
        cur, _ = run(i0, None, "stem", self.input_scale, staged=True)
        cur_scale = self.convs[i0]["out_scale"]
        for st in spec["stages"]:
            half, size = st["half"], st["size"]
            cur, _ = run(st["down"], cur, st["name"] + ".down", cur_scale)
            s_down = self.convs[st["down"]]["out_scale"]
            # route b: 1x1, residual blocks, 1x1
            xb_i8, xb_f32 = run(st["route_b"], cur, st["name"] + ".rb", s_down, want_f32=True)
            sb = self.convs[st["route_b"]]["out_scale"]
            for b in st["blocks"]:
                h, _ = run(b["conv1"], xb_i8, b["name"] + ".h", sb)
                xb_i8, xb_f32 = run(b["conv2"], h, b["name"] + ".y", self.convs[b["conv1"]]["out_scale"], want_f32=True,
                                    residual=xb_f32)
                sb = self.convs[b["conv2"]]["out_scale"]
            # the two tensors that are concatenated share the scale of the transition's input
            if calibrate:
                m_post = peek_max(st["post"], xb_i8, st["name"] + ".post", sb)
                m_a = peek_max(st["route_a"], cur, st["name"] + ".ra", s_down)
                s_cat = self._scale(max(m_post, m_a))
            else:
                s_cat = None
            post, _ = run(st["post"], xb_i8, st["name"] + ".post", sb, out_scale=s_cat)
            ra, _ = run(st["route_a"], cur, st["name"] + ".ra", s_down, out_scale=s_cat)
            if self.fuse_concat and not calibrate:
                cur = self._conv_concat(st["transition"], post, ra, st["name"] + ".out", act, LEAKY)
            else:
                cat = self._concat(post, half, ra, half, st["name"] + ".cat", size)
                cur, _ = run(st["transition"], cat, st["name"] + ".out", self.convs[st["post"]]["out_scale"])
            cur_scale = self.convs[st["transition"]]["out_scale"]
        return cur

    def calibrate(self, x):
        out = self._walk(x, calibrate=True)
        self.calibrated = True
        torch.cuda.synchronize()
        return dict(input=self.input_scale, convs=[(L["in_scale"], L["out_scale"]) for L in self.convs],
                    bn=[L["bn"] for L in self.convs])

    def forward(self, x):
        """x: fp32 NCHW [batch, 3, image, image] on the device -> int8 NHWC_PAD feature map of the last stage."""
        assert self.calibrated, "call calibrate() first"
        return self._walk(x, calibrate=False)


def _main():
    """python -m tennis_b200.nets {resnet50,cspdarknet53} [--batch N] [--passes K]: builds the synthetic network,
    calibrates it on one random batch and runs K eager forward passes (what a profiler is pointed at)."""
    import argparse
    ap = argparse.ArgumentParser(description=_main.__doc__)
    ap.add_argument("net", choices=["resnet50", "cspdarknet53"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--passes", type=int, default=3)
    args = ap.parse_args()
    torch.manual_seed(0)
    if args.net == "resnet50":
        batch = args.batch or 64
        spec = resnet_spec()
        net = QuantResNet(spec, make_params(spec, 0), batch)
        x = torch.randn((batch, 3, 224, 224), device="cuda")
    else:
        batch = args.batch or 16
        spec = cspdarknet_spec()
        net = QuantCSPDarknet(spec, make_conv_params(spec, 0), batch)
        x = torch.rand((batch, 3, 608, 608), device="cuda")
    net.calibrate(x)
    out = None
    for _ in range(args.passes):
        out = net.forward(x)
    torch.cuda.synchronize()
    net.status()
    print("%s batch %d: %d convolutions, %.1f GOP per pass, output checksum %.6g"
          % (args.net, batch, len(spec["convs"]), conv_ops(spec, batch) / 1e9, float(out.double().abs().sum())))


if __name__ == "__main__":
    _main()
