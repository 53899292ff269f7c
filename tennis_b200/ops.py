"""Python mirror of the two TenniS operators on the path, over the C ABI.

The shipping host side is the C++ plugin in tennis_b200/plugin/ (TS_REGISTER_OPERATOR on device "gpu"); this
module states the same interface for Python callers and for the parity tests: same operator names, same
attribute names and meaning, the same checks in ``init`` / ``infer`` and the same error texts as

* ts::base::Quantize          src/backend/base/base_quantize.cpp:12-49
* ts::base::Conv2DQuantized   src/backend/base/base_conv2d_quantized.cpp:13-219
* ts::Operator                src/runtime/operator.cpp:22-128 (fields, set, check_params)

Tensors are torch CUDA tensors used as device buffers; all arithmetic happens in libtennis_b200.so.
"""
import ctypes

import numpy as np
import torch

from . import _lib
from ._lib import (ACT_LEAKY_RELU, ACT_NONE, ACT_RELU, KERNEL_AUTO, KERNEL_DIRECT, KERNEL_TCGEN05, LAYOUT_NCHW,
                   LAYOUT_NHWC_PAD, LAYOUT_STAGED, ConvDesc, ConvEpilogue, TsbError, check, float_array)

REQUIRED, OPTIONAL = "required", "optional"


class EjectionException(RuntimeError):
    """What TS_LOG_ERROR << ... << eject raises in the reference (include/utils/log.h:162-166)."""


def _stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def padded_channels(c):
    return _lib.load().tsb_padded_channels(int(c))


def conv_out_dim(x, pad_lo, pad_hi, k, stride, dilation):
    """include/backend/common_function.h:30-40: integer division truncating toward zero."""
    num = x + pad_lo + pad_hi - (dilation * (k - 1) + 1)
    q = abs(num) // stride
    return (q if num >= 0 else -q) + 1


class Operator:
    """Field handling of ts::Operator (src/runtime/operator.cpp:22-128)."""

    op = "operator"

    def __init__(self):
        self._fields = {}
        self._params = {}

    def field(self, name, attr, default=None):
        self._fields[name] = attr
        if default is not None:
            self._params[name] = default

    def has(self, name):
        return name in self._params

    def get(self, name):
        if name not in self._params:
            raise EjectionException('Unidentified param "%s"' % name)
        return self._params[name]

    def set(self, name, value):
        if name not in self._fields:
            raise EjectionException('Unidentified param "%s", did you mean "%s"' % (name, self._closest(name)))
        self._params[name] = value

    def _closest(self, name):
        import difflib
        m = difflib.get_close_matches(name, list(self._fields), n=1, cutoff=0.0)
        return m[0] if m else ""

    def init(self):
        missing = [f for f, a in self._fields.items() if a == REQUIRED and f not in self._params]
        if missing:
            raise EjectionException("Operator %s has unsatisfied fields: %s" % (self.op, ", ".join(missing)))


def _auto_check(cond, text):
    if not cond:
        raise EjectionException("Check failed: (%s)." % text)


class Quantize(Operator):
    """Operator "quantize" on the GPU: fp32 -> int8, attribute ``quantize_scale`` (one scale per sample)."""

    op = "quantize"

    def __init__(self):
        super().__init__()
        self.field("quantize_scale", REQUIRED)
        self.scales = None

    def init(self):
        super().init()
        self.scales = [float(v) for v in np.asarray(self.get("quantize_scale"), dtype=np.float32).reshape(-1)]

    def infer(self, inputs):
        _auto_check(len(inputs) == 1, "stack.size() == 1")
        x = inputs[0]
        _auto_check(len(self.scales) == x.shape[0], "m_quantize_scales.size() == x_tensor.sizes()[0]")
        return [("int8", tuple(x.shape))]

    def run(self, inputs, stream=None):
        self.infer(inputs)
        x = inputs[0]
        if x.dtype not in (torch.float32, torch.float64):   # the reference's dispatch: src/kernels/cpu/quantize.cpp:130-141
            raise EjectionException("%s not support this data type: %s" % (self.op, str(x.dtype).replace("torch.", "")))
        x = x.contiguous()
        y = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        lib = _lib.load()
        fn = lib.tsb_quantize_f32_i8 if x.dtype == torch.float32 else lib.tsb_quantize_f64_i8
        check(fn(_ptr(x), _ptr(y), x.numel(), float_array(self.scales), len(self.scales), _stream_ptr(stream)))
        return y


class ConvPlan:
    """Owner of a tsb_conv_plan, its workspace and the device copies of the per-channel vectors."""

    def __init__(self, xshape, wshape, pad, stride, dilation, padding_value=0.0, kernel=KERNEL_AUTO, device="cuda",
                 mma_orientation=0, raw_row_mode=0, patch_mode=0):
        lib = _lib.load()
        d = ConvDesc()
        d.mma_orientation, d.raw_row_mode, d.patch_mode = int(mma_orientation), int(raw_row_mode), int(patch_mode)
        d.n, d.c, d.h, d.w = [int(v) for v in xshape]
        d.o, _, d.kh, d.kw = [int(v) for v in wshape]
        d.pad_top, d.pad_bottom, d.pad_left, d.pad_right = [int(v) for v in pad]
        d.stride_h, d.stride_w = [int(v) for v in stride]
        d.dilation_h, d.dilation_w = [int(v) for v in dilation]
        d.padding_value = float(padding_value)
        d.kernel = int(kernel)
        self.desc = d
        handle = ctypes.c_void_p()
        check(lib.tsb_conv2d_i8_plan_create(ctypes.byref(d), ctypes.byref(handle)))
        self.handle = handle
        shape = (ctypes.c_int * 4)()
        check(lib.tsb_conv2d_i8_output_shape(handle, shape))
        self.out_shape = tuple(shape)
        self.kernel = lib.tsb_conv2d_i8_kernel(handle)
        self.ws_bytes = lib.tsb_conv2d_i8_workspace_bytes(handle)
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=device)
        self.weights = None
        self.device = device

    def __del__(self):
        try:
            if self.handle:
                _lib.load().tsb_conv2d_i8_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    def set_weights(self, w, stream=None):
        assert w.dtype == torch.int8 and w.is_cuda
        self.weights = w.contiguous()  # the direct kernel reads this tensor at run time
        check(_lib.load().tsb_conv2d_i8_set_weights(self.handle, _ptr(self.weights), _ptr(self.workspace), self.ws_bytes,
                                                    _stream_ptr(stream)))

    def quantize_input(self, x_f32, scales, stream=None):
        """fp32 NCHW -> the plan's staged int8 input; run() is then called with x=None, x_layout=LAYOUT_STAGED."""
        arr = scales if not isinstance(scales, (list, tuple)) else float_array(scales)
        check(_lib.load().tsb_conv2d_i8_quantize_input(self.handle, _ptr(x_f32), arr, len(arr), _ptr(self.workspace),
                                                       self.ws_bytes, _stream_ptr(stream)))

    def run(self, x, x_layout, dq, bias=None, residual=None, activation=ACT_NONE, leaky=0.0, out_f32=None,
            out_f32_layout=LAYOUT_NCHW, out_i8=None, out_i8_layout=LAYOUT_NCHW, requant_scales=None, out_acc=None,
            stream=None, residual_after_activation=False):
        e = ConvEpilogue()
        e.residual_after_activation = 1 if residual_after_activation else 0
        e.dequantize_scales = dq.data_ptr()
        e.bias = bias.data_ptr() if bias is not None else None
        e.residual = residual.data_ptr() if residual is not None else None
        e.activation = int(activation)
        e.leaky_scale = float(leaky)
        e.out_f32 = out_f32.data_ptr() if out_f32 is not None else None
        e.out_f32_layout = int(out_f32_layout)
        e.out_i8 = out_i8.data_ptr() if out_i8 is not None else None
        e.out_i8_layout = int(out_i8_layout)
        keep = None
        if requant_scales is not None:
            keep = requant_scales if isinstance(requant_scales, ctypes.Array) else float_array(requant_scales)
            e.requant_scales_host = keep
            e.n_requant_scales = len(requant_scales)
        e.out_acc = out_acc.data_ptr() if out_acc is not None else None
        check(_lib.load().tsb_conv2d_i8_run(self.handle, _ptr(x), int(x_layout), ctypes.byref(e), _ptr(self.workspace),
                                            self.ws_bytes, _stream_ptr(stream)))

    def run_projected(self, x, shortcut, x_shortcut, dq, shortcut_dq, bias=None, shortcut_bias=None, activation=ACT_NONE,
                      leaky=0.0, out_f32=None, out_i8=None, requant_scales=None, stream=None,
                      residual_after_activation=False, tile_channels=0):
        """This convolution with the 1x1 projection `shortcut` (another ConvPlan, its weights set) as its residual, in
        one launch (tsb_conv2d_i8_run_projected): NHWC_PAD int8 inputs, pixel-major fp32 / NHWC_PAD int8 outputs."""
        e = ConvEpilogue()
        e.residual_after_activation = 1 if residual_after_activation else 0
        e.dequantize_scales = dq.data_ptr()
        e.bias = bias.data_ptr() if bias is not None else None
        e.residual = None
        e.activation = int(activation)
        e.leaky_scale = float(leaky)
        e.out_f32 = out_f32.data_ptr() if out_f32 is not None else None
        e.out_f32_layout = LAYOUT_NHWC_PAD
        e.out_i8 = out_i8.data_ptr() if out_i8 is not None else None
        e.out_i8_layout = LAYOUT_NHWC_PAD
        keep = None
        if requant_scales is not None:
            keep = requant_scales if isinstance(requant_scales, ctypes.Array) else float_array(requant_scales)
            e.requant_scales_host = keep
            e.n_requant_scales = len(requant_scales)
        check(_lib.load().tsb_conv2d_i8_run_projected(
            self.handle, _ptr(x), shortcut.handle, _ptr(x_shortcut), _ptr(shortcut_dq),
            _ptr(shortcut_bias) if shortcut_bias is not None else None, ctypes.byref(e), int(tile_channels),
            _ptr(self.workspace), self.ws_bytes, _stream_ptr(stream)))

    def run_concat(self, x, first, x_first, dq, bias=None, activation=ACT_NONE, leaky=0.0, out_f32=None, out_i8=None,
                   requant_scales=None, stream=None, tile_channels=0):
        """The convolution over concat(x_first, x) along channels in one launch (tsb_conv2d_i8_run_concat): `first` holds the
        weight columns of the leading channels (a 1x1 plan), this plan the rest; NHWC_PAD int8 inputs quantized with the
        same scales, pixel-major fp32 / NHWC_PAD int8 outputs."""
        e = ConvEpilogue()
        e.dequantize_scales = dq.data_ptr()
        e.bias = bias.data_ptr() if bias is not None else None
        e.residual = None
        e.activation = int(activation)
        e.leaky_scale = float(leaky)
        e.out_f32 = out_f32.data_ptr() if out_f32 is not None else None
        e.out_f32_layout = LAYOUT_NHWC_PAD
        e.out_i8 = out_i8.data_ptr() if out_i8 is not None else None
        e.out_i8_layout = LAYOUT_NHWC_PAD
        keep = None
        if requant_scales is not None:
            keep = requant_scales if isinstance(requant_scales, ctypes.Array) else float_array(requant_scales)
            e.requant_scales_host = keep
            e.n_requant_scales = len(requant_scales)
        check(_lib.load().tsb_conv2d_i8_run_concat(self.handle, _ptr(x), first.handle, _ptr(x_first), ctypes.byref(e),
                                                   int(tile_channels), _ptr(self.workspace), self.ws_bytes, _stream_ptr(stream)))

    def status(self, stream=None):
        check(_lib.load().tsb_conv2d_i8_status(self.handle, _ptr(self.workspace), _stream_ptr(stream)))

    def describe(self):
        buf = ctypes.create_string_buffer(512)
        n = _lib.load().tsb_conv2d_i8_plan_describe(self.handle, buf, len(buf))
        if n < 0:
            check(n)
        return buf.value.decode()


def _to_string(arr):
    return "[" + ", ".join(str(int(v)) for v in arr) + "]"


class Conv2DQuantized(Operator):
    """Operator "conv2d_quantized" on the GPU: int8 NCHW x int8 OIHW -> fp32 NCHW."""

    op = "conv2d_quantized"

    def __init__(self, kernel=KERNEL_AUTO):
        super().__init__()
        self.field("format", REQUIRED)
        self.field("padding", REQUIRED)
        self.field("padding_value", OPTIONAL, 0.0)
        self.field("stride", REQUIRED)
        self.field("dilation", OPTIONAL)
        self.field("dialations", OPTIONAL)
        self.field("dequantize_scales", REQUIRED)
        self._kernel = kernel
        self._plans = {}
        self._dq_dev = None

    def init(self):
        super().init()
        fmt = self.get("format")
        padding = np.asarray(self.get("padding")).astype(np.int32)
        self.padding_value = float(np.asarray(self.get("padding_value")).reshape(-1)[0])
        stride = np.asarray(self.get("stride")).astype(np.int32)
        dilation = None
        if self.has("dilation"):
            dilation = np.asarray(self.get("dilation")).astype(np.int32)
        elif self.has("dialations"):
            dilation = np.asarray(self.get("dialations")).astype(np.int32)
        if dilation is None or dilation.size == 0:
            raise EjectionException("%s must set dilation or dialations" % self.op)
        _auto_check(padding.shape == (4, 2), "padding_tensor.has_shape({ 4, 2 })")
        _auto_check(stride.shape == (4,), "stride_tensor.has_shape({ 4, })")
        _auto_check(dilation.shape == (4,), "dilation_tensor.has_shape({ 4, })")
        if fmt not in ("NCHW", "NHWC"):
            raise EjectionException("%s do not support format: %s" % (self.op, fmt))
        self.format = fmt
        p = padding.reshape(-1)
        if fmt == "NCHW":
            bad_p, bad_s, bad_d = p[:4].any(), (stride[:2] != 1).any(), (dilation[:2] != 1).any()
        else:
            bad_p = p[[0, 1, 6, 7]].any()
            bad_s, bad_d = (stride[[0, 3]] != 1).any(), (dilation[[0, 3]] != 1).any()
        if bad_p:
            raise EjectionException("%s do not support padding: %s" % (self.op, _to_string(p)))
        if bad_s:
            raise EjectionException("%s do not support stride: %s" % (self.op, _to_string(stride)))
        if bad_d:
            raise EjectionException("%s do not support dialations: %s" % (self.op, _to_string(dilation)))
        self.padding4x2, self.stride4, self.dilation4 = p, stride, dilation
        self.dequantize_scales = np.asarray(self.get("dequantize_scales"), dtype=np.float32).reshape(-1)

    def _geometry(self):
        p, s, d = self.padding4x2, self.stride4, self.dilation4
        if self.format == "NCHW":
            return (p[4], p[5], p[6], p[7]), (s[2], s[3]), (d[2], d[3])
        return (p[2], p[3], p[4], p[5]), (s[1], s[2]), (d[1], d[2])

    def infer(self, inputs):
        _auto_check(len(inputs) == 2, "stack.size() == 2")
        x, w = inputs
        _auto_check(x.dim() == 4, "x_tensor.dims() == 4")
        _auto_check(w.dim() == 4, "w_tensor.dims() == 4")
        _auto_check(x.dtype == w.dtype, "x_tensor.dtype() == w_tensor.dtype()")
        _auto_check(w.shape[1] == x.shape[1], "w_tensor.size(1) == x_tensor.size(1)")
        _auto_check(x.dtype == torch.int8, "x_tensor.dtype() == INT8")
        _auto_check(len(self.dequantize_scales) == w.shape[0], "m_dequantize_scales.size() == w_tensor.size(0)")
        pad, stride, dil = self._geometry()
        if self.format == "NCHW":
            H, W, KH, KW = x.shape[2], x.shape[3], w.shape[2], w.shape[3]
        else:
            H, W, KH, KW = x.shape[1], x.shape[2], w.shape[1], w.shape[2]
        OH = conv_out_dim(H, pad[0], pad[1], KH, stride[0], dil[0])
        OW = conv_out_dim(W, pad[2], pad[3], KW, stride[1], dil[1])
        if self.format == "NCHW":
            return [("float32", (x.shape[0], w.shape[0], OH, OW))]
        return [("float32", (x.shape[0], OH, OW, w.shape[0]))]

    def run(self, inputs, stream=None, out_acc=None):
        proto = self.infer(inputs)[0]
        if self.format != "NCHW":
            raise EjectionException("Conv2D_quantized only support NCHW")  # conv2d_quantized_core.cpp:131-133
        x, w = inputs
        x = x.contiguous()
        pad, stride, dil = self._geometry()
        key = (tuple(x.shape), tuple(w.shape), w.data_ptr())
        plan = self._plans.get(key)
        if plan is None:
            try:
                plan = ConvPlan(x.shape, w.shape, pad, stride, dil, self.padding_value, self._kernel, x.device)
            except TsbError as e:
                raise EjectionException(e.message)
            plan.set_weights(w, stream)
            self._plans[key] = plan
        if self._dq_dev is None or self._dq_dev.device != x.device:
            self._dq_dev = torch.from_numpy(self.dequantize_scales).to(x.device)
        out = torch.empty(proto[1], dtype=torch.float32, device=x.device)
        plan.run(x, LAYOUT_NCHW, self._dq_dev, out_f32=out, out_acc=out_acc, stream=stream)
        return out


def add_bias(x, bias, stream=None):
    """Operator "add_bias", format NCHW (src/kernels/gpu/add_bias.cu:19-26)."""
    x = x.contiguous()
    y = torch.empty_like(x)
    n, c = x.shape[0], x.shape[1]
    check(_lib.load().tsb_add_bias_f32_nchw(_ptr(x), _ptr(y), n, c, x.numel() // (n * c), _ptr(bias), _stream_ptr(stream)))
    return y


def relu(x, stream=None):
    x = x.contiguous()
    y = torch.empty_like(x)
    check(_lib.load().tsb_relu_f32(_ptr(x), _ptr(y), x.numel(), _stream_ptr(stream)))
    return y


def leaky_relu(x, scale, stream=None):
    x = x.contiguous()
    y = torch.empty_like(x)
    check(_lib.load().tsb_leaky_relu_f32(_ptr(x), _ptr(y), x.numel(), float(scale), _stream_ptr(stream)))
    return y


def quantize_nchw_to_nhwc(x, scales, stream=None):
    """fp32 NCHW -> int8 NHWC_PAD with the arithmetic of "quantize"."""
    x = x.contiguous()
    n, c, h, w = x.shape
    y = torch.empty((n, h, w, padded_channels(c)), dtype=torch.int8, device=x.device)
    check(_lib.load().tsb_quantize_f32_nchw_to_nhwc(_ptr(x), _ptr(y), n, c, h, w, float_array(scales), len(scales),
                                                    _stream_ptr(stream)))
    return y


def repack_nchw_to_nhwc(x, stream=None):
    x = x.contiguous()
    n, c, h, w = x.shape
    y = torch.empty((n, h, w, padded_channels(c)), dtype=torch.int8, device=x.device)
    check(_lib.load().tsb_repack_i8_nchw_to_nhwc(_ptr(x), _ptr(y), n, c, h, w, _stream_ptr(stream)))
    return y


def repack_nhwc_to_nchw(x, channels, stream=None):
    x = x.contiguous()
    n, h, w, _ = x.shape
    y = torch.empty((n, channels, h, w), dtype=torch.int8, device=x.device)
    check(_lib.load().tsb_repack_i8_nhwc_to_nchw(_ptr(x), _ptr(y), n, channels, h, w, _stream_ptr(stream)))
    return y
