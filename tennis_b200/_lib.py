"""ctypes binding of libtennis_b200.so (the C ABI declared in include/tennis_b200.h).

There is no CPU fallback: if the CUDA library has not been built, loading fails with an error that says how
to build it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtennis_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_WORKSPACE_TOO_SMALL = -3
ERR_DEVICE_TIMEOUT = -4

ACT_NONE, ACT_RELU, ACT_LEAKY_RELU = 0, 1, 2
LAYOUT_NCHW, LAYOUT_NHWC_PAD, LAYOUT_STAGED = 0, 1, 2
KERNEL_AUTO, KERNEL_DIRECT, KERNEL_TCGEN05 = 0, 1, 2
TUNE_AUTO, TUNE_OFF, TUNE_ON = 0, 1, 2
MAX_REQUANT_SCALES = 128


class ConvDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "n", "c", "h", "w", "o", "kh", "kw", "pad_top", "pad_bottom", "pad_left", "pad_right",
        "stride_h", "stride_w", "dilation_h", "dilation_w")] + [("padding_value", ctypes.c_float),
                                                                 ("kernel", ctypes.c_int),
                                                                 ("mma_orientation", ctypes.c_int),
                                                                 ("raw_row_mode", ctypes.c_int),
                                                                 ("patch_mode", ctypes.c_int)]


class ConvEpilogue(ctypes.Structure):
    _fields_ = [
        ("dequantize_scales", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("activation", ctypes.c_int),
        ("leaky_scale", ctypes.c_float),
        ("out_f32", ctypes.c_void_p),
        ("out_f32_layout", ctypes.c_int),
        ("out_i8", ctypes.c_void_p),
        ("out_i8_layout", ctypes.c_int),
        ("requant_scales_host", ctypes.POINTER(ctypes.c_float)),
        ("n_requant_scales", ctypes.c_int),
        ("out_acc", ctypes.c_void_p),
        ("residual_after_activation", ctypes.c_int),
    ]


# name -> (restype, argtypes); every symbol include/tennis_b200.h declares
_vp, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t
_fp = ctypes.POINTER(ctypes.c_float)
SYMBOLS = {
    "tsb_last_error": (ctypes.c_char_p, []),
    "tsb_status_string": (ctypes.c_char_p, [_i]),
    "tsb_version": (_i, []),
    "tsb_padded_channels": (_i, [_i]),
    "tsb_quantize_f32_i8": (_i, [_vp, _vp, _i64, _fp, _i, _vp]),
    "tsb_quantize_f64_i8": (_i, [_vp, _vp, _i64, _fp, _i, _vp]),
    "tsb_quantize_f32_i8_static": (_i, [_vp, _vp, _i64, _fp, _i, _vp]),
    "tsb_quantize_f32_nchw_to_nhwc": (_i, [_vp, _vp, _i, _i, _i, _i, _fp, _i, _vp]),
    "tsb_repack_i8_nchw_to_nhwc": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "tsb_repack_i8_nhwc_to_nchw": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "tsb_conv2d_i8_plan_create": (_i, [ctypes.POINTER(ConvDesc), ctypes.POINTER(_vp)]),
    "tsb_conv2d_i8_plan_destroy": (_i, [_vp]),
    "tsb_conv2d_i8_output_shape": (_i, [_vp, ctypes.POINTER(_i)]),
    "tsb_conv2d_i8_kernel": (_i, [_vp]),
    "tsb_conv2d_i8_plan_describe": (_i, [_vp, ctypes.c_char_p, _sz]),
    "tsb_conv2d_i8_workspace_bytes": (_sz, [_vp]),
    "tsb_conv2d_i8_set_weights": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "tsb_conv2d_i8_quantize_input": (_i, [_vp, _vp, _fp, _i, _vp, _sz, _vp]),
    "tsb_conv2d_i8_run": (_i, [_vp, _vp, _i, ctypes.POINTER(ConvEpilogue), _vp, _sz, _vp]),
    "tsb_conv2d_i8_run_projected": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(ConvEpilogue), _i, _vp, _sz, _vp]),
    "tsb_conv2d_i8_run_concat": (_i, [_vp, _vp, _vp, _vp, ctypes.POINTER(ConvEpilogue), _i, _vp, _sz, _vp]),
    "tsb_conv2d_i8_status": (_i, [_vp, _vp, _vp]),
    "tsb_conv2d_i8_status_async": (_i, [_vp, _vp, _vp, _vp]),
    "tsb_conv2d_i8_set_status_word": (_i, [_vp, _vp]),
    "tsb_conv2d_i8_status_decode": (_i, [_i]),
    "tsb_conv2d_host_scratch_bytes": (_sz, [_vp]),
    "tsb_conv2d_quantized_host": (_i, [_vp, _vp, _fp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _sz, _i, _vp]),
    "tsb_conv2d_quantized_host_async": (_i, [_vp, _vp, _fp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _sz, _i, _vp]),
    "tsb_add_bias_f32_nchw": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "tsb_relu_f32": (_i, [_vp, _vp, _i64, _vp]),
    "tsb_leaky_relu_f32": (_i, [_vp, _vp, _i64, _f, _vp]),
    "tsb_pool_out_dim": (_i, [_i, _i, _i, _i, _i]),
    "tsb_maxpool_i8_nhwc": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tsb_global_avgpool_f32_nhwc": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "tsb_inner_prod_f32": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "tsb_concat_i8_nhwc": (_i, [_vp, _i, _vp, _i, _vp, _i64, _vp]),
    "tsb_kernel_launch_count": (_i64, []),
}

_lib = None


class TsbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("tennis_b200 status %d: %s" % (status, message))
        self.status = status
        self.message = message


def load():
    """Load the CUDA library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "tennis_b200: %s is missing -- the CUDA library has not been built (python -c 'import __graft_entry__ as g; "
            "g.build()' or make -C tennis_b200/csrc); there is no CPU fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status):
    if status != OK:
        raise TsbError(status, load().tsb_last_error().decode(errors="replace"))


def float_array(values):
    values = [float(v) for v in values]
    return (ctypes.c_float * len(values))(*values)
