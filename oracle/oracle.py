"""numpy front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two checkers with the same call signatures:

* ``Port``  -- liboracle.so, the C restatement in oracle.c (always buildable);
* ``Reference`` -- _ref/libtsref.so, the reference's own CPU operators compiled from its sources and driven
  through Workbench::offline_run with one computing thread (ref_driver.cpp).  Present only where the
  reference tree was available at build time (the prebuilt library travels with the repository snapshot).

Only tests, the smoke check and the benchmark's CPU arm import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_c_int_p = ctypes.POINTER(ctypes.c_int)


def usable_cpus():
    """Host threads this process may really use: the affinity mask, cut down by a cgroup CPU quota when there is one.
    os.cpu_count() alone over-subscribes containers that see all of a big host's cores but may run on a few."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    for path in ("/sys/fs/cgroup/cpu.max", "/sys/fs/cgroup/cpu/cpu.cfs_quota_us"):
        try:
            text = open(path).read().split()
            if path.endswith("cpu.max"):
                quota, period = text[0], float(text[1])
            else:
                quota, period = text[0], float(open("/sys/fs/cgroup/cpu/cpu.cfs_period_us").read())
            if quota not in ("max", "-1") and period > 0:
                n = min(n, max(1, int(float(quota) / period)))
            break
        except (OSError, ValueError, IndexError):
            continue
    return max(1, n)


def limit_openmp(max_threads=None):
    """Keeps the OpenMP runtimes of the checker libraries from spawning one spinning thread per visible core."""
    n = min(usable_cpus(), max_threads or 16)
    os.environ.setdefault("OMP_NUM_THREADS", str(n))
    os.environ.setdefault("OMP_WAIT_POLICY", "PASSIVE")
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(os.environ["OMP_NUM_THREADS"]))
    except (OSError, AttributeError, ValueError):
        pass
    return n


def _ptr(a, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _ints(values):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


def reference_root():
    """Where the reference's source tree lies, or None: $TENNIS_REFERENCE if set, else the Makefile's default REF."""
    path = os.environ.get("TENNIS_REFERENCE")
    if not path:
        for line in open(os.path.join(_HERE, "Makefile")):
            if line.startswith("REF") and "?=" in line:
                path = line.split("?=", 1)[1].strip()
                break
    return path if path and os.path.isdir(os.path.join(path, "src")) else None


def build(force=False):
    """Compile liboracle.so (and _ref/ when the reference sources are present)."""
    lib = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(os.path.join(_HERE, "oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
    # the reference build (324 files) only where its sources are present and the library is missing or older than
    # its driver; a prebuilt library is used as it is
    ref_lib = os.path.join(_HERE, "_ref", "libtsref.so")
    stale = not os.path.exists(ref_lib) or os.path.getmtime(ref_lib) < os.path.getmtime(os.path.join(_HERE, "ref_driver.cpp"))
    ref = reference_root()
    if ref and (force or stale):
        subprocess.check_call(["make", "-C", _HERE, "-j8", "ref", "REF=" + ref], stdout=subprocess.DEVNULL)


def conv_out_dim(x, pad_lo, pad_hi, k, stride, dilation):
    """include/backend/common_function.h:30-40 (C integer division truncates toward zero)."""
    num = x + pad_lo + pad_hi - (dilation * (k - 1) + 1)
    q = abs(num) // stride
    return (q if num >= 0 else -q) + 1


class Port:
    """C restatement (oracle.c)."""

    kind = "port"

    def __init__(self):
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        limit_openmp()
        self.lib = ctypes.CDLL(path)
        self.lib.orc_quantize_group_len.restype = ctypes.c_int

    def quantize(self, x, scales):
        x = np.ascontiguousarray(x, dtype=np.float32)
        s = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        y = np.zeros(x.shape, dtype=np.int8)
        self.lib.orc_quantize_f32(_ptr(x, ctypes.c_float), ctypes.c_int(x.size), _ptr(s, ctypes.c_float),
                                  ctypes.c_int(s.size), _ptr(y, ctypes.c_int8))
        return y

    def quantize_f64(self, x, scales):
        """quantize of a FLOAT64 tensor (src/kernels/cpu/quantize.cpp:38-67,134)."""
        x = np.ascontiguousarray(x, dtype=np.float64)
        s = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        y = np.zeros(x.shape, dtype=np.int8)
        self.lib.orc_quantize_f64(_ptr(x, ctypes.c_double), ctypes.c_int(x.size), _ptr(s, ctypes.c_float),
                                  ctypes.c_int(s.size), _ptr(y, ctypes.c_int8))
        return y

    def max_pooling2d(self, x, k, stride, pad):
        """pooling2d, type max, NCHW fp32, pad = (top, bottom, left, right); the reference's ceil-mode extent."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        N, C, H, W = x.shape
        self.lib.orc_pool_out_dim.restype = ctypes.c_int
        OH = self.lib.orc_pool_out_dim(H, int(pad[0]), int(pad[1]), int(k), int(stride))
        OW = self.lib.orc_pool_out_dim(W, int(pad[2]), int(pad[3]), int(k), int(stride))
        y = np.zeros((N, C, max(OH, 0), max(OW, 0)), dtype=np.float32)
        rc = self.lib.orc_max_pooling2d(_ptr(x, ctypes.c_float), N, C, H, W, int(k), int(stride), int(pad[0]), int(pad[1]),
                                        int(pad[2]), int(pad[3]), _ptr(y, ctypes.c_float))
        if rc != 0:
            raise ValueError("a pooling window lies entirely in the padding")
        return y

    def conv2d_quantized(self, x, w, pad, stride, dilation, dq, padding_value=0.0, return_acc=False):
        x = np.ascontiguousarray(x, dtype=np.int8)
        w = np.ascontiguousarray(w, dtype=np.int8)
        dq = np.ascontiguousarray(dq, dtype=np.float32)
        N, C, H, W = x.shape
        O, _, KH, KW = w.shape
        OH = conv_out_dim(H, pad[0], pad[1], KH, stride[0], dilation[0])
        OW = conv_out_dim(W, pad[2], pad[3], KW, stride[1], dilation[1])
        out = np.zeros((N, O, OH, OW), dtype=np.float32)
        acc = np.zeros((N, O, OH, OW), dtype=np.int32)
        rc = self.lib.orc_conv2d_quantized(
            _ptr(x, ctypes.c_int8), N, C, H, W, _ptr(w, ctypes.c_int8), O, KH, KW,
            int(pad[0]), int(pad[1]), int(pad[2]), int(pad[3]), ctypes.c_float(padding_value),
            int(stride[0]), int(stride[1]), int(dilation[0]), int(dilation[1]),
            _ptr(dq, ctypes.c_float), _ptr(out, ctypes.c_float), _ptr(acc, ctypes.c_int32))
        if rc != 0:
            raise ValueError("empty convolution output")
        return (out, acc) if return_acc else out

    def add_bias(self, x, bias):
        x = np.ascontiguousarray(x, dtype=np.float32)
        b = np.ascontiguousarray(bias, dtype=np.float32)
        y = np.empty_like(x)
        N, C = x.shape[0], x.shape[1]
        self.lib.orc_add_bias_nchw(_ptr(x, ctypes.c_float), N, C, int(x.size // (N * C)), _ptr(b, ctypes.c_float),
                                   _ptr(y, ctypes.c_float))
        return y

    def relu(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.orc_relu(_ptr(x, ctypes.c_float), ctypes.c_size_t(x.size), _ptr(y, ctypes.c_float))
        return y

    def leaky_relu(self, x, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.orc_leaky_relu(_ptr(x, ctypes.c_float), ctypes.c_size_t(x.size), ctypes.c_float(scale),
                                _ptr(y, ctypes.c_float))
        return y

    # --- compositions (the same operator sequence a quantized TenniS graph carries) ---
    def activation(self, y, act, leaky=0.0):
        if act in (1, "relu"):
            return self.relu(y)
        if act in (2, "leaky_relu"):
            return self.leaky_relu(y, leaky)
        return y

    def conv_block(self, xq, w, pad, stride, dilation, dq, bias=None, act=0, leaky=0.0, residual=None,
                   requant_scales=None, padding_value=0.0, residual_after_activation=False):
        """conv2d_quantized -> add_bias -> [+ residual] -> relu|leaky_relu -> [+ residual] -> [quantize]; the residual
        (operator "add", fp32) comes before the activation (ResNet) or after it (Darknet shortcut)."""
        y = self.conv2d_quantized(xq, w, pad, stride, dilation, dq, padding_value)
        if bias is not None:
            y = self.add_bias(y, bias)
        if residual is not None and not residual_after_activation:
            y = (y + np.asarray(residual, dtype=np.float32)).astype(np.float32)
        y = self.activation(y, act, leaky)
        if residual is not None and residual_after_activation:
            y = (y + np.asarray(residual, dtype=np.float32)).astype(np.float32)
        if requant_scales is not None:
            return y, self.quantize(y, requant_scales)
        return y


class Reference(Port):
    """The reference's compiled CPU operators (ref_driver.cpp); one computing thread unless told otherwise."""

    kind = "reference"

    def __init__(self, threads=1):
        path = os.path.join(_HERE, "_ref", "libtsref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        limit_openmp()
        self.ref = ctypes.CDLL(path)
        self.ref.tsref_last_error.restype = ctypes.c_char_p
        self.threads = threads

    @staticmethod
    def available():
        return os.path.exists(os.path.join(_HERE, "_ref", "libtsref.so"))

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.ref.tsref_last_error().decode(errors="replace"))

    def quantize(self, x, scales):
        x = np.ascontiguousarray(x, dtype=np.float32)
        s = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        y = np.zeros(x.shape, dtype=np.int8)
        self._check(self.ref.tsref_quantize(_ptr(x, ctypes.c_float), _ints(x.shape), x.ndim, _ptr(s, ctypes.c_float),
                                            int(s.size), _ptr(y, ctypes.c_int8), self.threads))
        return y

    def tensor_roundtrip(self, path_in, path_out=None):
        """tensor::load of a .t file by the reference (and tensor::save of what it read, when path_out is given).
        Returns (fields, dtype code of field 0, shape of field 0)."""
        info = _ints([0] * 11)
        self._check(self.ref.tsref_tensor_roundtrip(os.fsencode(path_in), os.fsencode(path_out) if path_out else None, info))
        return info[0], info[1], tuple(info[3:3 + info[2]])

    def run_module(self, path, x):
        """Module::Load of a .tsm file, Workbench::Load on the cpu device, one fp32 input, the fp32 output."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        shape = _ints([0] * 9)
        args = [os.fsencode(path), _ptr(x, ctypes.c_float), _ints(x.shape), x.ndim]
        self._check(self.ref.tsref_run_module(*args, None, ctypes.c_long(0), shape, None, self.threads))
        y = np.zeros(tuple(shape[1:1 + shape[0]]), dtype=np.float32)
        self._check(self.ref.tsref_run_module(*args, _ptr(y, ctypes.c_float), ctypes.c_long(y.size), shape, None, self.threads))
        return y

    def quantize_f64(self, x, scales):
        x = np.ascontiguousarray(x, dtype=np.float64)
        s = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        y = np.zeros(x.shape, dtype=np.int8)
        self._check(self.ref.tsref_quantize_f64(_ptr(x, ctypes.c_double), _ints(x.shape), x.ndim, _ptr(s, ctypes.c_float),
                                                int(s.size), _ptr(y, ctypes.c_int8), self.threads))
        return y

    def max_pooling2d(self, x, k, stride, pad):
        x = np.ascontiguousarray(x, dtype=np.float32)
        shape = _ints([0, 0, 0, 0])
        self._check(self.ref.tsref_max_pooling2d(_ptr(x, ctypes.c_float), _ints(x.shape), int(k), int(stride), _ints(pad),
                                                 None, shape, self.threads))
        y = np.zeros(tuple(shape), dtype=np.float32)
        self._check(self.ref.tsref_max_pooling2d(_ptr(x, ctypes.c_float), _ints(x.shape), int(k), int(stride), _ints(pad),
                                                 _ptr(y, ctypes.c_float), shape, self.threads))
        return y

    def conv2d_quantized(self, x, w, pad, stride, dilation, dq, padding_value=0.0, return_acc=False):
        if return_acc:
            raise NotImplementedError("the reference operator does not expose its int32 scratch")
        x = np.ascontiguousarray(x, dtype=np.int8)
        w = np.ascontiguousarray(w, dtype=np.int8)
        dq = np.ascontiguousarray(dq, dtype=np.float32)
        shape = _ints([0, 0, 0, 0])
        args = [_ptr(x, ctypes.c_int8), _ints(x.shape), _ptr(w, ctypes.c_int8), _ints(w.shape), _ints(pad),
                ctypes.c_float(padding_value), 1 if padding_value != 0.0 else 0,
                int(stride[0]), int(stride[1]), int(dilation[0]), int(dilation[1]),
                _ptr(dq, ctypes.c_float), int(dq.size)]
        N, O = x.shape[0], w.shape[0]
        OH = conv_out_dim(x.shape[2], pad[0], pad[1], w.shape[2], stride[0], dilation[0])
        OW = conv_out_dim(x.shape[3], pad[2], pad[3], w.shape[3], stride[1], dilation[1])
        out = np.zeros((N, O, max(OH, 0), max(OW, 0)), dtype=np.float32)
        self._check(self.ref.tsref_conv2d_quantized(*args, _ptr(out, ctypes.c_float), shape, self.threads))
        assert list(shape) == list(out.shape), (list(shape), out.shape)
        return out

    def add_bias(self, x, bias):
        x = np.ascontiguousarray(x, dtype=np.float32)
        b = np.ascontiguousarray(bias, dtype=np.float32)
        y = np.empty_like(x)
        self._check(self.ref.tsref_add_bias(_ptr(x, ctypes.c_float), _ints(x.shape), x.ndim, _ptr(b, ctypes.c_float),
                                            int(b.size), _ptr(y, ctypes.c_float), self.threads))
        return y

    def relu(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self._check(self.ref.tsref_relu(_ptr(x, ctypes.c_float), _ints(x.shape), x.ndim, _ptr(y, ctypes.c_float),
                                        self.threads))
        return y

    def leaky_relu(self, x, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self._check(self.ref.tsref_leaky_relu(_ptr(x, ctypes.c_float), _ints(x.shape), x.ndim, ctypes.c_float(scale),
                                              _ptr(y, ctypes.c_float), self.threads))
        return y

    def time_layer(self, x, w, pad, stride, dilation, qscale, dq, bias, act=1, leaky=0.0, workers=1, repeats=1):
        """Seconds for quantize -> conv2d_quantized -> add_bias -> act on `workers` host threads, each its own
        Workbench over the whole of x.  Returns (seconds per repeat, seconds spent in quantize)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.int8)
        dq = np.ascontiguousarray(dq, dtype=np.float32)
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        sec = ctypes.c_double(0)
        qsec = ctypes.c_double(0)
        N, C, H, W = x.shape
        O, _, KH, KW = w.shape
        self._check(self.ref.tsref_time_layer(
            _ptr(x, ctypes.c_float), N, C, H, W, _ptr(w, ctypes.c_int8), O, KH, KW, _ints(pad),
            int(stride[0]), int(stride[1]), int(dilation[0]), int(dilation[1]), ctypes.c_float(qscale),
            _ptr(dq, ctypes.c_float), _ptr(bias, ctypes.c_float), int(act), ctypes.c_float(leaky),
            int(workers), int(repeats), ctypes.byref(sec), ctypes.byref(qsec)))
        return sec.value, qsec.value


def best():
    """The strongest checker present: the compiled reference if it is here, else the port."""
    return Reference() if Reference.available() else Port()
