"""TenniS file formats, written and read without the TenniS library: `.t` tensors, `.tsm` modules, and the case folders
that the reference's tools/run_test replays.

Formats (all integers little-endian):
  tensor file   Tensor::serialize, src/core/tensor.cpp:314-375:
                u32 field count, then per field  u8 dtype, u32 dims, u32 x dims shape, the elements
  module file   Module::Save, src/module/module.cpp:239-274, with src/module/header.cpp:10-16 (u32 fake, u32 code
                0x19910929, 120 reserved bytes), src/module/menu.cpp:88-118 (graph: u32 node count, per node the bubble
                and a u32 list of input node indices) and src/module/bubble.cpp:140-178 (bubble: u32 parameter count,
                per parameter u32 name length, the name, the value as a tensor file body; "#op" and "#name" are
                parameters like the others):
                header, u32 list of input nodes, u32 list of output nodes, graph
  case folder   tools/run_test/test_case.hpp:330-420:  0.<operator>.txt holding "params inputs outputs",
                1.<parameter>.t, 2.input_<i>.t, 3.output_<i>.t

Values are numpy arrays; a Python str stands for a CHAR8 tensor (tensor::from(std::string)), a list or tuple of arrays
for a packed tensor with several fields.
"""
import os
import struct

import numpy as np

MODULE_CODE_V1 = 0x19910929     # include/module/header.h

# include/core/dtype.h:11-37
VOID, INT8, UINT8, INT16, UINT16, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64 = range(12)
CHAR8 = 13
BOOLEAN = 21

_NUMPY_OF = {INT8: np.int8, UINT8: np.uint8, INT16: np.int16, UINT16: np.uint16, INT32: np.int32, UINT32: np.uint32,
             INT64: np.int64, UINT64: np.uint64, FLOAT16: np.float16, FLOAT32: np.float32, FLOAT64: np.float64,
             BOOLEAN: np.bool_}
_CODE_OF = {np.dtype(v): k for k, v in _NUMPY_OF.items()}


class Char8(str):
    """A CHAR8 tensor read back from a file."""


# ---- tensors --------------------------------------------------------------------------------------------------------
def _write_field(f, value):
    if isinstance(value, str):
        data = value.encode("utf-8")
        f.write(struct.pack("<BII", CHAR8, 1, len(data)))
        f.write(data)
        return
    a = np.asarray(value)
    if a.dtype not in _CODE_OF:
        raise TypeError("no TenniS dtype for numpy dtype %s" % a.dtype)
    if a.ndim == 0:
        a = a.reshape(1)           # tensor::build of a scalar makes shape [1] (src/core/tensor_builder.cpp:315-320)
    a = np.ascontiguousarray(a).astype(a.dtype.newbyteorder("<"), copy=False)
    f.write(struct.pack("<BI", _CODE_OF[a.dtype], a.ndim))
    f.write(struct.pack("<%dI" % a.ndim, *a.shape))
    f.write(a.tobytes())


def write_tensor(f, value):
    """Tensor::serialize into an open binary file."""
    fields = list(value) if isinstance(value, (list, tuple)) else [value]
    f.write(struct.pack("<I", len(fields)))
    for field in fields:
        _write_field(f, field)


def _read_exact(f, n):
    data = f.read(n)
    if len(data) != n:
        raise EOFError("truncated TenniS file: wanted %d bytes, got %d" % (n, len(data)))
    return data


def _read_field(f):
    dtype, dims = struct.unpack("<BI", _read_exact(f, 5))
    shape = struct.unpack("<%dI" % dims, _read_exact(f, 4 * dims)) if dims else ()
    count = int(np.prod(shape, dtype=np.int64)) if dims else 1
    if dtype == CHAR8:
        return Char8(_read_exact(f, count).decode("utf-8"))
    if dtype not in _NUMPY_OF:
        raise TypeError("TenniS dtype %d has no numpy counterpart here" % dtype)
    np_dtype = np.dtype(_NUMPY_OF[dtype]).newbyteorder("<")
    return np.frombuffer(_read_exact(f, count * np_dtype.itemsize), dtype=np_dtype).reshape(shape).copy()


def read_tensor(f):
    """Tensor::externalize: one array, or a list of arrays for a packed tensor."""
    (fields,) = struct.unpack("<I", _read_exact(f, 4))
    out = [_read_field(f) for _ in range(fields)]
    return out[0] if fields == 1 else out


def save_tensor(path, value):
    """tensor::save (include/core/tensor_builder.h:153-159)."""
    with open(path, "wb") as f:
        write_tensor(f, value)


def load_tensor(path):
    """tensor::load."""
    with open(path, "rb") as f:
        return read_tensor(f)


# ---- modules --------------------------------------------------------------------------------------------------------
class Node:
    """One node of a TenniS graph: operator name, node name, attributes (name -> array | str) and input node indices."""

    def __init__(self, op, name, params=None, inputs=()):
        self.op, self.name = op, name
        self.params = dict(params or {})
        self.inputs = list(inputs)

    def __repr__(self):
        return "Node(%s:%s <- %s)" % (self.op, self.name, self.inputs)


class GraphBuilder:
    """Collects nodes; the methods return node indices, which is what inputs and outputs are made of."""

    def __init__(self):
        self.nodes = []

    def add(self, op, name, inputs=(), **params):
        if any(len(k.encode()) >= 32 for k in params):
            raise ValueError("parameter names are shorter than 32 bytes (doc/zh_CN/module.md, section 4)")
        self.nodes.append(Node(op, name, params, inputs))
        return len(self.nodes) - 1

    def param(self, name, dtype=None, shape=None):
        """bubble::param (src/module/menu.cpp:14-64)."""
        extra = {}
        if shape is not None:
            extra["#shape"] = np.asarray(shape, dtype=np.int32)
        if dtype is not None:
            extra["#dtype"] = np.asarray([dtype], dtype=np.int32)
        return self.add("<param>", name, **extra)

    def data(self, name, value):
        """bubble::data: a constant."""
        return self.add("<const>", name, value=value)


def _write_bubble(f, node):
    params = dict(node.params)
    params["#op"] = node.op
    params["#name"] = node.name
    f.write(struct.pack("<I", len(params)))
    for key in sorted(params):
        raw = key.encode("utf-8")
        f.write(struct.pack("<I", len(raw)))
        f.write(raw)
        write_tensor(f, params[key])


def write_module(path, nodes, inputs, outputs):
    """Module::Save, BINARY format.  nodes: list of Node (inputs by index into this list); inputs / outputs: node indices."""
    for i, node in enumerate(nodes):
        for j in node.inputs:
            if not 0 <= j < len(nodes):
                raise ValueError("node %d (%s) reads node %d, which does not exist" % (i, node.name, j))
    with open(path, "wb") as f:
        f.write(struct.pack("<II", 0, MODULE_CODE_V1))
        f.write(b"\0" * 120)
        for index_list in (inputs, outputs):
            f.write(struct.pack("<I", len(index_list)))
            f.write(struct.pack("<%dI" % len(index_list), *index_list))
        f.write(struct.pack("<I", len(nodes)))
        for node in nodes:
            _write_bubble(f, node)
            f.write(struct.pack("<I", len(node.inputs)))
            f.write(struct.pack("<%dI" % len(node.inputs), *node.inputs))


def read_module(path):
    """Module::Load: (nodes, inputs, outputs)."""
    with open(path, "rb") as f:
        fake, code = struct.unpack("<II", _read_exact(f, 8))
        if code != MODULE_CODE_V1:
            raise ValueError("not a TenniS module: header code 0x%08x" % code)
        _read_exact(f, 120)
        lists = []
        for _ in range(2):
            (n,) = struct.unpack("<I", _read_exact(f, 4))
            lists.append(list(struct.unpack("<%dI" % n, _read_exact(f, 4 * n))))
        (count,) = struct.unpack("<I", _read_exact(f, 4))
        nodes = []
        for _ in range(count):
            (nparams,) = struct.unpack("<I", _read_exact(f, 4))
            params = {}
            for _ in range(nparams):
                (klen,) = struct.unpack("<I", _read_exact(f, 4))
                key = _read_exact(f, klen).decode("utf-8")
                params[key] = read_tensor(f)
            (nin,) = struct.unpack("<I", _read_exact(f, 4))
            ins = list(struct.unpack("<%dI" % nin, _read_exact(f, 4 * nin)))
            op, name = str(params.pop("#op")), str(params.pop("#name"))
            nodes.append(Node(op, name, params, ins))
        if f.read(1):
            raise ValueError("bytes left over after the graph")
    return nodes, lists[0], lists[1]


# ---- run_test case folders ------------------------------------------------------------------------------------------
def write_case(folder, op, params, inputs, outputs):
    """One operator case for tools/run_test: attributes, input tensors and the wanted output tensors."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "0.%s.txt" % op), "w") as f:
        f.write("%d %d %d\n" % (len(params), len(inputs), len(outputs)))
    for key, value in params.items():
        save_tensor(os.path.join(folder, "1.%s.t" % key), value)
    for i, value in enumerate(inputs):
        save_tensor(os.path.join(folder, "2.input_%d.t" % i), value)
    for i, value in enumerate(outputs):
        save_tensor(os.path.join(folder, "3.output_%d.t" % i), value)


def read_case(folder):
    """(op, params, inputs, outputs) of a case folder."""
    op, counts, params, inputs, outputs = None, None, {}, {}, {}
    for name in sorted(os.listdir(folder)):
        path = os.path.join(folder, name)
        if name.startswith("0.") and name.endswith(".txt"):
            op = name[2:-4]
            counts = tuple(int(v) for v in open(path).read().split()[:3])
        elif name.startswith("1.") and name.endswith(".t"):
            params[name[2:-2]] = load_tensor(path)
        elif name.startswith("2.input_") and name.endswith(".t"):
            inputs[int(name[8:-2])] = load_tensor(path)
        elif name.startswith("3.output_") and name.endswith(".t"):
            outputs[int(name[9:-2])] = load_tensor(path)
    if op is None:
        raise ValueError("%s is not a run_test case folder" % folder)
    if counts != (len(params), len(inputs), len(outputs)):
        raise ValueError("%s: 0.%s.txt says %s, found %s" % (folder, op, counts, (len(params), len(inputs), len(outputs))))
    return op, params, [inputs[i] for i in range(len(inputs))], [outputs[i] for i in range(len(outputs))]


# ---- the quantized layers and networks of this package as TenniS graphs -----------------------------------------------
def conv_attributes(pad, stride, dequantize_scales, dilation=1, padding_value=None):
    """Attributes of conv2d_quantized (src/backend/base/base_conv2d_quantized.cpp:13-117), format NCHW."""
    pads = (pad,) * 4 if np.isscalar(pad) else tuple(pad)        # top, bottom, left, right
    strides = (stride,) * 2 if np.isscalar(stride) else tuple(stride)
    dil = (dilation,) * 2 if np.isscalar(dilation) else tuple(dilation)
    out = {"format": "NCHW",
           "padding": np.array([[0, 0], [0, 0], [pads[0], pads[1]], [pads[2], pads[3]]], dtype=np.int32),
           "stride": np.array([1, 1, strides[0], strides[1]], dtype=np.int32),
           "dilation": np.array([1, 1, dil[0], dil[1]], dtype=np.int32),
           "dequantize_scales": np.asarray(dequantize_scales, dtype=np.float32)}
    if padding_value is not None:
        out["padding_value"] = np.array([padding_value], dtype=np.float32)
    return out


def quantized_layer(g, name, x, batch, in_scale, w, dq, bias, stride, pad, activation="relu", leaky=0.1, shortcut=None,
                    shortcut_after=False):
    """quantize -> conv2d_quantized -> add_bias [-> add shortcut] [-> relu | leaky_relu] [-> add shortcut], as a model
    converter writes a quantized layer; returns the index of the layer's last node."""
    q = g.add("quantize", name + ".q", [x], quantize_scale=np.full(batch, in_scale, dtype=np.float32))
    wn = g.data(name + ".w", np.asarray(w, dtype=np.int8))
    conv = g.add("conv2d_quantized", name + ".conv", [q, wn], **conv_attributes(pad, stride, dq))
    bn = g.data(name + ".b", np.asarray(bias, dtype=np.float32))
    y = g.add("add_bias", name + ".biased", [conv, bn], format="NCHW")
    if shortcut is not None and not shortcut_after:
        y = g.add("add", name + ".sum", [y, shortcut])
    if activation == "relu":
        y = g.add("relu", name + ".act", [y])
    elif activation == "leaky_relu":
        y = g.add("leaky_relu", name + ".act", [y], scale=np.array([leaky], dtype=np.float32))
    elif activation is not None:
        raise ValueError("activation %r" % (activation,))
    if shortcut is not None and shortcut_after:
        y = g.add("add", name + ".sum", [y, shortcut])
    return y


def resnet_graph(spec, params, batch, input_scale, act_scales, dq_of):
    """The bottleneck ResNet of nets.resnet_spec as a TenniS graph.  act_scales[i]: quantize scale of the input of
    convolution i; dq_of(i): its per-channel dequantize scales.  Returns (GraphBuilder, inputs, outputs)."""
    g = GraphBuilder()
    convs, P = spec["convs"], params["convs"]
    x = g.param("x", FLOAT32, (batch, 3, spec["image"], spec["image"]))

    def layer(i, src, **kw):
        c = convs[i]
        return quantized_layer(g, c["name"], src, batch, act_scales[i], P[i]["w"], dq_of(i), P[i]["bias"], c["stride"], c["pad"], **kw)

    y = layer(0, x)
    # pooling2d 3x3 / 2, padding {top 1, bottom 0, left 1, right 0}: the reference's output extent rounds up
    # (include/backend/common_function.h:13-20), so this is the usual pool with padding 1
    y = g.add("pooling2d", "pool", [y], format="NCHW", type=np.array([0], dtype=np.int32),
              padding=np.array([[0, 0], [0, 0], [1, 0], [1, 0]], dtype=np.int32),
              ksize=np.array([1, 1, 3, 3], dtype=np.int32), stride=np.array([1, 1, 2, 2], dtype=np.int32))
    for stage in spec["stages"]:
        for b in stage:
            a = layer(b["conv1"], y)
            a = layer(b["conv2"], a)
            shortcut = layer(b["proj"], y, activation=None) if b["projection"] else y
            y = layer(b["conv3"], a, shortcut=shortcut)
    y = g.add("global_pooling2d", "gap", [y], format="NCHW", type=np.array([1], dtype=np.int32))
    y = g.add("flatten", "flat", [y])
    fc_w = g.data("fc.w", np.ascontiguousarray(np.asarray(params["fc_w"], dtype=np.float32).T))     # [features, classes]
    y = g.add("inner_prod", "fc", [y, fc_w])
    fc_b = g.data("fc.b", np.asarray(params["fc_b"], dtype=np.float32))
    y = g.add("add_bias", "logits", [y, fc_b], dim=np.array([1], dtype=np.int32))
    return g, [x], [y]
