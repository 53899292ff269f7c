"""tennis_b200.tsfile against the reference's own readers and writers (oracle/_ref/libtsref.so: tensor::load / save,
Module::Load + Workbench::Load on the cpu device): .t tensors byte for byte, a .tsm module written from Python loaded,
compiled and run by the reference, and the run_test case folder layout."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from oracle import chains
from tennis_b200 import nets, tsfile

needs_reference = pytest.mark.skipif(not orc.Reference.available(), reason="oracle/_ref/libtsref.so not built")


@pytest.mark.parametrize("value, code", [
    (np.arange(-60, 60, dtype=np.int8).reshape(2, 3, 4, 5), tsfile.INT8),
    (np.linspace(-3, 3, 77, dtype=np.float32).reshape(7, 11), tsfile.FLOAT32),
    (np.array([[0, 0], [0, 0], [1, 2], [3, 4]], dtype=np.int32), tsfile.INT32),
    (np.array([0.5], dtype=np.float64), tsfile.FLOAT64),
    (np.zeros((0, 4), dtype=np.float32), tsfile.FLOAT32),
    ("NCHW", tsfile.CHAR8),
])
@needs_reference
def test_tensor_file_is_what_the_reference_reads_and_writes(tmp_path, value, code):
    ref = orc.Reference()
    mine, theirs = str(tmp_path / "mine.t"), str(tmp_path / "theirs.t")
    tsfile.save_tensor(mine, value)
    fields, dtype, shape = ref.tensor_roundtrip(mine, theirs)
    assert fields == 1 and dtype == code
    assert shape == ((len(value),) if isinstance(value, str) else value.shape)
    assert open(mine, "rb").read() == open(theirs, "rb").read()      # tensor::save writes the same bytes
    back = tsfile.load_tensor(theirs)
    if isinstance(value, str):
        assert back == value
    else:
        assert back.dtype == value.dtype and np.array_equal(back, value)


@needs_reference
def test_packed_tensor_file(tmp_path):
    ref = orc.Reference()
    fields = [np.arange(6, dtype=np.float32).reshape(2, 3), np.array([1, 2, 3], dtype=np.int8)]
    mine, theirs = str(tmp_path / "mine.t"), str(tmp_path / "theirs.t")
    tsfile.save_tensor(mine, fields)
    count, dtype, shape = ref.tensor_roundtrip(mine, theirs)
    assert (count, dtype, shape) == (2, tsfile.FLOAT32, (2, 3))
    assert open(mine, "rb").read() == open(theirs, "rb").read()
    back = tsfile.load_tensor(mine)
    assert len(back) == 2 and np.array_equal(back[0], fields[0]) and np.array_equal(back[1], fields[1])


def test_truncated_and_foreign_files_are_refused(tmp_path):
    path = str(tmp_path / "x.t")
    tsfile.save_tensor(path, np.arange(10, dtype=np.int32))
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-3])
    with pytest.raises(EOFError):
        tsfile.load_tensor(path)
    open(path, "wb").write(b"\0" * 200)
    with pytest.raises(ValueError):
        tsfile.read_module(path)
    with pytest.raises(TypeError):
        tsfile.save_tensor(path, np.zeros(3, dtype=np.complex64))


def small_resnet(batch):
    """A bottleneck ResNet small enough for the CPU reference: 4 blocks (one per stage, all with projection shortcuts),
    17 convolutions, 32 x 32 input."""
    spec = nets.resnet_spec(image=32, widths=(8, 16, 32, 64), blocks=(1, 1, 1, 1), stem_channels=16, classes=10)
    params = nets.make_params(spec, seed=3)
    convs = spec["convs"]
    # activation scales and BatchNorm factors that keep every layer's output within a few units (stands in for calibration)
    bn = [np.float32(1.0 / (73.0 * 30.0 * np.sqrt(c["c"] * c["k"] ** 2) * 0.0055)) for c in convs]
    s = np.float32(127.0 / 4.0)
    scales = {"input": np.float32(127.0 / 3.0), "bn": bn,
              "convs": [((np.float32(127.0 / 3.0) if i == 0 else s), s) for i in range(len(convs))]}
    rng = np.random.default_rng(5)
    x = rng.standard_normal((batch, 3, 32, 32), dtype=np.float32)
    return spec, params, scales, x


def resnet_module_file(path, spec, params, scales, batch):
    act = [scales["convs"][i][0] for i in range(len(spec["convs"]))]
    g, inputs, outputs = tsfile.resnet_graph(
        spec, params, batch, scales["input"], act,
        lambda i: nets.dequantize_scales(params["convs"][i]["sw"], scales["bn"][i], act[i]))
    tsfile.write_module(path, g.nodes, inputs, outputs)
    return g


@needs_reference
def test_module_written_from_python_runs_in_the_reference(tmp_path):
    """The ResNet graph of tsfile.resnet_graph as a .tsm: the reference loads it (Module::Load), compiles it for its cpu
    device and runs it; the logits equal the operator-by-operator chain of the oracle."""
    batch = 2
    spec, params, scales, x = small_resnet(batch)
    path = str(tmp_path / "resnet_small.tsm")
    g = resnet_module_file(path, spec, params, scales, batch)
    nodes, inputs, outputs = tsfile.read_module(path)
    assert len(nodes) == len(g.nodes) and inputs == [0] and outputs == [len(nodes) - 1]
    assert sum(n.op == "conv2d_quantized" for n in nodes) == 17
    assert nodes[0].op == "<param>" and tuple(nodes[0].params["#shape"]) == (batch, 3, 32, 32)
    ref = orc.Reference()
    logits = ref.run_module(path, x)
    assert logits.shape == (batch, 10)
    _, _, want = chains.resnet_forward(spec, params, scales, x, orc.Port())
    # average pool and inner product are floating-point reductions whose order the oracle does not pin
    np.testing.assert_allclose(logits, want, rtol=1e-4, atol=1e-5)
    assert np.abs(want).max() > 1e-3          # ... and the comparison is not of zeros


def test_case_folder_layout(tmp_path):
    folder = str(tmp_path / "case")
    x = np.arange(24, dtype=np.float32).reshape(1, 2, 3, 4)
    scales = np.array([2.0], dtype=np.float32)
    tsfile.write_case(folder, "quantize", {"quantize_scale": scales}, [x], [(x * 2).astype(np.int8)])
    assert sorted(os.listdir(folder)) == ["0.quantize.txt", "1.quantize_scale.t", "2.input_0.t", "3.output_0.t"]
    assert open(os.path.join(folder, "0.quantize.txt")).read().split() == ["1", "1", "1"]
    op, params, inputs, outputs = tsfile.read_case(folder)
    assert op == "quantize" and np.array_equal(params["quantize_scale"], scales)
    assert np.array_equal(inputs[0], x) and outputs[0].dtype == np.int8


def test_conv_attributes_follow_the_operator():
    a = tsfile.conv_attributes((1, 2, 3, 4), (2, 1), np.ones(5, dtype=np.float32), dilation=2, padding_value=0.0)
    assert a["format"] == "NCHW" and a["padding"].tolist() == [[0, 0], [0, 0], [1, 2], [3, 4]]
    assert a["stride"].tolist() == [1, 1, 2, 1] and a["dilation"].tolist() == [1, 1, 2, 2]
    assert a["dequantize_scales"].dtype == np.float32 and a["padding_value"].tolist() == [0.0]
