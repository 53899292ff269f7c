"""Files the stock TenniS tools replay: BASELINE configurations 0 and 1 as tools/run_test case folders, run by the
reference's own run_test binary (built from the reference's tools/run_test.cpp with this repo's operators linked in) on
device gpu; and a ResNet-50 module file written from Python, loaded with Module::Load and run on both devices."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from oracle import oracle as orc
from tennis_b200 import nets, tsfile
import run_test_cases

pytestmark = pytest.mark.gpu

RUN_TEST = os.path.join(ROOT, "tests", "plugin", "run_test")
WORKBENCH = os.path.join(ROOT, "tennis_b200", "libtennis_b200_workbench.so")


@pytest.mark.skipif(not os.path.exists(RUN_TEST), reason="tests/plugin/run_test was not built (needs the reference's sources)")
@pytest.mark.skipif(not orc.Reference.available(), reason="oracle/_ref/libtsref.so not built")
def test_run_test_replays_configurations_0_and_1_on_gpu(tmp_path):
    ref = orc.Reference(threads=1)
    names = []
    for spec in [run_test_cases.CONFIG0] + run_test_cases.CONFIG1:
        names += run_test_cases.write_layer_cases(str(tmp_path), spec, ref)
    assert len(names) == 24
    done = subprocess.run([RUN_TEST, str(tmp_path), "gpu"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=600)
    text = done.stdout.decode(errors="replace")
    ok = re.findall(r"^\[OK\]: (\S+) on", text, flags=re.M)
    assert done.returncode == 0, text[-3000:]
    assert "[OK]: 24, [SKIP]: 0, [WARNING]: 0, [FAILED]: 0" in text, text[-3000:]      # run_test's own summary line
    assert sorted(os.path.basename(n) for n in ok) == sorted(names), text[-3000:]


@pytest.mark.skipif(not os.path.exists(WORKBENCH), reason="tennis_b200/libtennis_b200_workbench.so was not built")
def test_resnet50_module_file_runs_unchanged_on_gpu(tmp_path):
    """The 53-convolution network of nets.resnet_spec written as a .tsm from Python (no TenniS library involved), then
    Module::Load + Workbench::Load + run on the cpu and on the gpu device: all 53 layers become fused nodes, and the
    logits agree (the average pool and inner product behind the trunk are the two devices' own floating-point
    reductions, hence a tolerance; the trunk itself is compared bit for bit in test_gpu_plugin.py)."""
    batch, image = 2, 64
    spec = nets.resnet_spec(image=image)
    params = nets.make_params(spec, seed=1)
    convs = spec["convs"]
    bn = [np.float32(1.0 / (73.0 * 30.0 * np.sqrt(c["c"] * c["k"] ** 2) * 0.0055)) for c in convs]
    act = [np.float32(127.0 / 3.0)] + [np.float32(127.0 / 4.0)] * (len(convs) - 1)
    g, inputs, outputs = tsfile.resnet_graph(spec, params, batch, act[0], act,
                                             lambda i: nets.dequantize_scales(params["convs"][i]["sw"], bn[i], act[i]))
    path = str(tmp_path / "resnet50.tsm")
    tsfile.write_module(path, g.nodes, inputs, outputs)
    x = np.random.default_rng(2).standard_normal((batch, 3, image, image), dtype=np.float32)

    lib = ctypes.CDLL(WORKBENCH)
    fptr, iptr = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int)
    lib.tsb_workbench_run_tsm.argtypes = [ctypes.c_char_p, ctypes.c_char_p, fptr, iptr, ctypes.c_int, fptr, ctypes.c_long, iptr,
                                          ctypes.POINTER(ctypes.c_double), ctypes.c_char_p, ctypes.c_int]
    results = {}
    for device in ("cpu", "gpu"):
        out = np.zeros((batch, 1000), dtype=np.float32)
        shape = (ctypes.c_int * 9)()
        counters = (ctypes.c_double * 4)()
        msg = ctypes.create_string_buffer(512)
        rc = lib.tsb_workbench_run_tsm(os.fsencode(path), device.encode(), x.ctypes.data_as(fptr), (ctypes.c_int * 4)(*x.shape), 4,
                                       out.ctypes.data_as(fptr), out.size, shape, counters, msg, 512)
        assert rc == 0, msg.value.decode(errors="replace")
        assert list(shape[:3]) == [2, batch, 1000]
        results[device] = (out, list(counters))
    assert results["cpu"][1][0] == 0                      # nothing of this library runs on the cpu device
    assert results["gpu"][1][:3] == [53, 32, 16]          # fused nodes, int8 hand-overs, shortcuts in the epilogue
    want, got = results["cpu"][0], results["gpu"][0]
    assert np.abs(want).max() > 1e-3
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
