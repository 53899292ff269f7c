"""Drop-in test: the TenniS operator classes of tennis_b200/plugin, registered on TenniS's "gpu" device, inside
the reference's own runtime (Workbench::Load of a graph built with its graph API, and offline_create/offline_run),
against the reference's CPU operators in the same process.  The driver is tests/plugin/plugin_driver.cpp."""
import ctypes
import os

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

DRIVER = os.path.join(ROOT, "tests", "plugin", "libplugin_driver.so")


@pytest.fixture(scope="module")
def driver():
    if not os.path.exists(DRIVER):
        pytest.skip("tests/plugin/libplugin_driver.so was not built (needs the reference sources at build time)")
    lib = ctypes.CDLL(DRIVER)
    lib.tsplug_selftest.argtypes = [ctypes.c_int] * 8 + [ctypes.c_uint, ctypes.c_char_p, ctypes.c_int]
    return lib


@pytest.mark.parametrize("case", [
    (2, 64, 14, 14, 96, 3, 1, 1),     # tensor-core kernel
    (3, 128, 9, 9, 40, 3, 2, 1),      # stride 2, odd extents
    (2, 256, 7, 7, 64, 1, 1, 0),      # 1x1
    (2, 3, 20, 20, 16, 7, 2, 3),      # stem-like: 3 input channels
])
def test_graph_runs_unchanged_on_gpu_device(driver, case):
    msg = ctypes.create_string_buffer(512)
    rc = driver.tsplug_selftest(*case, 7, msg, 512)
    text = msg.value.decode(errors="replace")
    assert rc == 0, text
    assert "graph mismatches=0" in text
    assert "fused operator runs=2" in text      # the compiled gpu program runs conv + bias + relu as one operator
    assert "quantize folded=1" in text          # ... and quantizes the fp32 input itself, straight into its staged layout
