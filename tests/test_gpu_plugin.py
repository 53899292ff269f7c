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
    lib.tsplug_block.argtypes = [ctypes.c_int] * 6 + [ctypes.c_uint, ctypes.c_char_p, ctypes.c_int]
    lib.tsplug_const_weights.argtypes = [ctypes.c_int] * 8 + [ctypes.c_uint, ctypes.c_char_p, ctypes.c_int]
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


@pytest.mark.parametrize("variant", [0, 1, 4, 5])
@pytest.mark.parametrize("case", [
    (2, 256, 64, 14, 14),     # a ResNet-50 bottleneck at 14 x 14: 1x1 256->64, 3x3 64->64, 1x1 64->256 + identity shortcut
    (3, 128, 32, 9, 11),      # odd extents, 32 channels in the middle
])
def test_bottleneck_block_passes_int8_between_fused_nodes(driver, case, variant):
    """A three-convolution block with a shortcut, loaded from ONE graph: on the gpu device the rewrite must leave three
    fused nodes that hand int8 to one another (no quantize or layout kernel between the layers) and fold the shortcut into
    the last one; the result must equal the cpu device's bit for bit.  variant bit 0: the shortcut is added after a
    leaky_relu (Darknet) instead of before a relu (ResNet); bit 2: a fourth layer reads the block's result, so the node
    with the shortcut hands int8 on too."""
    msg = ctypes.create_string_buffer(512)
    rc = driver.tsplug_block(*case, variant, 11, msg, 512)
    text = msg.value.decode(errors="replace")
    assert rc == 0, text
    hand = 6 if variant & 4 else 4
    assert "block mismatches=0" in text and f"int8 hand-overs={hand}" in text and "shortcuts folded=2" in text


@pytest.mark.parametrize("variant", [2, 3, 6, 7])
def test_broadcast_shortcut_is_left_to_the_add_operator(driver, variant):
    """Operator "add" broadcasts; no shape is known when the graph is rewritten.  A shortcut of shape [1, C, 1, 1] must
    therefore still give the cpu device's result: the fused node runs convolution and bias (and the activation, Darknet
    style) itself and finishes with the gpu device's own add -- and still hands int8 to a layer behind it."""
    msg = ctypes.create_string_buffer(512)
    rc = driver.tsplug_block(2, 128, 32, 10, 12, variant, 5, msg, 512)
    text = msg.value.decode(errors="replace")
    assert rc == 0, text
    assert "block mismatches=0" in text and "shortcuts folded=0" in text and "shortcuts by the add operator=2" in text


def test_resnet50_graph_on_gpu_device_equals_cpu_device():
    """53 convolutions, 16 shortcuts (4 of them projections), one max pool, as ONE TenniS graph: every quantized layer
    becomes a fused node, the three layers of a block hand int8 to one another, every shortcut goes into an epilogue,
    and the trunk's output equals the cpu device's bit for bit."""
    path = os.path.join(ROOT, "tennis_b200", "libtennis_b200_workbench.so")
    if not os.path.exists(path):
        pytest.skip("tennis_b200/libtennis_b200_workbench.so was not built (needs the reference sources at build time)")
    lib = ctypes.CDLL(path)
    lib.tsb_workbench_resnet50.argtypes = [ctypes.c_int] * 4 + [ctypes.c_uint, ctypes.POINTER(ctypes.c_double), ctypes.c_char_p,
                                           ctypes.c_int]
    out = (ctypes.c_double * 8)()
    msg = ctypes.create_string_buffer(512)
    rc = lib.tsb_workbench_resnet50(2, 64, 1, 17, 3, out, msg, 512)
    text = msg.value.decode(errors="replace")
    assert rc == 0, text
    assert "53 convolutions, trunk mismatches=0" in text
    assert out[2] == 53 and out[3] == 32 and out[4] == 16, text
    # 53 convolutions + the staging quantize of each layer that reads an fp32 tensor (53 - 32 hand-overs)
    assert out[1] == 53 + 21, text


@pytest.mark.parametrize("case", [
    (2, 64, 14, 14, 96, 3, 1, 1),
    (3, 40, 9, 9, 24, 1, 1, 0),       # 24 scales over 24 x 40 weights: groups of 40
])
def test_weights_quantized_at_compile_time_on_gpu(driver, case):
    """A module that carries fp32 weights behind a quantize node (one scale per output channel): Workbench::Load folds
    that node by running it once on the compiling device -- on gpu, through this repo's quantize operator."""
    msg = ctypes.create_string_buffer(512)
    rc = driver.tsplug_const_weights(*case, 9, msg, 512)
    text = msg.value.decode(errors="replace")
    assert rc == 0, text
    assert "mismatches=0" in text and "fused operator runs=1" in text
