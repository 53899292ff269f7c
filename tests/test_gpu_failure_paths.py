"""Failure detection and multi-device use of the C ABI, without faulting or hanging a GPU: the kernel's bounded waits
report through a status word, and the host half of that path is exercised by writing the word from the host."""
import ctypes
import threading

import numpy as np
import pytest
import torch

from conftest import same_bits

pytestmark = pytest.mark.gpu


def small_plan(dev, **tune):
    from tennis_b200 import _lib, ops
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.integers(-128, 128, size=(2, 64, 12, 12), dtype=np.int8)).to(dev)
    w = torch.from_numpy(rng.integers(-127, 128, size=(96, 64, 3, 3), dtype=np.int8)).to(dev)
    plan = ops.ConvPlan(x.shape, w.shape, (1, 1, 1, 1), (1, 1), (1, 1), 0.0, _lib.KERNEL_TCGEN05, dev, **tune)
    plan.set_weights(w)
    dq = torch.full((96,), 0.01, device=dev)
    out = torch.zeros(plan.out_shape, dtype=torch.float32, device=dev)
    return plan, x, w, dq, out


def test_a_timed_out_wait_is_reported_once_and_named():
    """No kernel is made to time out: the test writes the code a timed-out wait would leave into the status word and
    checks what the host side makes of it (status -4, the wait's name, cleared after the report)."""
    from tennis_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    plan, x, w, dq, out = small_plan(dev)
    plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
    plan.status()                                           # a healthy run: ok
    good = out.clone()
    for code, name in ((3, "tile loaded"), (5, "weight tile free"), (6, "weight tile loaded")):
        plan.workspace[:4].copy_(torch.tensor([code, 0, 0, 0], dtype=torch.uint8))
        torch.cuda.synchronize()
        with pytest.raises(_lib.TsbError) as err:
            plan.status()
        assert err.value.status == _lib.ERR_DEVICE_TIMEOUT and name in err.value.message and "wait %d" % code in err.value.message
        plan.status()                                       # reported once, then cleared
    # the non-waiting read: a 4-byte copy into pinned memory, decoded by the caller after its own synchronisation
    word = torch.zeros(1, dtype=torch.int32).pin_memory()
    plan.workspace[:4].copy_(torch.tensor([2, 0, 0, 0], dtype=torch.uint8))
    stream = torch.cuda.current_stream()
    _lib.check(lib.tsb_conv2d_i8_status_async(plan.handle, ctypes.c_void_p(plan.workspace.data_ptr()), ctypes.c_void_p(word.data_ptr()),
                                              ctypes.c_void_p(stream.cuda_stream)))
    stream.synchronize()
    assert int(word[0]) == 2 and lib.tsb_conv2d_i8_status_decode(int(word[0])) == _lib.ERR_DEVICE_TIMEOUT
    plan.workspace[:4].zero_()
    # the context is as usable as before
    out.zero_()
    plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
    plan.status()
    assert torch.equal(out, good)


def test_status_word_can_live_in_mapped_host_memory():
    """tsb_conv2d_i8_set_status_word: the plan's kernels report into a word the caller names.  With mapped pinned host
    memory (what the TenniS operator uses) a healthy run leaves the word alone, and the host reads it as plain memory."""
    from tennis_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    plan, x, w, dq, out = small_plan(dev)
    plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
    plan.status()
    good = out.clone()
    cudart = ctypes.CDLL("libcudart.so")
    host = ctypes.c_void_p()
    assert cudart.cudaHostAlloc(ctypes.byref(host), 4, 2) == 0              # 2 = cudaHostAllocMapped
    try:
        word = ctypes.cast(host, ctypes.POINTER(ctypes.c_int))
        word[0] = 0
        devptr = ctypes.c_void_p()
        assert cudart.cudaHostGetDevicePointer(ctypes.byref(devptr), host, 0) == 0
        _lib.check(lib.tsb_conv2d_i8_set_status_word(plan.handle, devptr))
        plan.workspace[:4].copy_(torch.tensor([9, 0, 0, 0], dtype=torch.uint8))     # the workspace word is out of the loop now
        out.zero_()
        plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
        torch.cuda.synchronize()
        assert word[0] == 0 and torch.equal(out, good)
        assert int(plan.workspace[0]) == 9                                        # ... and untouched by the run
        # what the host makes of a code found there
        assert lib.tsb_conv2d_i8_status_decode(4) == _lib.ERR_DEVICE_TIMEOUT
        _lib.check(lib.tsb_conv2d_i8_set_status_word(plan.handle, None))          # back to the workspace word
        plan.workspace[:4].zero_()
        plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
        plan.status()
    finally:
        torch.cuda.synchronize()
        cudart.cudaFreeHost(host)


def test_waiting_host_call_reports_the_status_word(checker):
    from tennis_b200 import _lib, workloads
    lib = _lib.load()
    dev = torch.device("cuda")
    layer = workloads.conv_layer("t", 2, 64, 10, 10, 48, 3, 1, 1)
    d = workloads.make_layer_data(layer, seed=1)
    from tennis_b200 import ops
    plan = ops.ConvPlan(d["x"].shape, d["w"].shape, (1, 1, 1, 1), (1, 1), (1, 1), 0.0, _lib.KERNEL_TCGEN05, dev)
    nbytes = lib.tsb_conv2d_host_scratch_bytes(plan.handle)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = np.zeros(plan.out_shape, np.float32)
    scales = _lib.float_array([float(d["qscale"])] * 2)

    def call(resident):
        return lib.tsb_conv2d_quantized_host(plan.handle, d["x"].ctypes.data, scales, 2, d["w"].ctypes.data, d["dq"].ctypes.data,
                                             d["bias"].ctypes.data, _lib.ACT_RELU, 0.0, out.ctypes.data, scratch.data_ptr(), nbytes,
                                             resident, None)
    assert call(0) == 0
    xq = checker.quantize(d["x"], [float(d["qscale"])] * 2)
    want = checker.conv_block(xq, d["w"], (1, 1, 1, 1), (1, 1), (1, 1), d["dq"], d["bias"], act="relu")
    assert same_bits(out, want)
    # plant a time-out code in the workspace's status word (the workspace sits at the end of the scratch block)
    ws_off = nbytes - ((plan.ws_bytes + 255) // 256) * 256
    scratch[ws_off:ws_off + 4].copy_(torch.tensor([4, 0, 0, 0], dtype=torch.uint8))
    torch.cuda.synchronize()
    assert call(1) == _lib.ERR_DEVICE_TIMEOUT and b"accumulator ready" in lib.tsb_last_error()
    assert call(1) == 0                                     # cleared with the report


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_from_two_threads_of_one_process():
    """The reference drives several GPUs as N threads x one Workbench per device in ONE process.  Plans are created
    and a kernel variant with more than 48 KB of dynamic shared memory is launched on cuda:1 first, then on cuda:0."""
    from tennis_b200 import _lib
    results, errors = {}, []

    def work(index):
        try:
            torch.cuda.set_device(index)
            dev = torch.device("cuda", index)
            with torch.cuda.device(index):
                plan, x, w, dq, out = small_plan(dev)
                assert "smem=" in plan.describe() and int(plan.describe().split("smem=")[1].split()[0]) > 48 * 1024
                plan.run(x, _lib.LAYOUT_NCHW, dq, out_f32=out)
                plan.status()
                # exact integer convolution in fp64, then the one fp32 multiply of the dequantize step
                ref = torch.nn.functional.conv2d(x.double(), w.double(), padding=1).float() * dq.view(1, -1, 1, 1)
                results[index] = bool(torch.equal(out, ref))
        except Exception as e:   # noqa: BLE001 - reported by the main thread
            errors.append((index, repr(e)))

    for order in ((1, 0),):
        for index in order:
            t = threading.Thread(target=work, args=(index,))
            t.start()
            t.join()
    threads = [threading.Thread(target=work, args=(i,)) for i in (1, 0)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert results == {0: True, 1: True}
