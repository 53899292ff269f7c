"""Host-side behaviour that needs no GPU: attribute parsing and checks of the operator mirrors, argument
validation of the C ABI (a rejected call launches nothing), kernel selection and the workload arithmetic."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tennis_b200 import _lib, ops, workloads


def make_conv(**over):
    op = ops.Conv2DQuantized()
    params = dict(format="NCHW", padding=np.array([[0, 0], [0, 0], [1, 1], [1, 1]]), stride=np.array([1, 1, 1, 1]),
                  dilation=np.array([1, 1, 1, 1]), dequantize_scales=np.ones(4, np.float32))
    params.update(over)
    for k, v in params.items():
        if v is not None:
            op.set(k, v)
    return op


def test_quantize_fields_and_infer():
    q = ops.Quantize()
    with pytest.raises(ops.EjectionException, match="quantize_scale"):
        q.init()
    with pytest.raises(ops.EjectionException, match="Unidentified param"):
        q.set("quantize_scales", [1.0])
    q.set("quantize_scale", np.array([1.0, 2.0], np.float32))
    q.init()
    assert q.infer([torch.zeros(2, 3, 4, 4)]) == [("int8", (2, 3, 4, 4))]
    with pytest.raises(ops.EjectionException, match=r"m_quantize_scales.size\(\) == x_tensor.sizes\(\)\[0\]"):
        q.infer([torch.zeros(3, 3, 4, 4)])


def test_conv_init_checks_follow_the_reference():
    make_conv().init()
    make_conv(dilation=None, dialations=np.array([1, 1, 2, 2])).init()  # the historical misspelling is accepted
    with pytest.raises(ops.EjectionException, match="must set dilation or dialations"):
        make_conv(dilation=None).init()
    with pytest.raises(ops.EjectionException, match="do not support format: NCWH"):
        make_conv(format="NCWH").init()
    with pytest.raises(ops.EjectionException, match=r"do not support padding: \[1, 0, 0, 0, 1, 1, 1, 1\]"):
        make_conv(padding=np.array([[1, 0], [0, 0], [1, 1], [1, 1]])).init()
    with pytest.raises(ops.EjectionException, match=r"do not support stride: \[2, 1, 1, 1\]"):
        make_conv(stride=np.array([2, 1, 1, 1])).init()
    with pytest.raises(ops.EjectionException, match="do not support dialations"):
        make_conv(dilation=np.array([1, 2, 1, 1])).init()
    with pytest.raises(ops.EjectionException, match=r"padding_tensor.has_shape"):
        make_conv(padding=np.zeros((4,), np.int32)).init()
    with pytest.raises(ops.EjectionException, match="unsatisfied fields"):
        make_conv(dequantize_scales=None).init()


def test_conv_infer_shapes_and_checks():
    op = make_conv(padding=np.array([[0, 0], [0, 0], [3, 3], [3, 3]]), stride=np.array([1, 1, 2, 2]))
    op.init()
    x = torch.zeros(2, 3, 224, 224, dtype=torch.int8)
    w = torch.zeros(4, 3, 7, 7, dtype=torch.int8)
    assert op.infer([x, w]) == [("float32", (2, 4, 112, 112))]
    with pytest.raises(ops.EjectionException, match=r"w_tensor.size\(1\) == x_tensor.size\(1\)"):
        op.infer([x, torch.zeros(4, 5, 7, 7, dtype=torch.int8)])
    with pytest.raises(ops.EjectionException, match=r"x_tensor.dtype\(\) == INT8"):
        op.infer([x.float(), w.float()])
    with pytest.raises(ops.EjectionException, match=r"m_dequantize_scales.size\(\) == w_tensor.size\(0\)"):
        op.infer([x, torch.zeros(5, 3, 7, 7, dtype=torch.int8)])


def desc(**over):
    d = _lib.ConvDesc()
    base = dict(n=1, c=64, h=8, w=8, o=64, kh=3, kw=3, pad_top=1, pad_bottom=1, pad_left=1, pad_right=1, stride_h=1,
                stride_w=1, dilation_h=1, dilation_w=1, padding_value=0.0, kernel=_lib.KERNEL_AUTO)
    base.update(over)
    for k, v in base.items():
        setattr(d, k, v)
    return d


def create(d):
    lib = _lib.load()
    h = ctypes.c_void_p()
    st = lib.tsb_conv2d_i8_plan_create(ctypes.byref(d), ctypes.byref(h))
    return st, h


def test_plan_create_validates_and_selects_kernel():
    lib = _lib.load()
    st, h = create(desc())
    assert st == 0 and lib.tsb_conv2d_i8_kernel(h) == _lib.KERNEL_TCGEN05
    shape = (ctypes.c_int * 4)()
    lib.tsb_conv2d_i8_output_shape(h, shape)
    assert list(shape) == [1, 64, 8, 8]
    assert lib.tsb_conv2d_i8_workspace_bytes(h) >= 256 + 64 * 9 * 64 + 64 * 64
    lib.tsb_conv2d_i8_plan_destroy(h)
    # small channel counts run on the tensor cores too (folded filter rows / channel padding)
    for over in (dict(c=3), dict(c=24), dict(c=3, kh=7, kw=7, pad_top=3, pad_bottom=3, pad_left=3, pad_right=3, stride_h=2, stride_w=2, h=32, w=32)):
        st, h = create(desc(**over))
        assert st == 0 and lib.tsb_conv2d_i8_kernel(h) == _lib.KERNEL_TCGEN05
        lib.tsb_conv2d_i8_plan_destroy(h)
    # geometries the tensor-core kernel does not take resolve to the direct kernel
    for over in (dict(padding_value=3.0), dict(c=3, kw=11, w=16, pad_left=5, pad_right=5)):
        st, h = create(desc(**over))
        assert st == 0 and lib.tsb_conv2d_i8_kernel(h) == _lib.KERNEL_DIRECT
        lib.tsb_conv2d_i8_plan_destroy(h)
    st, _ = create(desc(padding_value=3.0, kernel=_lib.KERNEL_TCGEN05))
    assert st == _lib.ERR_UNSUPPORTED and b"tcgen05 kernel not available" in lib.tsb_last_error()
    for over in (dict(n=0), dict(stride_h=0), dict(pad_left=-1), dict(kh=11, h=4, pad_top=0, pad_bottom=0), dict(kernel=9)):
        st, _ = create(desc(**over))
        assert st == _lib.ERR_INVALID_ARGUMENT, over


def describe(**over):
    lib = _lib.load()
    st, h = create(desc(**over))
    assert st == 0
    buf = ctypes.create_string_buffer(512)
    n = lib.tsb_conv2d_i8_plan_describe(h, buf, 512)
    assert n > 0
    lib.tsb_conv2d_i8_plan_destroy(h)
    return buf.value.decode()


def test_load_mode_and_orientation_of_the_benchmark_layers():
    """Which variant of the tensor-core kernel the plan picks, layer by layer (no device needed)."""
    same = dict(pad_top=1, pad_bottom=1, pad_left=1, pad_right=1)
    none = dict(pad_top=0, pad_bottom=0, pad_left=0, pad_right=0)
    stem = describe(n=32, c=3, h=224, w=224, o=64, kh=7, kw=7, stride_h=2, stride_w=2, pad_top=3, pad_bottom=3, pad_left=3, pad_right=3)
    assert "mode=rows swap=0 bn=64 bk=64" in stem and "resident=1" in stem and "alt:" not in stem
    c56 = describe(n=64, c=64, h=56, w=56, o=64, kh=3, kw=3, **same)
    assert c56.startswith("kernel=tcgen05 mode=patch swap=0 bn=64 bk=64 pix=128 tiles=1792x1")
    c28 = describe(n=64, c=128, h=28, w=28, o=128, kh=3, kw=3, **same)
    assert "mode=patch swap=0 bn=128 bk=128" in c28.split(" | ")[0]
    c14 = describe(n=64, c=256, h=14, w=14, o=256, kh=3, kw=3, **same)     # 590 KB of weights: no patch mode
    assert "mode=im2col swap=0 bn=256 bk=128" in c14.split(" | ")[0]
    s2 = describe(n=32, c=256, h=28, w=28, o=512, kh=3, kw=3, stride_h=2, stride_w=2, **same)
    assert "mode=im2col" in s2.split(" | ")[0]
    p1 = describe(n=32, c=256, h=14, w=14, o=1024, kh=1, kw=1, **none)
    assert "mode=tiled swap=0 bn=128" in p1.split(" | ")[0] and "alt: mode=tiled swap=1" in p1   # 49 pixel tiles: narrower N
    csp_stem = describe(n=16, c=3, h=608, w=608, o=32, kh=3, kw=3, **same)
    assert "mode=rows" in csp_stem and "tiles=48640x1" in csp_stem
    assert describe(padding_value=3.0).startswith("kernel=direct (non-zero padding_value)")


def test_raw_row_plans_keep_their_weights_resident():
    """A wide few-channel layer with more than 128 output channels: raw-row mode is admitted where two row stages fit
    beside the weight tile, and the plan must then keep the weights resident (the mode cannot stream them)."""
    text = describe(n=1, c=3, h=64, w=700, o=192, kh=7, kw=7, stride_h=2, stride_w=2, pad_top=3, pad_bottom=3, pad_left=3, pad_right=3)
    assert "mode=rows" in text and "resident=1" in text, text
    stages = int(text.split("stages=")[1].split()[0])
    assert 2 <= stages < 4, text
    # forced off, the same layer takes the folded im2col loads
    text = describe(n=1, c=3, h=64, w=700, o=192, kh=7, kw=7, stride_h=2, stride_w=2, pad_top=3, pad_bottom=3, pad_left=3, pad_right=3,
                    raw_row_mode=_lib.TUNE_OFF)
    assert "mode=fold" in text, text


def test_heuristic_overrides_travel_in_the_descriptor():
    same = dict(pad_top=1, pad_bottom=1, pad_left=1, pad_right=1)
    auto = describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, **same)
    normal = describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, mma_orientation=_lib.TUNE_OFF, **same)
    swapped = describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, mma_orientation=_lib.TUNE_ON, **same)
    assert "swap=0" in normal and "swap=1" in swapped and "alt:" not in normal and "alt:" not in swapped
    assert "mode=patch" in describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, patch_mode=_lib.TUNE_ON, **same)
    assert "mode=patch" not in describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, patch_mode=_lib.TUNE_OFF, **same)
    assert auto.startswith("kernel=tcgen05")
    st, _ = create(desc(mma_orientation=3))
    assert st == _lib.ERR_INVALID_ARGUMENT and b"TSB_TUNE" in _lib.load().tsb_last_error()
    # the environment no longer changes plans or layouts
    import os
    os.environ["TSB_SWAP"], os.environ["TSB_PAD128"] = "1", "1"
    try:
        assert describe(n=2, c=64, h=20, w=20, o=64, kh=3, kw=3, **same) == auto
        assert _lib.load().tsb_padded_channels(65) == 128 and _lib.load().tsb_padded_channels(129) == 192
    finally:
        del os.environ["TSB_SWAP"], os.environ["TSB_PAD128"]


def test_status_word_decoding_names_every_wait():
    lib = _lib.load()
    assert lib.tsb_conv2d_i8_status_decode(0) == 0
    for code, word in ((1, b"stage free"), (2, b"accumulator buffer free"), (3, b"tile loaded"), (4, b"accumulator ready"),
                       (5, b"weight tile free"), (6, b"weight tile loaded")):
        assert lib.tsb_conv2d_i8_status_decode(code) == _lib.ERR_DEVICE_TIMEOUT
        assert word in lib.tsb_last_error() and (b"wait %d" % code) in lib.tsb_last_error()


def test_pool_extent_follows_the_reference():
    lib = _lib.load()
    assert lib.tsb_pool_out_dim(112, 1, 1, 3, 2) == 57 and lib.tsb_pool_out_dim(112, 1, 0, 3, 2) == 56
    assert lib.tsb_pool_out_dim(9, 0, 0, 2, 2) == 5 and lib.tsb_pool_out_dim(6, 1, 1, 3, 1) == 6
    assert lib.tsb_pool_out_dim(0, 0, 0, 2, 2) == _lib.ERR_INVALID_ARGUMENT
    before = lib.tsb_kernel_launch_count()
    # a window wholly inside the padding is refused before any launch
    assert lib.tsb_maxpool_i8_nhwc(ctypes.c_void_p(256), ctypes.c_void_p(512), 1, 4, 4, 16, 2, 2, 0, 2, 0, 2, None) == _lib.ERR_UNSUPPORTED
    assert lib.tsb_kernel_launch_count() == before


def test_quantize_mirror_takes_fp32_and_fp64_only():
    q = ops.Quantize()
    q.set("quantize_scale", np.array([1.0], np.float32))
    q.init()
    with pytest.raises(ops.EjectionException, match="quantize not support this data type: float16"):
        q.run([torch.zeros(1, 4, dtype=torch.float16)])
    with pytest.raises(ops.EjectionException, match="not support this data type: int32"):
        q.run([torch.zeros(1, 4, dtype=torch.int32)])


def test_requantize_scale_limit_is_stated():
    assert _lib.MAX_REQUANT_SCALES == 128
    text = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "tennis_b200.h")).read()
    assert "#define TSB_MAX_REQUANT_SCALES 128" in text


def test_run_rejects_bad_arguments_before_any_launch():
    lib = _lib.load()
    before = lib.tsb_kernel_launch_count()
    st, h = create(desc())
    e = _lib.ConvEpilogue()
    assert lib.tsb_conv2d_i8_run(h, None, 0, ctypes.byref(e), None, 0, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.tsb_conv2d_i8_set_weights(h, ctypes.c_void_p(256), ctypes.c_void_p(256), 16, None) == _lib.ERR_WORKSPACE_TOO_SMALL
    assert lib.tsb_quantize_f32_i8(None, None, 4, _lib.float_array([1.0]), 1, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.tsb_quantize_f32_i8(ctypes.c_void_p(256), ctypes.c_void_p(512), 4, _lib.float_array([1.0]), 0, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.tsb_quantize_f32_i8(ctypes.c_void_p(256), ctypes.c_void_p(512), 2**31, _lib.float_array([1.0]), 1, None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.tsb_kernel_launch_count() == before
    lib.tsb_conv2d_i8_plan_destroy(h)


def test_workload_arithmetic():
    l = workloads.CONFIG0[0]
    assert workloads.out_hw(l) == (56, 56)
    assert workloads.layer_ops(l) == 2 * 64 * 56 * 56 * 64 * 9
    assert [workloads.out_hw(x) for x in workloads.CONFIG1] == [(14, 14), (28, 28), (14, 14), (7, 7), (112, 112)]
    d = workloads.make_layer_data(workloads.conv_layer("t", 2, 3, 5, 5, 4, 3, 1, 1), seed=0)
    d2 = workloads.make_layer_data(workloads.conv_layer("t", 2, 3, 5, 5, 4, 3, 1, 1), seed=0)
    assert all(np.array_equal(d[k], d2[k]) for k in d)
    assert abs(float(np.abs(d["x"]).max() * d["qscale"]) - 127.0) < 1e-3
    assert d["w"].min() >= -127 and d["dq"].shape == (4,)


def test_gpu_locality_and_binding_from_a_fake_sysfs(tmp_path):
    """The NUMA binding of a rank reads sysfs and changes only the process's own affinity mask."""
    from tennis_b200 import sharding
    assert sharding.parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert sharding.parse_cpu_list("") == []
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "numa_node").write_text("1\n")
    (dev / "local_cpulist").write_text("4-7\n")
    assert sharding.gpu_locality("0000:1B:00.0", str(tmp_path)) == (1, [4, 5, 6, 7])
    calls = []
    rec = sharding.bind_to_gpu("0000:1B:00.0", str(tmp_path), setaffinity=lambda pid, cpus: calls.append((pid, list(cpus))),
                               getaffinity=lambda pid: set(range(8)))
    assert calls == [(0, [4, 5, 6, 7])] and rec["numa_node"] == 1 and rec["bound_cpus"] == 4
    # none of the local CPUs is in the process's mask (a container's cpuset): nothing is bound
    calls.clear()
    rec = sharding.bind_to_gpu("0000:1B:00.0", str(tmp_path), setaffinity=lambda pid, cpus: calls.append(1),
                               getaffinity=lambda pid: {0, 1})
    assert calls == [] and rec["bound_cpus"] == 0
    # a platform that says nothing (no such device directory)
    rec = sharding.bind_to_gpu("0000:ff:00.0", str(tmp_path), setaffinity=lambda pid, cpus: calls.append(1),
                               getaffinity=lambda pid: {0, 1})
    assert calls == [] and rec["numa_node"] == -1


def test_gather_values_single_process():
    from tennis_b200 import sharding
    assert sharding.gather_values([1, 2.5]) == [[1.0, 2.5]]
