"""tsb_quantize_f32_i8_static: the quantize entry point for callers that may not allocate device memory.

Collected last on purpose: if it fails under ``pytest -x`` every other test has already run.
The new entry point keeps its device-side scale table in storage that is part of the library image, so it has
to agree bit for bit with tsb_quantize_f32_i8 (which takes a stream-ordered temporary for long scale lists),
and a second call has to see its own scales, not what the first call left in the shared table.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, x, scales):
    from tennis_b200 import _lib, ops
    arr = _lib.float_array(scales)
    y_old = torch.zeros(x.shape, dtype=torch.int8, device="cuda")
    y_new = torch.zeros(x.shape, dtype=torch.int8, device="cuda")
    _lib.check(lib.tsb_quantize_f32_i8(ops._ptr(x), ops._ptr(y_old), x.numel(), arr, len(scales), ops._stream_ptr()))
    _lib.check(lib.tsb_quantize_f32_i8_static(ops._ptr(x), ops._ptr(y_new), x.numel(), arr, len(scales), ops._stream_ptr()))
    torch.cuda.synchronize()
    return y_old, y_new


def test_static_table_quantize_matches_allocating_quantize_twice_in_a_row():
    from tennis_b200 import _lib
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(123)
    # first call: 200 scales (beyond the 64 that fit in kernel arguments), ragged last group, exact .5 ties
    x1 = torch.randn((200, 37), device="cuda", generator=g) * 40
    x1.view(-1)[::97] = 2.5
    x1.view(-1)[5::101] = -0.5
    s1 = (0.5 + torch.rand(200, generator=torch.Generator().manual_seed(1))).tolist()
    a_old, a_new = _both(lib, x1, s1)
    assert torch.equal(a_old, a_new)
    # second call straight after, other sizes and other scales: the shared table must have been refreshed
    x2 = torch.randn((7, 1003), device="cuda", generator=g) * 90
    s2 = [3.0, 0.25, 1.0, 0.5, 2.0, 0.125, 1.5]
    b_old, b_new = _both(lib, x2, s2)
    assert torch.equal(b_old, b_new)
    assert int(b_new.abs().max()) == 127  # 90 * 3 saturates
    # one scale (half-to-even body, half-away tail) through the table as well
    x3 = torch.tensor([[0.5, 2.5, 126.5, -0.5, -2.5, 1.5, 3.5, -1.5, 0.5, 2.5, 126.5]], device="cuda")
    c_old, c_new = _both(lib, x3, [1.0])
    assert c_new.tolist() == [[0, 2, 126, 0, -2, 2, 4, -2, 1, 3, 127]] and torch.equal(c_old, c_new)
    # the property the entry point exists for: no device memory is obtained by a call.  The allocating variant takes a
    # stream-ordered temporary for 200 scales (the device's free memory drops while the pool holds it); the static
    # variant must leave the free-memory figure of the driver exactly where it was.
    torch.cuda.synchronize()
    y = torch.zeros(x1.shape, dtype=torch.int8, device="cuda")
    arr = _lib.float_array(s1)
    from tennis_b200 import ops
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        _lib.check(lib.tsb_quantize_f32_i8_static(ops._ptr(x1), ops._ptr(y), x1.numel(), arr, len(s1), ops._stream_ptr()))
        assert torch.cuda.mem_get_info()[0] == free_before     # while the work may still be in flight
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(y, a_old)
    # beyond the table: refused, nothing launched, output untouched
    before = lib.tsb_kernel_launch_count()
    y = torch.full((8,), 7, dtype=torch.int8, device="cuda")
    from tennis_b200 import ops
    st = lib.tsb_quantize_f32_i8_static(ops._ptr(x3), ops._ptr(y), 8, _lib.float_array([1.0] * 4097), 4097, ops._stream_ptr())
    assert st == _lib.ERR_UNSUPPORTED and b"4096" in lib.tsb_last_error()
    assert lib.tsb_kernel_launch_count() == before and int(y.sum()) == 56
