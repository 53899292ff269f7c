"""The shared library loads without a GPU and exports every entry point include/tennis_b200.h declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tennis_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#ifdef TSB_ENABLE_TRACE.*?#endif", "", text, flags=re.S)   # profiling builds only
    return sorted(set(re.findall(r"\b(tsb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "tsb_quantize_f32_i8" in names and "tsb_conv2d_i8_run" in names and len(names) >= 20


def test_library_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    from tennis_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), "libtennis_b200.so does not export " + name
    # the Python binding covers the same set
    assert sorted(_lib.SYMBOLS) == declared_symbols()


def test_simple_host_calls_work_without_gpu():
    from tennis_b200 import _lib
    lib = _lib.load()
    assert lib.tsb_version() >= 100
    assert [lib.tsb_padded_channels(c) for c in (1, 3, 16, 17, 32, 33, 64, 65, 2048)] == [16, 16, 16, 64, 64, 64, 64, 128, 2048]
    assert lib.tsb_status_string(0) == b"ok"
    assert lib.tsb_status_string(_lib.ERR_DEVICE_TIMEOUT).startswith(b"a device-side wait")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tennis_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
