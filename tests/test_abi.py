"""The C-ABI library loads without a GPU and exports every symbol that
include/evoattn.h declares; argument validation returns codes."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    src = open(os.path.join(ROOT, "include", "evoattn.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(evo_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported():
    import _evoattn
    names = _declared_symbols()
    assert "evo_fwd" in names and "evo_bwd" in names and len(names) >= 8
    h = C.CDLL(_evoattn.LIB_PATH)
    for n in names:
        assert hasattr(h, n), f"{n} declared in include/evoattn.h but not exported"
    # and the binding covers them all
    assert sorted(_evoattn.SYMBOLS) == names


def test_version_and_strerror():
    import _evoattn
    lib = _evoattn.lib()
    assert lib.evo_version() // 100 == 1
    assert _evoattn.strerror(0) == "ok"
    assert "dimensions" in _evoattn.strerror(-1)
    assert _evoattn.strerror(-12345) == "unknown error"


def test_argument_validation_without_gpu():
    import _evoattn
    lib = _evoattn.lib()
    good = _evoattn.EvoDims(1, 4, 128, 2, 32)
    assert lib.evo_bwd_workspace_bytes(C.byref(good)) > 4 * 4 * 128 * 2 * 32
    for bad in (_evoattn.EvoDims(1, 4, 128, 2, 256), _evoattn.EvoDims(1, 4, 100, 2, 32),
                _evoattn.EvoDims(0, 4, 128, 2, 32), _evoattn.EvoDims(1, 4, 128, 2, 48), _evoattn.EvoDims(1, 4, 128, 2, 8)):
        assert lib.evo_bwd_workspace_bytes(C.byref(bad)) == 0
        rc = lib.evo_fwd(C.byref(bad), 16, 16, 16, 16, 16, 16, None, 16, 0.0, None)
        assert rc == -1
    assert lib.evo_fwd(C.byref(good), None, 16, 16, 16, 16, 16, None, 16, 0.0, None) == -2
    assert lib.evo_fwd(C.byref(good), 8, 16, 16, 16, 16, 16, None, 16, 0.0, None) == -3
    assert lib.evo_fwd(C.byref(good), 16, 16, 16, 16, 16, 16, 8, 16, 0.0, None) == -3    # o_resid misaligned
    assert lib.evo_fwd(None, 16, 16, 16, 16, 16, 16, None, 16, 0.0, None) == -2
    args = [16] * 13
    assert lib.evo_bwd(C.byref(good), *args, 256, 0, 0.0, None) == -4    # workspace too small
    assert lib.evo_selftest_mma(48, 16, 16, 16, 16, 16, 16, 16, None) == -1


def test_missing_library_fails_loudly(monkeypatch):
    import _evoattn
    monkeypatch.setattr(_evoattn, "_lib", None)
    monkeypatch.setattr(_evoattn, "LIB_PATH", "/nonexistent/libevoattn.so")
    with pytest.raises(ImportError):
        _evoattn.lib()
