"""CPU tests of the C-ABI library: it loads, exports every declared symbol, and reports argument
errors synchronously without touching a GPU."""
import ctypes
import os
import re

import pytest

from ditto_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(ditto_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared()
    assert declared >= set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_version_and_strerror():
    lib = _lib.load()
    assert lib.ditto_b200_version() >= 100
    assert lib.ditto_b200_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert lib.ditto_b200_strerror(code) not in (b"ok", b"unknown error")
    assert lib.ditto_b200_strerror(-99) == b"unknown error"


def test_argument_errors_are_synchronous():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 255) & ~255  # 256-byte aligned dummy pointer, never dereferenced by these calls
    call = lib.ditto_b200_bmm_softmax_bmm
    assert call(None, p, p, p, 1, 128, 64, 64, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert call(p, p, p, p, 0, 128, 64, 64, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert call(p + 2, p, p, p, 1, 128, 64, 64, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert call(p, p, p, p, 1, 120, 64, 64, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_INVALID_ARG  # M % 16
    assert call(p, p, p, p, 1, 128, 64, 64, 128, 0, 1, -1.0, 0, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert call(p, p, p, p, 1, 128, 64, 64, 128, 7, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_UNSUPPORTED  # dtype
    assert call(p, p, p, p, 1, 128, 144, 144, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_UNSUPPORTED  # d > 128
    assert call(p, p, p, p, 1, 128, 144, 64, 128, 0, 1, 1.0, 0, None, 0, None, None) == _lib.ERR_UNSUPPORTED  # N > 128
    mlp = lib.ditto_b200_gemm_relu_gemm
    assert mlp(None, p, p, p, 1, 128, 64, 64, 128, 1, 0, 1, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert mlp(p, p, p, p, 1, 128, 64, 64, 128, 1, 0, 5, None, 0, None, None) == _lib.ERR_INVALID_ARG
    st = lib.ditto_b200_selftest_umma
    assert st(p, p, None, 128, 64, 0, 0, 0, None, None) == _lib.ERR_INVALID_ARG
    assert st(p, p, p, 100, 64, 0, 0, 0, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.ditto_b200_workspace_bytes(0, 12, 512, 64, 64, 512, 0) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("DITTO_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(ImportError):
        _lib.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from ditto_b200 import ops
    q = torch.zeros(1, 128, 64, dtype=torch.float16)
    with pytest.raises(TypeError):
        ops.bmm_softmax_bmm(q, q, q)
    with pytest.raises(TypeError):
        ops.gemm_relu_gemm(q, q, q)
