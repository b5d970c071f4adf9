"""The shared library loads without a GPU and exports every symbol the public
header declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(sparse_b200_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from sparse_attention_b200_b200 import build, _lib
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 4
    for name in names:
        assert hasattr(lib, name), name


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from sparse_attention_b200_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    import pytest
    with pytest.raises(_lib.SparseB200Error):
        _lib.lib()


def test_invalid_arguments_return_error_codes_without_a_gpu():
    from sparse_attention_b200_b200 import _lib
    lib = _lib.lib()
    rc = lib.sparse_b200_q_centric(None, None, None, None, None, None, None, 1, 8, 8, 256, 256, 1, None)
    assert rc == _lib.ERR_INVALID and b"non-null" in lib.sparse_b200_last_error()
    one = ctypes.c_void_p(4096)
    rc = lib.sparse_b200_q_centric(one, one, one, one, None, ctypes.c_void_p(8192), None, 1, 8, 3, 256, 256, 1, None)
    assert rc == _lib.ERR_INVALID and b"multiple" in lib.sparse_b200_last_error()
    rc = lib.sparse_b200_q_centric(one, one, one, one, None, ctypes.c_void_p(8192), None, 1, 8, 8, 200, 256, 1, None)
    assert rc == _lib.ERR_INVALID
    rc = lib.sparse_b200_q_centric(one, one, one, one, None, ctypes.c_void_p(8192), None, 1, 8, 8, 256, 256, 3, None)
    assert rc == _lib.ERR_INVALID and b"exceed" in lib.sparse_b200_last_error()
