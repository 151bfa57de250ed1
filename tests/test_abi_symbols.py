"""The C-ABI library loads without a GPU and exports every symbol include/ztq.h declares."""
import ctypes
import os
import re

from ztensor_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(?:cudaError_t|int|size_t)\s+(\w+)\s*\(", text))
    return names


def test_library_loads_and_exports_every_declared_symbol():
    handle = _lib.lib()
    decl = declared_symbols()
    assert {"gemm_q4_f32", "gemm_q8_f32", "ternary_gemv_f32", "ztq_gemv_w4g"} <= decl
    for name in decl:
        assert isinstance(getattr(handle, name), ctypes._CFuncPtr), name
    assert decl == set(_lib.SIGNATURES), decl ^ set(_lib.SIGNATURES)
    assert handle.ztq_abi_version() >= 1


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libztq_sm100a.so")
    try:
        _lib.lib()
    except _lib.KernelLibraryMissing as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("expected KernelLibraryMissing")


def test_host_library_binds_nccl_at_run_time():
    """libztq_host.so loads libnccl.so.2 with dlopen (internal/nccl/nccl_purego.go's scheme) and makes a unique id;
    communicators need GPUs and are covered by the tensor-parallel GPU test."""
    from ztensor_b200 import nccl
    if nccl.find_libnccl() is None and not nccl.available():
        import pytest
        pytest.skip("no libnccl on this machine")
    uid = nccl.get_unique_id()
    assert len(uid) == nccl.UNIQUE_ID_BYTES and any(uid)
    assert nccl.get_unique_id() != uid
    assert "invalid usage" in nccl.error_string(5)
    import pytest
    with pytest.raises(nccl.NcclError, match="expected 128 bytes, got 3"):
        nccl.Comm(b"123", 2, 0)
