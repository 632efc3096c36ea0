"""The C-ABI library loads and exports exactly what include/cdssm_b200.h declares.
No kernel is launched here (these run without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "cdssm_b200.h")).read()
    return sorted(set(re.findall(r"CDSSM_API\s+\w+\s+(cdssm_b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import cdssm_b200
    from cdssm_b200 import build
    build.build()                      # nvcc cross-compiles without a GPU
    return cdssm_b200._lib


def test_header_and_binding_agree(lib):
    names = _declared()
    assert len(names) >= 11
    assert sorted(lib.SIGNATURES) == names


def test_every_declared_symbol_is_exported(lib):
    handle = lib.lib()
    for name in _declared():
        assert hasattr(handle, name), name
    assert handle.cdssm_b200_version() >= 100


def test_no_torch_types_in_abi():
    text = open(os.path.join(ROOT, "include", "cdssm_b200.h")).read()
    assert "torch" not in text.lower().replace("pytorch", "") and "at::" not in text


def test_argument_validation_needs_no_gpu(lib):
    h = lib.lib()
    # workspace size is pure host arithmetic
    n = h.cdssm_b200_scan_fused_workspace_bytes(2, 512, 4, 64, 2, 64)
    assert n >= 2 * 8 * 4 * (2 + 128) * 4
    assert h.cdssm_b200_scan_fused_workspace_bytes(2, 512, 4, 64, 3, 64) == 0      # odd state_dim
    # null pointers and bad sizes are refused before anything touches CUDA
    null = ctypes.c_void_p(0)
    assert h.cdssm_b200_normalize_kq_fwd(null, null, null, null, 4, 64, 0, null) == -1
    one = ctypes.c_void_p(256)
    assert h.cdssm_b200_intra_chunk_scan_fwd(one, one, one, one, one, one, 1, 64, 1, 64, 3, 0, null) == -1
    assert h.cdssm_b200_intra_chunk_scan_fwd(one, one, one, one, one, one, 1, 64, 1, 256, 2, 0, null) == -2
    assert h.cdssm_b200_intra_chunk_scan_fwd(one, one, one, one, one, one, 1, 64, 1, 64, 34, 0, null) == -2


def test_missing_library_fails_loudly(monkeypatch, lib):
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", "/nonexistent/libcdssm_b200.so")
    with pytest.raises(lib.CdssmError):
        lib.lib()


def test_cpu_tensors_are_refused():
    import torch
    import cdssm_b200
    x = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(cdssm_b200.CdssmError):
        cdssm_b200.NormalizeKQFn.apply(x, x)
