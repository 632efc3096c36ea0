"""ctypes binding of libcdssm_b200.so (the C ABI declared in include/cdssm_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libcdssm_b200.so")

OK = 0
ERRORS = {
    -1: "bad argument (null pointer, non-positive size, odd state_dim, misaligned buffer)",
    -2: "unsupported size (state_dim > 32, head_dim > 128, chunk > 256, ...)",
    -3: "workspace missing, misaligned or too small",
    -4: "CUDA runtime error",
    -5: "device-side wait timed out",
}
BF16, F32 = 0, 1

_c_void_p, _c_int, _c_float, _c_size_t, _c_int64 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float,
                                                    ctypes.c_size_t, ctypes.c_int64)
_P, _I, _F = _c_void_p, _c_int, _c_float

# name -> (restype, argtypes); must list every function include/cdssm_b200.h declares
SIGNATURES = {
    "cdssm_b200_version": (_I, []),
    "cdssm_b200_last_cuda_error": (_I, []),
    "cdssm_b200_dynamics_fwd": (_I, [_P] * 7 + [_F] * 5 + [_I] * 6 + [_P]),
    "cdssm_b200_intra_chunk_scan_bwd": (_I, [_P] * 12 + [_I] * 6 + [_P]),
    "cdssm_b200_exact_correction_bwd": (_I, [_P] * 9 + [_I] * 8 + [_P]),
    "cdssm_b200_inter_chunk_scan_bwd": (_I, [_P] * 5 + [_I] * 6 + [_P]),
    "cdssm_b200_conv1d_silu_bwd": (_I, [_P] * 7 + [_I] * 4 + [_P]),
    "cdssm_b200_dynamics_bwd": (_I, [_P] * 9 + [_F] * 5 + [_I] * 6 + [_P]),
    "cdssm_b200_normalize_kq_bwd": (_I, [_P] * 6 + [_c_int64, _I, _I, _P]),
    "cdssm_b200_normalize_kq_fwd": (_I, [_P] * 4 + [_c_int64, _I, _I, _P]),
    "cdssm_b200_intra_chunk_scan_fwd": (_I, [_P] * 6 + [_I] * 6 + [_P]),
    "cdssm_b200_inter_chunk_scan_fwd": (_I, [_P] * 3 + [_I] * 6 + [_P]),
    "cdssm_b200_exact_correction_fwd": (_I, [_P] * 5 + [_I] * 7 + [_P]),
    "cdssm_b200_conv1d_silu_fwd": (_I, [_P] * 4 + [_I] * 4 + [_P]),
    "cdssm_b200_rmsnorm_fwd": (_I, [_P, _P, _P, _c_int64, _I, _F, _I, _P]),
    "cdssm_b200_groupnorm_stats_floats": (_c_size_t, [_I] * 3),
    "cdssm_b200_groupnorm_stats": (_I, [_P, _P, _I, _I, _I, _I, _F, _I, _P]),
    "cdssm_b200_groupnorm_gate_fwd": (_I, [_P] * 5 + [_c_int64] + [_P] * 3 + [_I] * 4 + [_F, _I, _P]),
    "cdssm_b200_conv1d_silu_step": (_I, [_P, _c_int64, _P, _P, _P, _P, _I, _I, _I, _P]),
    "cdssm_b200_scan_fused_workspace_bytes": (_c_size_t, [_I] * 6),
    "cdssm_b200_scan_fused_fwd": (_I, [_P] * 11 + [_c_size_t] + [_F] * 6 + [_I] * 9 + [_P]),
    "cdssm_b200_scan_summary_fwd": (_I, [_P] * 9 + [_c_size_t] + [_F] * 5 + [_I] * 10 + [_P]),
    "cdssm_b200_scan_fused_segmented_fwd": (_I, [_P] * 10 + [_c_size_t] + [_F] * 6 + [_I] * 10 + [_P]),
    "cdssm_b200_compose_carries": (_I, [_P] * 6 + [_I] * 5 + [_c_int64, _c_int64, _P]),
    "cdssm_b200_scan_fused_fwd_noalloc": (_I, [_P] * 10 + [_F] * 6 + [_I] * 9 + [_P]),
    "cdssm_b200_scan_fused_noalloc_max_bytes": (_c_size_t, []),
    "cdssm_b200_scan_fused_status": (_I, [_P, _P, _P]),
    "cdssm_b200_scan_fused_noalloc_status": (_I, [_P, _P]),
    "cdssm_b200_set_wait_limit_ns": (ctypes.c_uint64, [ctypes.c_uint64]),
    "cdssm_b200_selftest_bounded_wait": (_I, [_P, ctypes.c_uint64, _P]),
    "cdssm_b200_decode_step": (_I, [_P] * 8 + [_F] * 6 + [_I] * 6 + [_P]),
    "cdssm_b200_decode_step_strided": (_I, [_P, _P, _c_int64, _P, _c_int64, _P, _c_int64, _P, _P, _P, _c_int64] + [_P] * 3 + [_F] * 6 + [_I] * 5 + [_P, _I, _P]),
    "cdssm_b200_decode_step_reference": (_I, [_P] * 11 + [_F] * 6 + [_I] * 6 + [_P, _I, _P]),
    "cdssm_b200_decode_step_at": (_I, [_P] * 8 + [_F] * 6 + [_I] * 4 + [_P, _I, _P]),
}

_lib = None


class CdssmError(RuntimeError):
    pass


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CdssmError(
                f"{LIB_PATH} not found: build it with `python __graft_entry__.py` "
                "(there is no CPU or PyTorch fallback for this path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc, what):
    if rc != OK:
        msg = ERRORS.get(rc, f"error {rc}")
        if rc == -4:
            msg += f" (cudaError {lib().cdssm_b200_last_cuda_error()})"
        raise CdssmError(f"{what}: {msg}")
