"""ctypes binding of ``libnlfa.so`` (declared in ``include/nlfa.h``).

Nothing here touches torch: plain pointers and sizes go in, status codes come
out.  ``load()`` raises when the library is missing and cannot be built -- there
is no CPU fallback behind this boundary.
"""
from __future__ import annotations

import ctypes
import pathlib

PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = PKG / "libnlfa.so"

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2
PASS_DELTA, PASS_DKV, PASS_DQ, PASS_ALL, PASS_FUSED = 1, 2, 4, 7, 8
OK = 0
ERR_DEVICE_TIMEOUT = 10
ERR_SELFTEST_MISMATCH = 12

_c_void_p, _c_int, _c_float, _c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/nlfa.h declaration by declaration
SIGNATURES = {
    "nlfa_version": (_c_int, []),
    "nlfa_strerror": (ctypes.c_char_p, [_c_int]),
    "nlfa_device_supported": (_c_int, []),
    "nlfa_resolve_path": (_c_int, [_c_int, _c_int, _c_int]),
    "nlfa_fwd": (_c_int, [_c_void_p] * 5 + [_c_int] * 5 + [_c_float] + [_c_int] * 4 + [_c_void_p]),
    "nlfa_fwd_masked": (_c_int, [_c_void_p] * 5 + [_c_int] * 5 + [_c_float] + [_c_int] * 5 + [_c_void_p]),
    "nlfa_bwd_masked": (_c_int, [_c_void_p] * 10 + [_c_size_t] + [_c_int] * 5 + [_c_float]
                        + [_c_int] * 6 + [_c_void_p]),
    "nlfa_bwd_scratch_bytes": (_c_size_t, [_c_int, _c_int, _c_int]),
    "nlfa_bwd": (_c_int, [_c_void_p] * 10 + [_c_size_t] + [_c_int] * 5 + [_c_float]
                 + [_c_int] * 4 + [_c_void_p]),
    "nlfa_bwd_passes": (_c_int, [_c_void_p] * 10 + [_c_size_t] + [_c_int] * 5 + [_c_float]
                        + [_c_int] * 5 + [_c_void_p]),
    "nlfa_bwd_fused_scratch_bytes": (_c_size_t, [_c_int, _c_int, _c_int, _c_int]),
    "nlfa_bwd_kernel_count": (_c_int, [_c_int] * 7),
    "nlfa_bwd_fused": (_c_int, [_c_void_p] * 10 + [_c_size_t] + [_c_int] * 5 + [_c_float]
                       + [_c_int] * 4 + [_c_void_p]),
    "nlfa_static_scratch_max_rows": (_c_size_t, []),
    "nlfa_bwd_static_scratch": (_c_int, [_c_void_p] * 9 + [_c_int] * 5 + [_c_float]
                                + [_c_int] * 4 + [_c_void_p]),
    "nlfa_qk_prologue_fwd": (_c_int, [_c_void_p, _c_int] + [_c_void_p] * 4 + [_c_int, _c_void_p]
                             + [_c_int] * 4 + [_c_float, _c_void_p]),
    "nlfa_qk_prologue_scratch_bytes": (_c_size_t, [_c_int]),
    "nlfa_qk_prologue_bwd": (_c_int, [_c_void_p, _c_int, _c_void_p, _c_int] + [_c_void_p] * 7 + [_c_size_t]
                             + [_c_int] * 4 + [_c_void_p]),
    "nlfa_value_blend_fwd": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                                      ctypes.c_longlong, _c_void_p]),
    "nlfa_value_blend_scratch_bytes": (_c_size_t, []),
    "nlfa_value_blend_bwd": (_c_int, [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int] + [_c_void_p] * 5
                             + [_c_size_t, ctypes.c_longlong, _c_void_p]),
    "nlfa_head_gate_fwd": (_c_int, [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, ctypes.c_longlong, _c_int,
                                    _c_void_p]),
    "nlfa_head_gate_bwd": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                    ctypes.c_longlong, _c_int, _c_void_p]),
    "nlfa_fwd_cached_scratch_bytes": (_c_size_t, [_c_int] * 6),
    "nlfa_fwd_cached": (_c_int, [_c_void_p] * 7 + [_c_int] * 6 + [_c_float] + [_c_int] * 4
                        + [_c_void_p, _c_size_t, _c_void_p]),
    "nlfa_fwd_cached_path": (_c_int, [_c_void_p] * 7 + [_c_int] * 6 + [_c_float] + [_c_int] * 5
                             + [_c_void_p, _c_size_t, _c_void_p]),
    "nlfa_selftest_workspace_bytes": (_c_size_t, []),
    "nlfa_selftest": (_c_int, [_c_int, _c_int, _c_void_p, _c_size_t,
                               ctypes.POINTER(_c_float), _c_void_p]),
    "nlfa_selftest_tiles": (_c_int, [_c_int, _c_int] + [_c_void_p] * 6),
    "nlfa_check_mask_geometry": (_c_int, [_c_int] * 4),
    "nlfa_check_mask_geometry_masked": (_c_int, [_c_int] * 5),
    "nlfa_device_status": (_c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "nlfa_set_status_mirror": (_c_int, [_c_void_p]),
    "nlfa_peek_status": (_c_int, []),
    "nlfa_test_wait_timeout": (_c_int, [ctypes.c_ulonglong, _c_void_p]),
}

_lib = None


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """The loaded library; builds it in-tree first when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if not build_if_missing:
            raise OSError(f"{LIB_PATH} is missing; run python -m machinelearning_b200._build")
        from . import _build
        _build.build()
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def strerror(status: int) -> str:
    return load().nlfa_strerror(int(status)).decode()


class NlfaError(RuntimeError):
    """A non-zero status from the C ABI."""

    def __init__(self, fn: str, status: int):
        self.status = int(status)
        super().__init__(f"{fn} failed with status {status}: {strerror(status)}")


def check(fn: str, status: int) -> None:
    if status != OK:
        raise NlfaError(fn, status)
