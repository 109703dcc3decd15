"""ctypes binding of `libbraid_b200.so` — the C ABI declared in include/braid_b200.h.

The library has no torch types in its signatures: device pointers travel as
integers (`tensor.data_ptr()`), the stream as `torch.cuda.current_stream().cuda_stream`.
Loading fails loudly; there is no other implementation to fall back to.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

# BRAID_B200_LIB selects another build of the same library (the development build with phase
# stamps, `python -m braid_b200.build --phases`); unset, the in-tree product library is loaded.
LIB_PATH = Path(os.environ.get("BRAID_B200_LIB") or Path(__file__).resolve().parent / "libbraid_b200.so")

BQ_OK = 0
BQ_ERR_BAD_ARG = 1
BQ_ERR_UNSUPPORTED = 2
BQ_ERR_LAUNCH = 3
BQ_ERR_WORKSPACE = 4
BQ_ERR_DEVICE_WAIT = 5
BQ_ERR_NO_DRIVER = 6
BQ_ERR_TOO_LARGE = 7

BQ_DTYPE_F32, BQ_DTYPE_BF16, BQ_DTYPE_F16 = 0, 1, 2
BQ_MAX_SEGMENTS = 8

# name -> (restype, argtypes); the single source of truth for the symbol check
_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
SIGNATURES = {
    "bq_version": (_int, []),
    "bq_status_string": (ctypes.c_char_p, [_int]),
    "bq_scratchless_status": (_int, [ctypes.POINTER(ctypes.c_int)]),
    "bq_quant_workspace_bytes": (_sz, []),
    "bq_quantize_act": (_int, [_vp, _int, _i64, _vp, _vp, _vp, _sz, _vp]),
    "bq_quantize_act_static": (_int, [_vp, _int, _i64, _vp, _vp, _vp]),
    "bq_silu_mul_quant": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    "bq_silu_mul_scale": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _sz, _vp]),
    "bq_silu_mul_cast": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp]),
    "bq_sigmoid_gate_quant": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, _i64,
                                     _vp, _vp, _vp, _sz, _vp]),
    "bq_silu_mul": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp]),
    "bq_sigmoid_mul": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "bq_silu_mul_dense_scale": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    "bq_sigmoid_mul_dense_scale": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp,
                                          _vp, _sz, _vp]),
    "bq_rmsnorm_quant": (_int, [_vp, _int, _i64, _i64, _i64, _vp, ctypes.c_float, _vp, _i64, _vp, _vp,
                                _vp, _sz, _vp]),
    "bq_rmsnorm_scale": (_int, [_vp, _int, _i64, _i64, _i64, _vp, ctypes.c_float, _vp, _i64, _vp,
                                _vp, _sz, _vp]),
    "bq_gated_rmsnorm_quant": (_int, [_vp, _int, _i64, _vp, _int, _i64, _vp, ctypes.c_float, _i64, _i64,
                                      _i64, _vp, _vp, _vp, _sz, _vp]),
    "bq_gated_rmsnorm_scale": (_int, [_vp, _int, _i64, _vp, _int, _i64, _vp, ctypes.c_float, _i64, _i64,
                                      _i64, _vp, _i64, _vp, _vp, _sz, _vp]),
    "bq_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "bq_gemm_w8a8": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    "bq_gemm_w8a8_residual": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _int, _i64, _i64, _i64, _i64,
                                     _vp, _sz, _vp]),
    "bq_gate_up_silu_quant_w8a8": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp,
                                          _vp, _vp, _sz, _vp]),
    "bq_enable_peer_access": (_int, [_int]),
    "bq_peer_alloc": (_int, [_sz, ctypes.POINTER(_vp), _vp]),
    "bq_peer_free": (_int, [_vp]),
    "bq_peer_open": (_int, [_vp, ctypes.POINTER(_vp)]),
    "bq_peer_close": (_int, [_vp]),
    "bq_gemm_w8a8_push": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _int,
                                 ctypes.POINTER(_vp), _i64, ctypes.POINTER(_vp), _vp, _sz, _vp]),
    "bq_gate_up_silu_push_w8a8": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int,
                                         ctypes.POINTER(_vp), _i64, ctypes.POINTER(_vp),
                                         ctypes.POINTER(_vp), _vp, _sz, _vp]),
    "bq_wait_flag": (_int, [_vp, _vp, ctypes.c_uint, _vp, _vp]),
    "bq_wait_flag_scale": (_int, [_vp, _vp, ctypes.c_uint, _vp, _vp, _int, _int, _vp, _vp]),
    "bq_word_push": (_int, [_vp, _int, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _vp]),
    "bq_cast_act_push": (_int, [_vp, _int, _i64, _i64, _i64, _vp, _int, ctypes.POINTER(_vp), _i64,
                                ctypes.POINTER(_vp), _vp, _sz, _vp]),
    "bq_rows_push": (_int, [_vp, _int, _i64, _i64, _i64, _int, ctypes.POINTER(_vp), _i64,
                            ctypes.POINTER(_vp), _vp, _sz, _vp]),
    "bq_quantize_act_after": (_int, [_vp, _int, _i64, _vp, _vp, _vp, _vp, ctypes.c_uint, _vp, _sz, _vp]),
    "bq_gemm_w8a8_grouped": (_int, [_vp, _vp, _i64, _i64, _int,
                                    ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                    ctypes.POINTER(_i64), ctypes.POINTER(_i64), _int,
                                    _vp, _sz, _vp]),
    "bq_project_mixed": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _int,
                                ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_int),
                                ctypes.POINTER(_vp), ctypes.POINTER(_i64), ctypes.POINTER(_i64), _int,
                                _vp, _sz, _vp]),
    "bq_lm_head_argmax_workspace_bytes": (_sz, [_i64, _i64]),
    "bq_lm_head_argmax": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _sz,
                                 _vp, _sz, _vp]),
    "bq_gate_up_silu_w8a8": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _i64, _vp,
                                    _vp, _sz, _vp]),
    "bq_cast_act": (_int, [_vp, _int, _i64, _vp, _vp, _vp]),
    "bq_read_device_status": (_int, [_vp, _vp, ctypes.POINTER(_int)]),
    "bq_set_option": (_int, [ctypes.c_char_p, _i64]),
    "bq_last_gemm_launch": (_int, [ctypes.POINTER(_i64)]),
}

_lib: ctypes.CDLL | None = None


class LibraryMissing(RuntimeError):
    """`libbraid_b200.so` is not built or cannot be loaded."""


def load() -> ctypes.CDLL:
    """Load the library once and attach the signatures.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryMissing(
            f"{LIB_PATH} not found: build it with `python -m braid_b200.build` "
            "(needs nvcc); braid_b200 has no other implementation of its kernels")
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError as e:
        raise LibraryMissing(f"cannot load {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the symbol is missing: loud
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().bq_status_string(code).decode()


def check(code: int, what: str) -> None:
    """Turn a non-zero status into the exception class the reference would raise."""
    if code == BQ_OK:
        return
    msg = f"{what}: {status_string(code)} (status {code})"
    if code in (BQ_ERR_BAD_ARG, BQ_ERR_UNSUPPORTED, BQ_ERR_TOO_LARGE):
        raise ValueError(msg)
    raise RuntimeError(msg)
