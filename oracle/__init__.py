"""CPU oracle for the FP8 W8A8 projection path — TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke test and the benchmark's CPU-baseline leg may
import this package, and only as the checker / the timed baseline.  The product
package (`braid_b200`) never imports it and has no CPU fallback.

`w8a8_oracle.c` is the restatement (plain C, OpenMP for the product); this
module builds it with gcc and exposes it over numpy arrays.  Inputs of a 16-bit
type are passed widened to fp32, which is exact.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "w8a8_oracle.c"
LIB = HERE / "_build" / "libw8a8_oracle.so"

SCALE_RCP = 0   # amax * (1/448): what torch evaluates on a CUDA device
SCALE_DIV = 1   # amax / 448:     what torch evaluates on the CPU

DT_F32, DT_BF16, DT_F16 = 0, 1, 2

_lib = None


def build(force: bool = False) -> Path:
    """gcc -O3 -fopenmp -shared; strict IEEE (no -ffast-math, no contraction)."""
    if LIB.exists() and not force and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    LIB.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-mavx2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off",
           "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("gcc failed building the oracle:\n" + proc.stderr)
    return LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
        u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
        i64, f32, i32 = ctypes.c_int64, ctypes.c_float, ctypes.c_int
        _lib.oracle_e4m3_decode.restype = f32
        _lib.oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
        _lib.oracle_e4m3_encode.restype = ctypes.c_uint8
        _lib.oracle_e4m3_encode.argtypes = [f32]
        _lib.oracle_e4m3_encode_array.restype = None
        _lib.oracle_e4m3_encode_array.argtypes = [f32p, i64, u8p]
        _lib.oracle_amax.restype = f32
        _lib.oracle_amax.argtypes = [f32p, i64]
        _lib.oracle_scale_from_amax.restype = f32
        _lib.oracle_scale_from_amax.argtypes = [f32, i32]
        _lib.oracle_cast.restype = None
        _lib.oracle_cast.argtypes = [f32p, i64, f32, u8p]
        _lib.oracle_quantize.restype = f32
        _lib.oracle_quantize.argtypes = [f32p, i64, i32, u8p]
        _lib.oracle_silu_mul.restype = None
        _lib.oracle_silu_mul.argtypes = [f32p, f32p, i64, i32, f32p]
        _lib.oracle_sigmoid_gate.restype = None
        _lib.oracle_sigmoid_gate.argtypes = [f32p, f32p, i64, i32, f32p]
        _lib.oracle_gemm.restype = None
        _lib.oracle_gemm.argtypes = [u8p, u8p, f32, f32, i64, i64, i64, f32p]
        _lib.oracle_gemm_f32.restype = None
        _lib.oracle_gemm_f32.argtypes = [u8p, u8p, f32, f32, i64, i64, i64, f32p, f32p, f32p]
        _lib.oracle_num_threads.restype = i32
        _lib.oracle_num_threads.argtypes = []
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint8))


def e4m3_decode_table() -> np.ndarray:
    """All 256 codes as fp32 (0x7F / 0xFF are NaN)."""
    L = lib()
    return np.array([L.oracle_e4m3_decode(i) for i in range(256)], dtype=np.float32)


def e4m3_encode(x) -> np.ndarray:
    """Elementwise round-to-nearest-even cast of fp32 values, no scaling, no clamp."""
    x = _f32(x)
    q = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_e4m3_encode_array(x.reshape(-1), x.size, q.reshape(-1))
    return q


def amax(x) -> float:
    x = _f32(x)
    return float(lib().oracle_amax(x.reshape(-1), x.size))


def scale_from_amax(a: float, mode: int = SCALE_RCP) -> np.float32:
    return np.float32(lib().oracle_scale_from_amax(np.float32(a), mode))


def quantize(x, mode: int = SCALE_RCP):
    """`quantize_act` / `quantize_weight`: (codes uint8 of x.shape, scale fp32)."""
    x = _f32(x)
    q = np.empty(x.shape, dtype=np.uint8)
    s = lib().oracle_quantize(x.reshape(-1), x.size, mode, q.reshape(-1))
    return q, np.float32(s)


def cast(x, scale) -> np.ndarray:
    """clamp(x / scale, +-448) -> e4m3fn codes, for a scale decided elsewhere."""
    x = _f32(x)
    q = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_cast(x.reshape(-1), x.size, np.float32(scale), q.reshape(-1))
    return q


def silu_mul(gate, up, dt: int = DT_BF16) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    h = np.empty(gate.shape, dtype=np.float32)
    lib().oracle_silu_mul(gate.reshape(-1), up.reshape(-1), gate.size, dt, h.reshape(-1))
    return h


def sigmoid_gate(o, gate, dt: int = DT_BF16) -> np.ndarray:
    o, gate = _f32(o), _f32(gate)
    h = np.empty(o.shape, dtype=np.float32)
    lib().oracle_sigmoid_gate(o.reshape(-1), gate.reshape(-1), o.size, dt, h.reshape(-1))
    return h


def gemm(xq, wq, sx, sw) -> np.ndarray:
    """Exact dequantize-and-multiply, fp32 result [M, N]."""
    xq, wq = _u8(xq), _u8(wq)
    M, K = xq.shape
    N, K2 = wq.shape
    assert K == K2
    y = np.empty((M, N), dtype=np.float32)
    lib().oracle_gemm(xq, wq, np.float32(sx), np.float32(sw), M, N, K, y)
    return y


def gemm_f32(xq, wq, sx, sw) -> np.ndarray:
    """The fast CPU spelling (fp32 accumulate, all cores): the timed baseline."""
    xq, wq = _u8(xq), _u8(wq)
    M, K = xq.shape
    N, _ = wq.shape
    y = np.empty((M, N), dtype=np.float32)
    xf = np.empty((M, K), dtype=np.float32)
    scratch = np.empty((1,), dtype=np.float32)
    lib().oracle_gemm_f32(xq, wq, np.float32(sx), np.float32(sw), M, N, K, xf, scratch, y)
    return y


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def max_rel(y, ref) -> float:
    """max|y - ref| / max|ref| over the tensor — the GEMM tolerance metric."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = float(np.max(np.abs(ref)))
    return float(np.max(np.abs(y - ref)) / denom) if denom > 0 else float(np.max(np.abs(y)))
