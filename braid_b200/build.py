"""Ahead-of-time build of the C-ABI library (`libbraid_b200.so`) with nvcc.

The reference engine JIT-builds its extension on first use
(braid/kernels/loader.py:10-44: `torch.utils.cpp_extension.load`, `-O3 -lineinfo`,
no fast-math).  Here the library is built once, in-tree, for sm_100a only, and
loaded with ctypes — it has no torch or Python dependency at all.  Flags keep
the reference's numerics contract: no `--use_fast_math`, IEEE division and
square root, no flush-to-zero.

Run `python -m braid_b200.build` to (re)build; `python -m braid_b200.build -v`
adds `-Xptxas -v` (registers, spills, shared memory per kernel).
`python -m braid_b200.build --phases` builds a second, development-only library
(`libbraid_b200_phases.so`, compiled with `-DBQ_PHASES`) whose decode-regime kernels stamp
the time of each of their phases; `BRAID_B200_LIB=<path>` makes the package load it
(`python bench.py --sweep --only phases` prints the table).  The shipped library contains
none of that code.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libbraid_b200.so"
SOURCES = ("quant_act.cu", "norm_quant.cu", "gemm_w8a8.cu", "cabi.cu")
HEADERS = (CSRC / "ptx.cuh", CSRC / "quant_device.cuh", CSRC / "grid_amax.cuh",
           PKG.parent / "include" / "braid_b200.h")


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is needed to build libbraid_b200.so")
    return cand


def is_stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(HEADERS)
    return any(d.stat().st_mtime > built for d in deps)


PHASES_LIB = PKG / "libbraid_b200_phases.so"


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (),
          out: Path | None = None) -> Path:
    """Compile the CUDA sources for sm_100a into one shared library."""
    if out is None and not defines and not force and not is_stale():
        return LIB
    LIB = out if out is not None else globals()["LIB"]
    cmd = [
        nvcc_path(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-shared", "-Xcompiler", "-fPIC",
        "--ftz=false", "--prec-div=true", "--prec-sqrt=true", "--fmad=true",
        "-cudart", "static",
        "-I", str(PKG.parent / "include"),
        "-o", str(LIB),
    ]
    cmd += [f"-D{d}" for d in defines]
    if verbose or os.environ.get("BRAID_B200_VERBOSE") == "1":
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    if "--phases" in sys.argv[1:]:
        print(build(force=True, verbose="-v" in sys.argv[1:], defines=("BQ_PHASES",), out=PHASES_LIB))
    else:
        print(build(force=True, verbose="-v" in sys.argv[1:]))
