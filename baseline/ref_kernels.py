"""The reference's own CUDA extension (GDN scan, slotted conv1d, its two-launch fused quantizer),
built ahead of time for sm_100a so the reference engine can run with `use_kernels=True` on a box
that has neither the reference checkout nor time to JIT-compile.

    python baseline/ref_kernels.py --reference <checkout of the reference>

compiles `braid/kernels/csrc/{bindings.cpp,gdn_decode.cu,conv1d_decode.cu,quant_act.cu}` where
they lie in that checkout, with the flags of the reference's own loader
(braid/kernels/loader.py:20-44: `-O3 -lineinfo`, no fast-math) and `TORCH_CUDA_ARCH_LIST=10.0a`
in place of its 12.0a default, into `baseline/_ref/_prebuilt/` (beside the pip install of the
reference; neither is part of the repository).  No source file is copied.

`attach()` imports the prebuilt module and makes the installed reference's
`braid.kernels.loader.load_gdn` return it, which is the only thing `GatedDeltaNet` and
`warm_fused` ask of that loader (braid/model/gdn.py:98-100, braid/model/quant.py:174-201).
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_INSTALL = HERE / "_ref"
PREBUILT = REF_INSTALL / "_prebuilt"
NAME = "braid_gdn"
SOURCES = ("bindings.cpp", "gdn_decode.cu", "conv1d_decode.cu", "quant_act.cu")


def build(reference: Path, verbose: bool = False) -> Path:
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    os.environ.setdefault("MAX_JOBS", "8")
    from torch.utils.cpp_extension import load
    csrc = Path(reference) / "braid" / "kernels" / "csrc"
    missing = [s for s in SOURCES if not (csrc / s).exists()]
    if missing:
        raise FileNotFoundError(f"{csrc}: missing {missing}")
    PREBUILT.mkdir(parents=True, exist_ok=True)
    load(name=NAME, sources=[str(csrc / s) for s in SOURCES], extra_cuda_cflags=["-O3", "-lineinfo"],
         build_directory=str(PREBUILT), verbose=verbose)
    return prebuilt_path()


def prebuilt_path() -> Path:
    return PREBUILT / f"{NAME}.so"


def available() -> bool:
    return prebuilt_path().exists() and (REF_INSTALL / "braid" / "kernels" / "loader.py").exists()


def attach():
    """Import the prebuilt extension and route the installed reference's loader to it."""
    if not available():
        raise FileNotFoundError(f"no prebuilt reference extension at {prebuilt_path()}")
    import torch  # noqa: F401  (the extension links against libtorch)
    if NAME in sys.modules:
        mod = sys.modules[NAME]
    else:
        spec = importlib.util.spec_from_file_location(NAME, prebuilt_path())
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[NAME] = mod
    loader = importlib.import_module("braid.kernels.loader")
    loader.load_gdn = lambda: mod
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", required=True, type=Path)
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.verbose))
