"""braid_b200 — the FP8 W8A8 projection path of plind-junior/braid, rebuilt for B200 (sm_100a).

`braid_b200.quant` mirrors `braid.model.quant`; `braid_b200.integrate.install_into`
rebinds a loaded reference module onto these kernels; `braid_b200.parallel` holds the
data-parallel and column-parallel (N-split MLP) multi-GPU forms.
"""
from . import quant  # noqa: F401

__all__ = ["quant"]
__version__ = "0.1.0"
