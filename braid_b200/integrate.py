"""Rebinding a loaded `braid.model.quant` (and the modules that imported names from it) onto
these kernels — the drop-in step a maintainer of the reference would take.

The reference binds some names at import time (`braid/model/mlp.py:16` imports `fp8_matmul` and
`quantize_act` by name; `gdn.py:35` and `attention.py:27` import `project` and `linear`), so
replacing attributes of `braid.model.quant` alone is not enough: every module that holds its own
reference is patched as well.  `FP8Weight` objects are duck-compatible (`data`, `scale`, `shape`),
so weights quantized by either module work with either set of functions.
"""
from __future__ import annotations

import sys
from types import ModuleType

from . import quant as Q

_REBOUND = ("quantize_act", "fp8_matmul", "fp8_linear", "linear", "project", "warm_fused",
            "fused_state")


def install_into(ref_quant: ModuleType, extra_modules: tuple[str, ...] = (
        "braid.model.mlp", "braid.model.gdn", "braid.model.attention", "braid.model.engine")) -> list[str]:
    """Point the reference's quant API at braid_b200.  Returns the names that were rebound.

    `isinstance(w, FP8Weight)` checks inside the rebound functions use braid_b200's class, so the
    reference's `FP8Weight` is replaced too; weights must be quantized after installing (or be
    re-wrapped with `adopt_weight`).
    """
    Q.warm_fused(True)
    done = []
    for name in _REBOUND + ("FP8Weight", "quantize_weight", "maybe_quantize"):
        setattr(ref_quant, name, getattr(Q, name))
        done.append(f"{ref_quant.__name__}.{name}")
    ref_quant._FUSED = Q._FUSED
    ref_quant._FUSED_STATE = Q._FUSED_STATE
    for mod_name in extra_modules:
        mod = sys.modules.get(mod_name)
        if mod is None:
            continue
        for name in _REBOUND + ("FP8Weight", "maybe_quantize"):
            if hasattr(mod, name):
                setattr(mod, name, getattr(Q, name))
                done.append(f"{mod_name}.{name}")
    return done


def adopt_weight(w) -> Q.FP8Weight:
    """Wrap a reference `FP8Weight` (same fields) as a braid_b200 one without copying."""
    return Q.FP8Weight(data=w.data, scale=w.scale, shape=tuple(w.shape))


def fused_mlp_forward(self, x):
    """Replacement for `MLP.forward` (braid/model/mlp.py:34-49): quantized branch in 4 launches."""
    import torch.nn.functional as F
    if not isinstance(self.gate_proj, Q.FP8Weight):
        return F.linear(F.silu(F.linear(x, self.gate_proj)) * F.linear(x, self.up_proj), self.down_proj)
    return Q.mlp_forward(x, self.gate_proj, self.up_proj, self.down_proj)
