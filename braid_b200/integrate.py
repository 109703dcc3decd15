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


def fused_mlp_forward(self, x, residual=None):
    """Replacement for `MLP.forward` (braid/model/mlp.py:34-49): the quantized branch as
    `quant.mlp_forward` runs it (3 launches at decode sizes, 4 at prefill sizes); `residual`, if
    given, is added in the epilogue of the down projection."""
    import torch.nn.functional as F
    if not isinstance(self.gate_proj, Q.FP8Weight):
        y = F.linear(F.silu(F.linear(x, self.gate_proj)) * F.linear(x, self.up_proj), self.down_proj)
        return y if residual is None else residual + y
    return Q.mlp_forward(x, self.gate_proj, self.up_proj, self.down_proj, residual=residual)


def fused_layer_forward(self, x, cos, sin, cache=None, slots=None, positions=None, kv_len=None,
                        attn_mask=None, slots_i32=None, seq_lens=None):
    """Replacement for `DecoderLayer.forward` (braid/model/layer.py:37-60): each pre-norm is fused
    into the quantizer of the sublayer it feeds, so the mixer's `project` and the MLP receive an
    already-quantized activation.  A sublayer whose weights are not FP8 gets the plain norm.  The
    GDN mixer also reads the normalised activation unquantized (its bf16 a/b gates,
    braid/model/gdn.py:73-81), so that one is written out as well.  Both residual adds
    (layer.py:57,60) ride in the epilogue of the projection that produces the summand: the
    mixer's out_proj / o_proj through `residual_into`, the MLP's down_proj directly."""
    eps = self.cfg.rms_norm_eps
    if self.mixer.quantized:
        h = Q.rms_norm_quant(x, self.input_layernorm, eps, keep_dense=self.is_gdn)
    else:
        h = Q.torch_rms_norm(x, self.input_layernorm, eps)
    # the residual add rides in the epilogue of the mixer's output projection when that is FP8
    out_w = self.mixer.out_proj if self.is_gdn else self.mixer.o_proj
    with Q.residual_into(out_w if isinstance(out_w, Q.FP8Weight) else None, x) as slot:
        if self.is_gdn:
            h = self.mixer(h, cache=cache, slots=slots, slots_i32=slots_i32, seq_lens=seq_lens)
        else:
            h = self.mixer(h, cos, sin, attn_mask=attn_mask, cache=cache, slots=slots,
                           positions=positions, kv_len=kv_len, seq_lens=seq_lens)
    x = h if slot.taken else x + h
    if self.mlp.quantized:
        h = Q.rms_norm_quant(x, self.post_attention_layernorm, eps)
        return fused_mlp_forward(self.mlp, h, residual=x)
    h = Q.torch_rms_norm(x, self.post_attention_layernorm, eps)
    return x + self.mlp(h)


def fused_gdn_readout(self, z, y, B, T, dtype):
    """Replacement for `GatedDeltaNet._readout` (braid/model/gdn.py:373-387): the cast of the scan
    output, the gated norm and the quantization of out_proj's input in one launch."""
    g = self.g
    if not isinstance(self.out_proj, Q.FP8Weight) or z.dtype != dtype:
        core = Q.torch_rms_norm_gated(y.to(dtype).reshape(-1, g.head_dim), z.reshape(-1, g.head_dim),
                                      self.norm, self.cfg.rms_norm_eps)
        return Q.linear(core.reshape(B, T, g.inner_size), self.out_proj)
    core = Q.gated_rms_norm_quant(y.reshape(B, T, g.inner_size), z.reshape(B, T, g.inner_size),
                                  self.norm, self.cfg.rms_norm_eps, g.head_dim)
    return Q.linear(core, self.out_proj)


def fused_final_norm(x, weight, eps):
    """Replacement for the `rms_norm` name the engine module imported (braid/model/engine.py:29):
    its two call sites are the final norm in front of lm_head (:263, :348).  Returns the
    normalised tensor torch would have returned, bit for bit, but computed together with its FP8
    codes in one launch; the codes ride along on the tensor (`quant.attach_quantized`), so the
    `linear(h, self.lm_head)` that follows skips its quantizer when lm_head is FP8.  Anything the
    kernel does not take runs the reference's spelling."""
    if (not x.is_cuda or x.dtype not in Q._DTYPE_CODE or weight.dtype is not __import__("torch").float32
            or weight.numel() != x.shape[-1]):
        return Q.torch_rms_norm(x, weight, eps)
    qa = Q.rms_norm_quant(x, weight, eps, keep_dense=True)
    return Q.attach_quantized(qa.dense, qa)
