"""The reference's torch spelling of the path, restated — TEST INFRASTRUCTURE ONLY.

Run on the SAME CUDA device as the kernels, this is the arbiter of bit-exactness
for the quantizers, exactly as the reference gates its own fused kernel
(`_quant_arms`, tests/test_quant.py:371-384): torch's CUDA kernels decide what
`amax / 448.0`, `x / scale`, `F.silu`, `torch.sigmoid` and the bf16 roundings
evaluate to.  Lines follow braid/model/quant.py:108-115 and :228-229,
braid/model/mlp.py:48, braid/model/attention.py:215 and braid/model/norm.py:31-71.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
EPS = 1e-12


def act_scale(t: torch.Tensor) -> torch.Tensor:
    return (t.detach().float().abs().amax() / FP8_MAX).clamp(min=EPS).reshape(1, 1)


def quantize_act(x: torch.Tensor):
    scale = act_scale(x)
    return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8), scale


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return o * torch.sigmoid(gate)


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """braid/model/norm.py:31-45: fp32 norm with the effective gamma, one cast back."""
    return F.rms_norm(x.float(), (x.shape[-1],), gamma, eps).type_as(x)


def rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """braid/model/norm.py:48-71: normalise, round to the activation type, gamma, silu(gate) in fp32."""
    input_dtype = x.dtype
    xf = F.rms_norm(x.float(), (x.shape[-1],), None, eps)
    h = gamma * xf.to(input_dtype)
    h = h * F.silu(gate.float())
    return h.to(input_dtype)


def scaled_mm(xq, sx, wq, sw, out_dtype=torch.bfloat16):
    """The library GEMM the reference calls (braid/model/quant.py:240-241)."""
    return torch._scaled_mm(xq, wq.t(), scale_a=sx, scale_b=sw, out_dtype=out_dtype)


def dequant_matmul(xq, sx, wq, sw) -> torch.Tensor:
    """fp32 dequantize-and-multiply: the tolerance reference for large shapes on the GPU."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return (xq.float() * sx) @ (wq.float() * sw).t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
