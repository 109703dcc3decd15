"""The path spelled for a CPU with torch ops — TEST INFRASTRUCTURE / TIMED BASELINE ONLY.

The quantizer is the reference's spelling verbatim in meaning (braid/model/quant.py:108-115,
:228-229; on a CPU `amax / 448.0` is a true division).  The product is the practical CPU form
of braid/model/quant.py:232-241: dequantize both operands to fp32 and multiply on all cores
(torch's CPU `_scaled_mm` is a scalar loop — minutes for one decode projection — so it is only
timed on slices, see `scaled_mm_slice_seconds`).
"""
from __future__ import annotations

import time

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
EPS = 1e-12


def quantize(x: torch.Tensor):
    scale = (x.detach().float().abs().amax() / FP8_MAX).clamp(min=EPS).reshape(1, 1)
    return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8), scale


def matmul(xq, sx, wq, sw, out_dtype=torch.bfloat16):
    return ((xq.float() * sx) @ (wq.float() * sw).t()).to(out_dtype)


def linear(x, wq, sw):
    xq, sx = quantize(x)
    return matmul(xq, sx, wq, sw, x.dtype)


def project(x, *weights):
    xq, sx = quantize(x)
    return [matmul(xq, sx, wq, sw, x.dtype) for wq, sw in weights]


def mlp(x, gate, up, down):
    g, u = project(x, gate, up)
    return linear(F.silu(g) * u, *down)


def scaled_mm_slice_seconds(xq, sx, wq, sw, rows: int = 256) -> float:
    """Seconds torch's own CPU `_scaled_mm` takes on the first `rows` weight rows."""
    w = wq[:rows].contiguous()
    t0 = time.perf_counter()
    torch._scaled_mm(xq, w.t(), scale_a=sx, scale_b=sw, out_dtype=torch.bfloat16)
    return time.perf_counter() - t0
