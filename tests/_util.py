"""Helpers shared by the tests: bit views, seeded inputs, numpy bridges."""
from __future__ import annotations

import numpy as np
import torch


def u8(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


def to_np_f32(t: torch.Tensor) -> np.ndarray:
    """Exact widening of a float tensor to a numpy fp32 array."""
    return t.detach().float().cpu().numpy()


def codes_np(t: torch.Tensor) -> np.ndarray:
    return u8(t).cpu().numpy()


def from_bits16(bits: np.ndarray, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(dtype)


def from_bits32(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int32).copy()).view(torch.float32)


def f32_bits(t: torch.Tensor) -> int:
    return int(t.detach().float().cpu().view(torch.int32).reshape(-1)[0].item()) & 0xFFFFFFFF


def randn_cpu(shape, seed, dtype=torch.bfloat16, scale=1.0) -> torch.Tensor:
    """Seeded on the CPU so that CPU and GPU arms see identical bits."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def config1_inputs(seed: int = 0):
    """BASELINE config 1 inputs, generated exactly as tests/golden/make_golden.py does."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(8, 4096, generator=g, dtype=torch.float32)
    mask = torch.rand(8, 4096, generator=g) < 1e-3
    x = torch.where(mask, x * 50.0, x).to(torch.bfloat16)
    w = (torch.randn(4096, 4096, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return x, w


def max_rel(y: torch.Tensor, ref: torch.Tensor) -> float:
    y, ref = y.double(), ref.double()
    return float((y - ref).abs().max() / ref.abs().max().clamp_min(1e-300))
