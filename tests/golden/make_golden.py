"""Generates tests/golden/w8a8_golden.npz by RUNNING THE REFERENCE ITSELF on the CPU.

Usage (needs the reference checkout; it is not needed to run the tests):

    PYTHONPATH=/path/to/braid python tests/golden/make_golden.py

Everything stored is an output of `braid.model.quant` / `braid.model.mlp` (torch
spelling; `fused_state() == "not tried"`), on seeded inputs that are either
stored beside the outputs (small cases) or regenerated from the seed and guarded
by a checksum (large cases).  On a CPU torch evaluates `amax / 448.0` as a true
division, so these vectors pin the oracle's SCALE_DIV spelling, the e4m3 cast,
the bf16 double rounding of SiLU*mul / sigmoid-gate, and the GEMM tolerance; the
CUDA spelling of the scale (reciprocal multiply) is pinned on the GPU against
torch's own CUDA kernels.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "w8a8_golden.npz"


def sha(t: torch.Tensor) -> np.ndarray:
    raw = t.contiguous().view(torch.uint8).numpy().tobytes()
    return np.frombuffer(hashlib.sha256(raw).digest(), dtype=np.uint8).copy()


def bits16(t: torch.Tensor) -> np.ndarray:
    """bf16 / fp16 tensor -> its raw uint16 bit patterns."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def f32bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int32).numpy().view(np.uint32).copy()


def codes(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def config1_inputs(seed: int = 0):
    """BASELINE config 1: X [8,4096] ~N(0,1) with 0.1% of entries x50, W [4096,4096] ~N(0,0.02)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(8, 4096, generator=g, dtype=torch.float32)
    mask = torch.rand(8, 4096, generator=g) < 1e-3
    x = torch.where(mask, x * 50.0, x).to(torch.bfloat16)
    w = (torch.randn(4096, 4096, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return x, w


def main() -> None:
    from braid.model import quant as Q
    from braid.model.mlp import MLP

    assert Q.fused_state() == "not tried"
    torch.manual_seed(0)
    out: dict[str, np.ndarray] = {}

    # ---- quantize_act, the reference's own parity shapes (tests/test_quant.py:387-390)
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16"), (torch.float32, "f32")):
        for shape in ((1, 4096), (8, 4096), (37, 12288)):
            g = torch.Generator().manual_seed(17)
            x = (torch.randn(*shape, generator=g, dtype=torch.float32) * 3.5).to(dt)
            q, s = Q.quantize_act(x)
            key = f"act_{tag}_{shape[0]}x{shape[1]}"
            out[key + "_xsha"] = sha(x)
            out[key + "_scale"] = f32bits(s)
            out[key + "_qsha"] = sha(q)
            if shape[0] <= 8:
                out[key + "_x"] = f32bits(x) if dt is torch.float32 else bits16(x)
                out[key + "_q"] = codes(q)

    # ---- degenerate scales and NaN (tests/test_quant.py:404-421, :452-477)
    for label, fill in (("zeros", 0.0), ("huge", 60000.0), ("tiny", 1e-10)):
        x = torch.full((4, 4096), fill, dtype=torch.bfloat16)
        q, s = Q.quantize_act(x)
        out[f"deg_{label}_scale"] = f32bits(s)
        out[f"deg_{label}_q"] = codes(q)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 4096, generator=g, dtype=torch.bfloat16)
    x[2, 100] = float("nan")
    q, s = Q.quantize_act(x)
    out["nan_x"] = bits16(x)
    out["nan_scale"] = f32bits(s)
    out["nan_q"] = codes(q)

    # ---- quantize_weight (the generator of tests/test_quant.py:41-43, smaller shape)
    g = torch.Generator().manual_seed(7)
    w = torch.randn(256, 128, generator=g, dtype=torch.bfloat16) * 0.02
    fw = Q.quantize_weight(w)
    out["weight_w"] = bits16(w)
    out["weight_scale"] = f32bits(fw.scale)
    out["weight_q"] = codes(fw.data)

    # ---- small GEMM through the reference: fp8_linear and project
    g = torch.Generator().manual_seed(11)
    x = torch.randn(16, 128, generator=g, dtype=torch.bfloat16)
    b = torch.randn(64, 128, generator=g, dtype=torch.bfloat16) * 0.03
    fb = Q.quantize_weight(b)
    xq, sx = Q.quantize_act(x)
    ya, yb = Q.project(x, fw, fb)
    out["gemm_x"] = bits16(x)
    out["gemm_xq"] = codes(xq)
    out["gemm_sx"] = f32bits(sx)
    out["gemm_wb"] = bits16(b)
    out["gemm_wbq"] = codes(fb.data)
    out["gemm_wb_scale"] = f32bits(fb.scale)
    out["gemm_ya"] = bits16(ya)
    out["gemm_yb"] = bits16(yb)
    assert torch.equal(ya, Q.fp8_linear(x, fw))

    # ---- the quantized MLP, with its bf16 intermediate (braid/model/mlp.py:44-49)
    cfg = SimpleNamespace(hidden_act="silu")
    g = torch.Generator().manual_seed(3)
    r = lambda N, K: torch.randn(N, K, generator=g, dtype=torch.bfloat16) * 0.05  # noqa: E731
    wts = {"mlp.gate_proj": r(256, 128), "mlp.up_proj": r(256, 128), "mlp.down_proj": r(128, 256)}
    x = torch.randn(4, 128, generator=g, dtype=torch.bfloat16)
    mlp = MLP(cfg, wts, quant=True)
    y = mlp(x)
    xq, sx = Q.quantize_act(x)
    gate = Q.fp8_matmul(xq, sx, mlp.gate_proj, out_dtype=x.dtype)
    up = Q.fp8_matmul(xq, sx, mlp.up_proj, out_dtype=x.dtype)
    h = F.silu(gate) * up
    hq, sh = Q.quantize_act(h)
    for k, v in wts.items():
        out["mlp_" + k.split(".")[1]] = bits16(v)
    out["mlp_x"] = bits16(x)
    out["mlp_gate"] = bits16(gate)
    out["mlp_up"] = bits16(up)
    out["mlp_h"] = bits16(h)
    out["mlp_hq"] = codes(hq)
    out["mlp_sh"] = f32bits(sh)
    out["mlp_y"] = bits16(y)

    # ---- sigmoid gate (braid/model/attention.py:215) on the strided per-head view
    g = torch.Generator().manual_seed(21)
    H, D = 4, 64
    qg = torch.randn(2, 3, H * 2 * D, generator=g, dtype=torch.bfloat16) * 2.0
    o = torch.randn(2, 3, H * D, generator=g, dtype=torch.bfloat16)
    _, gate_v = qg.view(2, 3, H, 2 * D).chunk(2, dim=-1)
    og = o * torch.sigmoid(gate_v.reshape(2, 3, H * D))
    oq, so = Q.quantize_act(og.reshape(-1, H * D))
    out["sig_qg"] = bits16(qg)
    out["sig_o"] = bits16(o)
    out["sig_og"] = bits16(og)
    out["sig_oq"] = codes(oq)
    out["sig_so"] = f32bits(so)

    # ---- BASELINE config 1 end to end on the CPU (about 2 s of scalar _scaled_mm)
    x, w = config1_inputs(0)
    fw1 = Q.quantize_weight(w)
    xq, sx = Q.quantize_act(x)
    y = Q.fp8_matmul(xq, sx, fw1, out_dtype=torch.bfloat16)
    ref = (xq.float() * sx) @ (fw1.data.float() * fw1.scale).t()
    out["c1_xsha"] = sha(x)
    out["c1_wsha"] = sha(w)
    out["c1_xq"] = codes(xq)
    out["c1_sx"] = f32bits(sx)
    out["c1_wqsha"] = sha(fw1.data)
    out["c1_sw"] = f32bits(fw1.scale)
    out["c1_y"] = bits16(y)
    out["c1_maxrel"] = np.array([float((y.float() - ref).abs().max() / ref.abs().max())])

    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.1f} KiB, {len(out)} arrays), "
          f"torch {torch.__version__}, config-1 max-rel {out['c1_maxrel'][0]:.3e}")


if __name__ == "__main__":
    if not any(Path(p, "braid", "model", "quant.py").exists() for p in sys.path if p):
        sys.exit("put the reference checkout on PYTHONPATH (see the docstring)")
    main()
