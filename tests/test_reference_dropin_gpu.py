"""The drop-in claim, exercised with the reference's own code on the GPU.

Needs an install of the reference under baseline/_ref (made with
`python -m pip install --no-index --no-build-isolation --target baseline/_ref <reference checkout>`;
the folder is not part of the repository).  Skipped when it is absent.  The reference's
sublayers (`braid.model.mlp.MLP`) and operator functions are run twice on the same inputs: once
stock (torch spelling + `torch._scaled_mm`), once after `braid_b200.integrate.install_into` has
rebound them onto these kernels.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from _util import max_rel, randn_cpu

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "braid" / "model" / "quant.py").exists(),
                                 reason="no reference install under baseline/_ref")]


@pytest.fixture()
def ref_modules():
    """Freshly imported reference modules, removed again afterwards."""
    sys.path.insert(0, str(REF))
    for name in [m for m in sys.modules if m == "braid" or m.startswith("braid.")]:
        del sys.modules[name]
    rq = importlib.import_module("braid.model.quant")
    mlp = importlib.import_module("braid.model.mlp")
    yield rq, mlp
    for name in [m for m in sys.modules if m == "braid" or m.startswith("braid.")]:
        del sys.modules[name]
    sys.path.remove(str(REF))


def test_reference_mlp_runs_on_these_kernels(Q, ref_modules):
    from braid_b200.integrate import install_into
    rq, mlp_mod = ref_modules
    assert rq.fused_state() == "not tried"            # stock reference: torch spelling arm
    cfg = SimpleNamespace(hidden_act="silu")
    H, I, M = 1024, 2048, 16
    w = {"mlp.gate_proj": randn_cpu((I, H), seed=1, scale=0.05).cuda(),
         "mlp.up_proj": randn_cpu((I, H), seed=2, scale=0.05).cuda(),
         "mlp.down_proj": randn_cpu((H, I), seed=3, scale=0.05).cuda()}
    x = randn_cpu((2, M // 2, H), seed=4).cuda()

    stock = mlp_mod.MLP(cfg, w, quant=True)
    assert isinstance(stock.gate_proj, rq.FP8Weight)
    y_stock = stock(x)                                 # torch spelling + torch._scaled_mm
    y_bf16 = mlp_mod.MLP(cfg, w, quant=False)(x)

    done = install_into(rq)
    assert "braid.model.mlp.fp8_matmul" in done and rq.fp8_matmul is Q.fp8_matmul
    ours = mlp_mod.MLP(cfg, w, quant=True)             # the reference's class, these kernels
    assert isinstance(ours.gate_proj, Q.FP8Weight)
    # same weights: the quantized payloads and scales are bit-identical to the reference's
    for a, b in ((stock.gate_proj, ours.gate_proj), (stock.down_proj, ours.down_proj)):
        assert torch.equal(a.data.view(torch.uint8), b.data.view(torch.uint8))
        assert torch.equal(a.scale, b.scale)
    y_ours = ours(x)
    assert y_ours.shape == y_stock.shape and y_ours.dtype is y_stock.dtype
    assert max_rel(y_ours, y_stock) <= 1e-2
    assert F.cosine_similarity(y_ours.float().flatten(), y_bf16.float().flatten(), dim=0) > 0.99
    # and the reference's forward, spelled with separate calls, equals the fused 4-launch form
    assert torch.equal(y_ours, Q.mlp_forward(x, ours.gate_proj, ours.up_proj, ours.down_proj))
    assert Q.device_status() == 0


def test_reference_operator_functions_after_install(Q, ref_modules):
    from braid_b200.integrate import install_into
    rq, _ = ref_modules
    x = randn_cpu((4, 256), seed=5).cuda()
    a, b = randn_cpu((512, 256), seed=6, scale=0.02).cuda(), randn_cpu((32, 256), seed=7, scale=0.02).cuda()
    stock_q, stock_s = rq.quantize_act(x)
    stock_y = rq.fp8_linear(x, rq.quantize_weight(a))
    install_into(rq)
    q, s = rq.quantize_act(x)
    assert torch.equal(s, stock_s) and torch.equal(q.view(torch.uint8), stock_q.view(torch.uint8))
    fa = rq.quantize_weight(a)
    assert max_rel(rq.fp8_linear(x, fa), stock_y) <= 1e-2
    ya, yb = rq.project(x, fa, b)
    assert torch.equal(ya, rq.fp8_linear(x, fa)) and torch.equal(yb, F.linear(x, b))
    assert rq.fused_state() == "active" and rq.parse_groups("all") == frozenset(rq.GROUPS)
