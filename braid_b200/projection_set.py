"""The projection set of one decode (or prefill) step of a Qwen3.5-class hybrid stack.

This is the call pattern of the reference's sublayers, reduced to the projections:

  GDN layer        project(x, qkv, z, a, b)            braid/model/gdn.py:254-255
                   linear(core, out_proj)              braid/model/gdn.py:387
  attention layer  project(x, q, k, v)                 braid/model/attention.py:173
                   linear(o * sigmoid(gate), o_proj)   braid/model/attention.py:215-216
  every layer      MLP.forward quantized branch        braid/model/mlp.py:44-49

The mixers between the projections (scan, conv, attention, norms, residuals) are
not part of this path, so their outputs are stood in for by fixed N(0,1)
buffers (`core`, `o`), and every layer reads the same step input `x`.  The
attention output gate IS real data flow: it is the strided per-head half of the
q projection's output.

Two arms build the same step from the same weights:

  "b200"     this package's kernels (fused prologues, grouped GEMM launches)
  "library"  the reference's spelling on the same GPU: torch-spelling quantizer,
             `torch._scaled_mm` per weight, SiLU*mul and sigmoid-gate as bf16
             torch kernels (braid/model/quant.py:228-241) — the on-box baseline.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import quant as Q


@dataclass(frozen=True)
class StackShapes:
    """Qwen3.5-9B-class widths (braid/model/loader.py:307-328 is the shape table)."""

    hidden: int = 4096
    intermediate: int = 12288
    gdn_qkv: int = 8192          # q/k 2 x (16 x 128) + v 32 x 128
    gdn_z: int = 4096
    gdn_gate: int = 32           # in_proj_a / in_proj_b rows, kept bf16 by design
    gdn_inner: int = 4096
    attn_heads: int = 16
    attn_head_dim: int = 256
    attn_kv: int = 1024          # 4 KV heads x 256
    n_layers: int = 32
    attn_every: int = 4          # layers 3, 7, ... are full attention

    @property
    def attn_q(self) -> int:     # output-gated: [q | gate] per head
        return 2 * self.attn_heads * self.attn_head_dim

    def is_attention(self, layer: int) -> bool:
        return layer % self.attn_every == self.attn_every - 1

    def layer_weight_shapes(self, layer: int) -> dict[str, tuple[int, int]]:
        H, I = self.hidden, self.intermediate
        if self.is_attention(layer):
            mix = {"q": (self.attn_q, H), "k": (self.attn_kv, H), "v": (self.attn_kv, H),
                   "o": (H, self.attn_heads * self.attn_head_dim)}
        else:
            mix = {"qkv": (self.gdn_qkv, H), "z": (self.gdn_z, H), "a": (self.gdn_gate, H),
                   "b": (self.gdn_gate, H), "out": (H, self.gdn_inner)}
        mix.update({"gate": (I, H), "up": (I, H), "down": (H, I)})
        return mix

    def fp8_weight_bytes(self) -> int:
        total = 0
        for layer in range(self.n_layers):
            for name, (n, k) in self.layer_weight_shapes(layer).items():
                if name not in ("a", "b"):
                    total += n * k
        return total

    def step_flops(self, rows: int) -> int:
        return 2 * rows * self.fp8_weight_bytes()


class ProjectionSet:
    """Random-init weights of the whole stack plus the step that runs every projection once."""

    def __init__(self, shapes: StackShapes, rows: int, device: torch.device, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, layers: int | None = None):
        self.shapes, self.rows, self.device, self.dtype = shapes, rows, device, dtype
        self.n_layers = shapes.n_layers if layers is None else layers
        g = torch.Generator(device=device).manual_seed(seed)
        self.layers: list[dict] = []
        for layer in range(self.n_layers):
            ws = {}
            for name, (n, k) in shapes.layer_weight_shapes(layer).items():
                w = (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
                # the reference never quantizes the GDN gates a/b (braid/model/gdn.py:73-81)
                ws[name] = w if name in ("a", "b") else Q.quantize_weight(w)
                del w
            self.layers.append(ws)
        # stand-ins for what the mixers would hand to the output projections
        self.core = torch.randn(rows, shapes.gdn_inner, generator=g, device=device).to(dtype)
        self.o = torch.randn(rows, shapes.attn_heads * shapes.attn_head_dim, generator=g,
                             device=device).to(dtype)
        self.x = torch.randn(rows, shapes.hidden, generator=g, device=device).to(dtype)

    # -- counts ---------------------------------------------------------------------------
    def fp8_weight_bytes(self) -> int:
        return sum(w.data.numel() for ws in self.layers for w in ws.values()
                   if isinstance(w, Q.FP8Weight))

    def gemm_algorithmic_bytes(self) -> int:
        """N*K weight bytes + M*K activation codes + 2*M*N outputs, summed over the FP8 GEMMs
        (one activation read per LAUNCH: grouped weights share it)."""
        M, total = self.rows, 0
        for ws in self.layers:
            groups = ([("qkv", "z"), ("out",)] if "qkv" in ws else [("q", "k", "v"), ("o",)])
            groups += [("gate", "up"), ("down",)]
            for grp in groups:
                k = ws[grp[0]].shape[1]
                total += M * k + sum(ws[n].shape[0] * k + 2 * M * ws[n].shape[0] for n in grp)
        return total

    # dram__bytes_read.sum + dram__bytes_write.sum of one gemm_stream_kernel launch at 128 rows,
    # measured with ncu on a 4-layer stack (weights larger than L2), per launch shape: every
    # weight byte and the activation codes cross HBM once; the outputs are still in L2 when the
    # kernel ends, so they do not show.  Other row counts use the mean measured/algorithmic ratio.
    MEASURED_TRAFFIC_M128 = {
        ("qkv", "z"): 50.98e6, ("out",): 17.39e6, ("gate", "up"): 101.45e6, ("down",): 51.99e6,
        ("q", "k", "v"): 42.57e6,
    }

    def gemm_measured_traffic_bytes(self) -> dict:
        """DRAM bytes of the step's FP8 GEMM launches from the per-shape ncu measurements."""
        M, total, covered, alg_cov = self.rows, 0.0, 0, 0.0
        per_shape = {}
        for ws in self.layers:
            groups = ([("qkv", "z"), ("out",)] if "qkv" in ws else [("q", "k", "v"), ("o",)])
            groups += [("gate", "up"), ("down",)]
            for grp in groups:
                k = ws[grp[0]].shape[1]
                alg = M * k + sum(ws[n].shape[0] * k + 2 * M * ws[n].shape[0] for n in grp)
                key = ("out",) if grp == ("o",) else grp
                if M == 128 and key in self.MEASURED_TRAFFIC_M128:
                    per_shape[grp] = (self.MEASURED_TRAFFIC_M128[key], alg)
        ratios = [t / a for t, a in per_shape.values()] or [1.02]
        mean_ratio = sum(ratios) / len(ratios)
        for ws in self.layers:
            groups = ([("qkv", "z"), ("out",)] if "qkv" in ws else [("q", "k", "v"), ("o",)])
            groups += [("gate", "up"), ("down",)]
            for grp in groups:
                k = ws[grp[0]].shape[1]
                alg = M * k + sum(ws[n].shape[0] * k + 2 * M * ws[n].shape[0] for n in grp)
                if grp in per_shape:
                    total += per_shape[grp][0]
                    covered += 1
                else:
                    total += mean_ratio * alg
        n = 4 * len(self.layers)
        return {"bytes": total,
                "source": f"ncu dram__bytes_read+write per launch shape at 128 rows on a 4-layer stack "
                          f"({covered} of {n} launches of this step have a measured shape; the others use "
                          f"the mean measured/algorithmic ratio {mean_ratio:.3f})"}

    def quant_algorithmic_bytes(self) -> int:
        """3 bytes per element for the plain quantizer (bf16 in, code out), 5 for the two-input
        prologues."""
        M, s, total = self.rows, self.shapes, 0
        for ws in self.layers:
            total += 3 * M * s.hidden                      # mixer input
            total += (3 * M * s.gdn_inner) if "qkv" in ws else (5 * M * s.hidden)
            total += 3 * M * s.hidden                      # MLP input
            total += 5 * M * s.intermediate                # SiLU*mul prologue
        return total

    # -- the step, this package's kernels ------------------------------------------------------
    def step_b200(self, x: torch.Tensor, bf16_gates: bool = True) -> torch.Tensor:
        """`bf16_gates=False` leaves out the two tiny bf16 projections (a, b) the reference keeps
        in bf16: the step then contains this package's kernels only."""
        s = self.shapes
        y = x
        for ws in self.layers:
            if "qkv" in ws and not bf16_gates:
                Q.project(x, ws["qkv"], ws["z"])
                y = Q.linear(self.core, ws["out"])
            elif "qkv" in ws:
                qkv, z, a, b = Q.project(x, ws["qkv"], ws["z"], ws["a"], ws["b"])
                y = Q.linear(self.core, ws["out"])
            else:
                qg, k, v = Q.project(x, ws["q"], ws["k"], ws["v"])
                gate = qg.view(self.rows, s.attn_heads, 2 * s.attn_head_dim)[..., s.attn_head_dim:]
                y = Q.gated_output_projection(self.o, gate, ws["o"])
            y = Q.mlp_forward(x, ws["gate"], ws["up"], ws["down"])
        return y

    # -- the step, the reference's spelling on the same GPU ---------------------------------
    @staticmethod
    def _lib_quant(x):
        scale = (x.detach().float().abs().amax() / Q.FP8_MAX).clamp(min=Q.EPS).reshape(1, 1)
        return (x.float() / scale).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(Q.FP8), scale

    @staticmethod
    def _lib_mm(xq, sx, w, dtype):
        return torch._scaled_mm(xq, w.data.t(), scale_a=sx, scale_b=w.scale, out_dtype=dtype)

    def _lib_project(self, x, *weights):
        xq, sx = self._quantizer(x)
        return [self._lib_mm(xq, sx, w, x.dtype) if isinstance(w, Q.FP8Weight) else F.linear(x, w)
                for w in weights]

    def _lib_linear(self, x, w):
        xq, sx = self._quantizer(x)
        return self._lib_mm(xq, sx, w, x.dtype)

    def step_library(self, x: torch.Tensor, quantizer=None) -> torch.Tensor:
        """`quantizer`: `x -> (codes, scale)`; default the reference's torch spelling (nine
        kernels); the benchmark also passes the reference's own fused two-launch kernel."""
        s = self.shapes
        y = x
        self._quantizer = quantizer or self._lib_quant
        for ws in self.layers:
            if "qkv" in ws:
                self._lib_project(x, ws["qkv"], ws["z"], ws["a"], ws["b"])
                y = self._lib_linear(self.core, ws["out"])
            else:
                qg, k, v = self._lib_project(x, ws["q"], ws["k"], ws["v"])
                _, gate = qg.view(self.rows, s.attn_heads, 2 * s.attn_head_dim).chunk(2, dim=-1)
                gate = gate.reshape(self.rows, s.attn_heads * s.attn_head_dim)
                y = self._lib_linear(self.o * torch.sigmoid(gate), ws["o"])
            xq, sx = self._quantizer(x)
            g_ = self._lib_mm(xq, sx, ws["gate"], x.dtype)
            u_ = self._lib_mm(xq, sx, ws["up"], x.dtype)
            y = self._lib_linear(F.silu(g_) * u_, ws["down"])
        return y

    # -- only the FP8 GEMM launches of the step (for the roofline of the dominant kernel) -----
    def gemms_only_b200(self, xq, sx, coreq, oq, hq, out_bufs) -> None:
        for ws, bufs in zip(self.layers, out_bufs):
            if "qkv" in ws:
                Q.fp8_matmul_grouped(xq, sx, (ws["qkv"], ws["z"]), self.dtype, out=bufs["in"])
                Q.fp8_matmul_grouped(coreq, sx, (ws["out"],), self.dtype, out=bufs["out"])
            else:
                Q.fp8_matmul_grouped(xq, sx, (ws["q"], ws["k"], ws["v"]), self.dtype, out=bufs["in"])
                Q.fp8_matmul_grouped(oq, sx, (ws["o"],), self.dtype, out=bufs["out"])
            Q.fp8_matmul_grouped(xq, sx, (ws["gate"], ws["up"]), self.dtype, out=bufs["gu"])
            Q.fp8_matmul_grouped(hq, sx, (ws["down"],), self.dtype, out=bufs["down"])

    def gemm_out_buffers(self):
        M, dev, dt = self.rows, self.device, self.dtype
        mk = lambda n: torch.empty((M, n), dtype=dt, device=dev)  # noqa: E731
        shared = {}   # one set of output buffers reused by every layer
        def get(key, ns):
            if key not in shared:
                shared[key] = tuple(mk(n) for n in ns)
            return shared[key]
        bufs = []
        for ws in self.layers:
            first = ("qkv", "z") if "qkv" in ws else ("q", "k", "v")
            last = "out" if "qkv" in ws else "o"
            bufs.append({"in": get(first, [ws[n].shape[0] for n in first]),
                         "out": get(last, [ws[last].shape[0]]),
                         "gu": get("gu", [ws["gate"].shape[0], ws["up"].shape[0]]),
                         "down": get("down", [ws["down"].shape[0]])})
        return bufs
