#!/usr/bin/env python
"""Benchmark of the FP8 W8A8 projection path on B200.

Default workload (`config.workload = "decode_step_projection_set"`): the full projection set of
one decode step of a 32-layer Qwen3.5-9B-class hybrid (24 Gated-DeltaNet + 8 attention layers,
MLP in every layer) at batch 128 — 128 activation quantizations (32 of them done in the
epilogue of the paired gate/up GEMM) and 128 FP8 GEMM launches covering 200 weights (6.9 GB of
e4m3), captured once in a CUDA graph and replayed.
One step = one replay.  metric = projection-set tokens per second = rows x steps / time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows 128] [--impl b200|reference]
    python bench.py --sweep            # per-projection GB/s and TFLOP/s tables (JSON lines)

N > 1 is launched by torchrun, one rank per GPU: data-parallel replicas, weights replicated, no
collective on the data path (`"scaling": "weak"`); rank 0 also times the column-parallel MLP
(N-split weights + NCCL all-gather) and reports it under `column_parallel`.

`--impl reference` times the reference's CPU spelling of the same path (oracle/cpu_spelling.py)
on all host cores; every step is the same bounded sample: one layer of each kind in full, scaled
by the layer counts.  It also times torch's own CPU `_scaled_mm` on a slice and extrapolates.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_step_projection_set_tokens_per_s"


# ------------------------------------------------------------------------------------------
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v.strip()]
        try:
            return int(ids[local])
        except (ValueError, IndexError):
            return local
    return local


def timed_replays(fn, steps: int, warmup: int, dist=None, sampler_index=None):
    """warmup untimed, then `steps` timed calls between barrier+synchronize, CUDA events on the
    launching stream; returns (ms_total_max_over_ranks, clocks)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if sampler:
        sampler.__enter__()
        time.sleep(0.15)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    # keep the GPU busy a little longer if the region was too short to be sampled
    clocks = None
    if sampler:
        if ms < 400:
            t_end = time.time() + 0.5
            while time.time() < t_end:
                fn()
            torch.cuda.synchronize()
        sampler.__exit__()
        clocks = sampler.summary()
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, clocks


def capture(fn, warm: int = 3):
    """Side-stream warm-up then capture, as braid/model/graph.py:101-134 does."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fn()
    return graph, out


# ------------------------------------------------------------------------------------------
def workload_config(rows: int, layers: int, world: int) -> dict:
    """The `config` both arms print: what one step is."""
    from braid_b200.projection_set import StackShapes
    s = StackShapes()
    n_att = sum(1 for i in range(layers) if s.is_attention(i))
    return {"workload": "decode_step_projection_set", "rows": rows, "layers": layers,
            "hidden": s.hidden, "intermediate": s.intermediate, "gdn_layers": layers - n_att,
            "attn_layers": n_att, "fp8_weight_bytes": s.fp8_weight_bytes() * layers // s.n_layers,
            "parallelism": f"dp{world}",
            "l2": "inputs larger than L2 (6.9 GB of weights streamed per step)",
            "timing": "b200 arm: CUDA-graph replay, CUDA events, max over ranks; reference arm: "
                      "host wall clock around the sampled step",
            "ab_gates": "kept in bf16 as in the reference; multiplied unquantized"}


class CpuSample:
    """The reference's CPU spelling on a bounded sample of one step: one GDN, one attention and
    one MLP layer of projections, each timed in full and scaled by the stack's layer counts."""

    def __init__(self, rows: int, layers: int = 32):
        from braid_b200.projection_set import StackShapes
        from oracle import cpu_spelling as C
        torch.set_num_threads(os.cpu_count() or 1)    # torchrun sets OMP_NUM_THREADS=1
        self.C, self.rows, s = C, rows, StackShapes()
        self.s = s
        g = torch.Generator().manual_seed(0)

        def weight(n, k):
            return C.quantize((torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16))

        H, I = s.hidden, s.intermediate
        self.x = torch.randn(rows, H, generator=g).to(torch.bfloat16)
        self.core = torch.randn(rows, s.gdn_inner, generator=g).to(torch.bfloat16)
        self.gdn = [weight(s.gdn_qkv, H), weight(s.gdn_z, H), weight(H, s.gdn_inner)]
        self.att = [weight(s.attn_q, H), weight(s.attn_kv, H), weight(s.attn_kv, H), weight(H, H)]
        self.mlp = [weight(I, H), weight(I, H), weight(H, I)]
        self.n_att = sum(1 for i in range(layers) if s.is_attention(i))
        self.n_gdn, self.n_mlp = layers - self.n_att, layers

    def step(self) -> tuple[float, float]:
        """One sampled step: (seconds the sample took, seconds the whole step would take)."""
        C, s, rows = self.C, self.s, self.rows
        t0 = time.perf_counter()
        C.project(self.x, self.gdn[0], self.gdn[1])
        C.linear(self.core, *self.gdn[2])
        t1 = time.perf_counter()
        qg, _, _ = C.project(self.x, self.att[0], self.att[1], self.att[2])
        gate = qg.view(rows, s.attn_heads, 2 * s.attn_head_dim)[..., s.attn_head_dim:]
        C.linear(self.core * torch.sigmoid(gate.reshape(rows, s.hidden)), *self.att[3])
        t2 = time.perf_counter()
        C.mlp(self.x, self.mlp[0], self.mlp[1], self.mlp[2])
        t3 = time.perf_counter()
        return t3 - t0, self.n_gdn * (t1 - t0) + self.n_att * (t2 - t1) + self.n_mlp * (t3 - t2)

    def scaled_mm_extrapolated(self, slice_rows: int = 64) -> dict:
        """torch's own CPU `_scaled_mm` (the literal call of braid/model/quant.py:240-241; a scalar
        loop on CPU) on the first `slice_rows` rows of the gate weight, extrapolated by bytes to
        the FP8 weights of one step."""
        C = self.C
        xq, sx = C.quantize(self.x)
        wq, sw = self.mlp[0]
        sec = C.scaled_mm_slice_seconds(xq, sx, wq, sw, rows=slice_rows)
        total = self.s.fp8_weight_bytes() * self.n_mlp // self.s.n_layers
        step_s = sec / (slice_rows * wq.shape[1]) * total
        return {"slice_rows": slice_rows, "slice_seconds": sec, "step_seconds_extrapolated": step_s,
                "value": self.rows / step_s, "unit": "tok/s",
                "what": "torch._scaled_mm on CPU, one N-slice timed, scaled by weight bytes"}

    def describe(self, sample_s: float, step_s: float) -> str:
        return (f"1 GDN + 1 attention + 1 MLP layer of projections at {self.rows} rows timed in full "
                f"with the reference's CPU spelling (torch quantizer + fp32 dequant-matmul on "
                f"{torch.get_num_threads()} threads) = {sample_s * 1e3:.0f} ms per sampled step, scaled "
                f"by {self.n_gdn}/{self.n_att}/{self.n_mlp} layers to {step_s * 1e3:.0f} ms per step")


def cpu_baseline(rows: int, layers: int = 32, steps: int = 3, warmup: int = 1, sample=None,
                 with_scaled_mm: bool = False):
    sample = sample or CpuSample(rows, layers)
    for _ in range(warmup):
        sample.step()
    got = [sample.step() for _ in range(max(1, steps))]
    sample_s = statistics.mean(t[0] for t in got)
    step_s = statistics.mean(t[1] for t in got)
    out = {"value": rows / step_s, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
           "sample": sample.describe(sample_s, step_s), "host_cpus": os.cpu_count(),
           "timed_steps": len(got), "sample_seconds_per_step": sample_s,
           "step_seconds_extrapolated": step_s}
    if with_scaled_mm:
        try:
            out["reference_scaled_mm"] = sample.scaled_mm_extrapolated()
        except Exception as e:  # noqa: BLE001
            out["reference_scaled_mm"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    best = cpu_baseline(args.rows, args.layers, steps=args.steps, warmup=args.warmup,
                        with_scaled_mm=True)
    line = {
        "impl": "reference", "metric": METRIC, "value": best["value"], "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": best["step_seconds_extrapolated"] * 1e3,
        "sample_ms_per_step": best["sample_seconds_per_step"] * 1e3,
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f8e4m3xf8e4m3->f32",
        "data": "synthetic",
        "config": workload_config(args.rows, args.layers, world),
        "cpu_baseline": best,
        "e2e": {"value": best["value"], "unit": "tok/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
def run_engine_compare(args):
    """Whole-engine decode step of the reference (an install under baseline/_ref), stock and with
    this package installed into it.  Not the headline metric: the mixers, norms and cache are the
    reference's own code in every arm; only the FP8 projection path is swapped."""
    root = Path(__file__).resolve().parent
    ref = root / "baseline" / "_ref"
    if not (ref / "braid" / "model" / "engine.py").exists():
        print(json.dumps({"metric": "engine_decode_tokens_per_s",
                          "unavailable": "no install of the reference under baseline/_ref"}))
        return
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(root / "baseline"))
    import ref_kernels
    from braid_b200 import engine_dropin
    use_kernels = ref_kernels.available()
    if use_kernels:
        ref_kernels.attach()
    torch.cuda.set_device(0)
    res = engine_dropin.compare_arms(torch.device("cuda", 0), layers=args.layers, vocab=args.vocab,
                                     batch=args.rows, steps=args.steps, prompt_len=args.prompt_len,
                                     use_kernels=use_kernels)
    res = {"metric": "engine_decode_tokens_per_s", "unit": "tok/s", "n_gpus": 1, **res}
    print(json.dumps(res), flush=True)


def reference_fused_quantizer():
    """The reference's shipped fused quantizer (braid/kernels/csrc/quant_act.cu:140-176), from the
    extension baseline/ref_kernels.py builds for sm_100a out of the reference checkout.  Returns
    the callable `x -> (q, scale)` or a one-line reason why it is not there."""
    try:
        sys.path.insert(0, str(ROOT / "baseline"))
        import ref_kernels
        if not ref_kernels.prebuilt_path().exists():
            return "no prebuilt reference extension under baseline/_ref/_prebuilt"
        import importlib.util
        name = ref_kernels.NAME
        if name in sys.modules:
            mod = sys.modules[name]
        else:
            spec = importlib.util.spec_from_file_location(name, ref_kernels.prebuilt_path())
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.modules[name] = mod
        fn = mod.quantize_act

        def quantizer(x):
            q, scale = fn(x)
            return q, scale
        return quantizer
    except Exception as e:  # noqa: BLE001
        return f"{type(e).__name__}: {str(e)[:140]}"


def projection_tables(dev, peaks):
    """BASELINE's per-projection half of the metric, in the same run: decode-regime GB/s as a
    fraction of the HBM copy peak over the config-2 / config-3 launch shapes at M = 1, 16, 128,
    and prefill-regime TFLOP/s at config 4's packed row count, each beside the library GEMM
    (`torch._scaled_mm`) on the same shapes (method: braid_b200/sweep.py)."""
    from braid_b200 import sweep
    rows = []
    for name in ("mlp.gate_up", "mlp.down", "gdn.in_proj_qkv_z", "gdn.out_proj", "attn.qkv",
                 "attn.k_proj"):
        ns, k = sweep.PROJECTIONS[name]
        for m in (1, 16, 128):
            r = sweep.gemm_row(name, ns, k, m, dev, peaks, reps=9)
            rows.append({"proj": name, "M": m, "us": r["us"], "gbs": r["gbs"], "frac_hbm": r["frac_hbm"],
                         "vs_scaled_mm": r.get("speedup_vs_lib")})
    fr = sorted(r["frac_hbm"] for r in rows)
    ratio = sorted(r["vs_scaled_mm"] for r in rows if r["vs_scaled_mm"])
    per_projection = {
        "rows": rows, "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
        "frac_hbm": {"min": fr[0], "median": statistics.median(fr), "max": fr[-1]},
        "frac_hbm_M128": {r["proj"]: r["frac_hbm"] for r in rows if r["M"] == 128},
        "vs_scaled_mm": {"min": ratio[0], "median": statistics.median(ratio), "max": ratio[-1]} if ratio else None,
        "note": "attn.o_proj has out_proj's shape; frac = algorithmic bytes (N*K + M*K + 2*M*N) / time / peak"}
    try:
        per_projection["lm_head"] = sweep.lm_head_rows(dev, peaks)
    except Exception as e:  # noqa: BLE001
        torch.cuda.synchronize()
        per_projection["lm_head"] = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}
    g = torch.Generator().manual_seed(4)
    m4 = int(torch.randint(64, 1025, (16,), generator=g).sum().item())
    peak8 = sweep.fp8_library_peak(dev, seconds=1.0)
    prows = []
    for name in ("mlp.gate_up", "mlp.down", "gdn.in_proj_qkv_z", "gdn.out_proj"):
        ns, k = sweep.PROJECTIONS[name]
        for m in (m4, 8192):
            r = sweep.gemm_row(name, ns, k, m, dev, peaks, inner=4, reps=7)
            prows.append({"proj": name, "M": m, "us": r["us"], "tflops": r["tflops"],
                          "frac_fp8_measured_burst": r["tflops"] / peak8["fp8_tflops_burst"],
                          "frac_fp8_nominal_4500": r["tflops"] / 4500.0,
                          "vs_scaled_mm": r.get("speedup_vs_lib"), "kernel": r["launch"]["kernel"]})
    at = lambda m: [r for r in prows if r["M"] == m]  # noqa: E731
    prefill = {"workload": "config 4: 16 packed sequences, lengths ~U[64,1024] (seed 4), and the "
                           "round 8192 rows beside it", "M": m4,
               "rows": prows, "fp8_peak_measured": peak8,
               "fp8_peak_how": "torch._scaled_mm 8192^3, best of 10 (burst) / back to back 1 s (sustained)",
               "min_vs_scaled_mm": {str(m): min((r["vs_scaled_mm"] or 0.0) for r in at(m)) for m in (m4, 8192)},
               "min_frac_fp8_measured_burst": {str(m): min(r["frac_fp8_measured_burst"] for r in at(m))
                                               for m in (m4, 8192)}}
    return per_projection, prefill


def column_parallel_block(dist, rows_list, steps, warmup):
    """gate_up [2 x 12288, 4096] and down [4096, 12288] N-split over the ranks, bf16 all-gather of
    the h shards and of the output shards (NCCL over NVLink)."""
    from braid_b200 import quant as Q
    from braid_b200.parallel import ColumnParallelMLP
    out = {}
    for rows in rows_list:
        mlp = ColumnParallelMLP.random_init(4096, 12288, torch.device("cuda"), dist.group.WORLD, seed=1)
        gx = torch.Generator(device="cuda").manual_seed(7)       # the same activation on every rank
        x = torch.randn(rows, 4096, generator=gx, device="cuda").to(torch.bfloat16)
        fn = lambda: mlp.forward(x)  # noqa: E731
        # one CUDA graph per rank holding the kernels AND the two NCCL all-gathers, replayed like
        # the decode step; eager launches if the collective cannot be captured here
        how = "graph replay"
        try:
            graph, _ = capture(fn)
            call = graph.replay
        except Exception:  # noqa: BLE001
            torch.cuda.synchronize()
            how, call = "eager launches", fn
        ms, _ = timed_replays(call, steps, warmup, dist=dist)
        flops = 2 * rows * 3 * 4096 * 12288
        entry = {"ms_per_call": ms / steps, "tflops": flops / (ms / steps * 1e-3) / 1e12,
                 "all_gather_bytes": mlp.gather_bytes(rows), "timing": how}
        if how == "graph replay":
            del graph
        y_nccl = fn().clone()
        del mlp
        # the same sharded MLP with the all-gathers folded into the GEMM epilogues (peer-mapped
        # buffers over CUDA IPC, per-rank arrival counters, no collective)
        if True:   # decode sizes and prefill sizes alike
            try:
                from braid_b200.parallel import FusedColumnParallelMLP
                fmlp = FusedColumnParallelMLP.random_init(4096, 12288, torch.device("cuda"),
                                                          dist.group.WORLD, seed=1,
                                                          rows_max=max(256, rows))
                fmlp.connect()
                y_fused = fmlp.forward(x).clone()
                torch.cuda.synchronize()
                dist.barrier()
                gf, _ = capture(lambda: fmlp.forward(x))
                msf, _ = timed_replays(gf.replay, steps, warmup, dist=dist)
                entry["fused"] = {"ms_per_call": msf / steps,
                                  "equals_nccl_form": bool(torch.equal(y_fused, y_nccl)),
                                  "wait_status": int(fmlp.buffers.status.item()),
                                  "launches_per_call": 4 if rows <= 256 else 8,
                                  "what": ("GEMM epilogues store into every rank's gathered buffer "
                                           "through peer pointers; arrival waits in the consumer / a "
                                           "one-thread kernel; no NCCL") if rows <= 256 else
                                          ("h exchanged as e4m3 codes: shard scales as 4-byte words, "
                                           "their maximum, an elementwise cast-and-store kernel into "
                                           "every rank's buffer; y from the down GEMM's epilogue; peer "
                                           "pointers, arrival counters, bounded waits; no NCCL")}
                del gf
                fmlp.close()
                del fmlp
            except Exception as e:  # noqa: BLE001
                entry["fused"] = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}
        # the same MLP, unsharded, on one GPU of the same box (every rank runs it; rank 0 reports)
        g = torch.Generator(device="cuda").manual_seed(1)
        mk = lambda n, k: Q.quantize_weight(  # noqa: E731
            (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
        wg, wu, wd = mk(12288, 4096), mk(12288, 4096), mk(4096, 12288)
        g1, _ = capture(lambda: Q.mlp_forward(x, wg, wu, wd))
        ms1, _ = timed_replays(g1.replay, steps, warmup, dist=dist)
        del g1
        entry["single_gpu_ms_per_call"] = ms1 / steps
        entry["speedup_vs_single_gpu"] = ms1 / ms
        # prefill sizes: the sharded result equals the unsharded one bit for bit (same codes, same
        # scale, and the prefill GEMM sums K in one order whatever rows of the weight it is given)
        if rows > 256:
            entry["equals_single_gpu"] = bool(torch.equal(y_nccl, Q.mlp_forward(x, wg, wu, wd)))
        entry["best"] = {"form": "nccl", "ms_per_call": ms / steps, "speedup_vs_single_gpu": ms1 / ms}
        if "fused" in entry and "ms_per_call" in entry["fused"]:
            entry["fused"]["speedup_vs_single_gpu"] = (ms1 / steps) / entry["fused"]["ms_per_call"]
            entry["fused"]["speedup_vs_nccl_form"] = (ms / steps) / entry["fused"]["ms_per_call"]
            if entry["fused"]["ms_per_call"] < ms / steps and entry["fused"].get("equals_nccl_form"):
                entry["best"] = {"form": "fused (peer memory, no collective)",
                                 "ms_per_call": entry["fused"]["ms_per_call"],
                                 "speedup_vs_single_gpu": entry["fused"]["speedup_vs_single_gpu"]}
        out[f"M{rows}"] = entry
        del wg, wu, wd
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--only", default=None, help="with --sweep: one projection name, at --rows")
    ap.add_argument("--no-library-arm", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-tables", action="store_true",
                    help="skip the per-projection decode table and the prefill (config 4) record")
    ap.add_argument("--engine", action="store_true",
                    help="the reference's whole graphed decode step (installed under baseline/_ref) "
                         "stock vs on these kernels; one GPU, its own JSON line")
    ap.add_argument("--vocab", type=int, default=248320)
    ap.add_argument("--prompt-len", type=int, default=128)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    if args.sweep:
        from braid_b200 import sweep
        sweep.main(args)
        return

    if args.engine:
        run_engine_compare(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        # NCCL's version banner goes to stdout and would precede the one JSON line
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        import torch.distributed as dist_mod
        # ... and at any level above NONE it still prints it when the communicator is created:
        # point fd 1 at stderr until that has happened, so stdout carries the JSON line only
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist_mod.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
        dist = dist_mod

    from braid_b200 import quant as Q
    from braid_b200.projection_set import ProjectionSet, StackShapes
    Q.warm_fused(True)
    for kv in filter(None, os.environ.get("BQ_OPTIONS", "").split(",")):   # tuning experiments
        k, v = kv.split("=")
        Q.set_option(k, int(v))
    dev = torch.device("cuda", local)
    shapes = StackShapes()
    ps = ProjectionSet(shapes, args.rows, dev, seed=rank, layers=args.layers)
    static_x = ps.x.clone()

    # ---- main timed region: graph replays, inputs resident in HBM -------------------------
    n0 = Q.launch_count()
    graph, static_y = capture(lambda: ps.step_b200(static_x))
    launches_per_step = (Q.launch_count() - n0) // 4      # 3 warm-up passes + the capture
    ms, clocks = timed_replays(graph.replay, args.steps, args.warmup, dist=dist,
                               sampler_index=physical_gpu_index(local) if rank == 0 else None)
    ms_per_step = ms / args.steps
    value = world * args.rows / (ms_per_step * 1e-3)

    # ---- end to end: host buffers in, host result out, every step -------------------------
    x_host = ps.x.cpu().pin_memory()
    y_host = torch.empty(static_y.shape, dtype=static_y.dtype).pin_memory()

    def e2e_step():
        static_x.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(static_y, non_blocking=True)

    ms_e2e, _ = timed_replays(e2e_step, args.steps, args.warmup, dist=dist)
    e2e_value = world * args.rows / (ms_e2e / args.steps * 1e-3)
    h2d = x_host.numel() * x_host.element_size()
    d2h = y_host.numel() * y_host.element_size()

    # ---- dominant kernel alone: the step's FP8 GEMM launches, same shapes and order ---------
    # (gate|up in its plain grouped form: the paired form the step uses adds the SiLU*mul and
    # quantization epilogue, which is not GEMM time)
    xq, sx = Q.quantize_act(static_x)
    coreq, _ = Q.quantize_act(ps.core)
    oq, _ = Q.quantize_act(ps.o)
    hq, _ = Q.quantize_act(torch.randn(args.rows, shapes.intermediate, device=dev).to(torch.bfloat16))
    bufs = ps.gemm_out_buffers()
    n1 = Q.launch_count()
    g_gemm, _ = capture(lambda: ps.gemms_only_b200(xq, sx, coreq, oq, hq, bufs))
    gemm_launches = (Q.launch_count() - n1) // 4
    ms_gemm, _ = timed_replays(g_gemm.replay, args.steps, args.warmup, dist=None)
    peaks = measured_peaks()
    gemm_bytes = ps.gemm_algorithmic_bytes()
    achieved = gemm_bytes / (ms_gemm / args.steps * 1e-3) / 1e9
    traffic = ps.gemm_measured_traffic_bytes()
    roofline = {"bound": "hbm", "kernel": "gemm_stream_kernel", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"],
                "traffic": traffic["bytes"] / max(1, gemm_launches),
                "traffic_source": traffic["source"],
                "launches_per_step": gemm_launches,
                "algorithmic_bytes_per_launch": gemm_bytes / max(1, gemm_launches),
                "avg_launch_us": ms_gemm / args.steps / max(1, gemm_launches) * 1e3}
    step_bytes = gemm_bytes + ps.quant_algorithmic_bytes()
    status = Q.device_status()

    # ---- the step with the 48 gate projections through F.linear (cuBLAS), as the reference runs them
    Q.set_dense_segments(False)
    g_fl, _ = capture(lambda: ps.step_b200(static_x))
    ms_fl, _ = timed_replays(g_fl.replay, args.steps, args.warmup, dist=None)
    del g_fl
    Q.set_dense_segments(True)

    # ---- the step without the 48 bf16 gate projections: this package's kernels only ----------
    n2 = Q.launch_count()
    g_fp8, _ = capture(lambda: ps.step_b200(static_x, bf16_gates=False))
    fp8_launches = (Q.launch_count() - n2) // 4
    ms_fp8, _ = timed_replays(g_fp8.replay, args.steps, args.warmup, dist=None)
    del g_fp8

    # ---- the same step built from the library GEMM, with each of the reference's quantizers ----
    library, library_fused = None, None
    if not args.no_library_arm and rank == 0:
        def library_arm(quantizer, what):
            try:
                g_lib, _ = capture(lambda: ps.step_library(static_x, quantizer))
                ms_lib, _ = timed_replays(g_lib.replay, args.steps, args.warmup, dist=None)
                del g_lib
                return {"value": args.rows / (ms_lib / args.steps * 1e-3), "unit": "tok/s",
                        "ms_per_step": ms_lib / args.steps, "what": what}
            except Exception as e:  # noqa: BLE001 - reported in the JSON line
                torch.cuda.synchronize()
                return {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

        library = library_arm(None, "same step from torch._scaled_mm + the reference's torch-spelling "
                                    "quantizer (nine kernels), one CUDA graph, same weights, one GPU")
        ref_quant = reference_fused_quantizer()
        if callable(ref_quant):
            library_fused = library_arm(ref_quant, "same step from torch._scaled_mm + the reference's own "
                                                   "fused two-launch quantizer (its CUDA source built for "
                                                   "sm_100a), one CUDA graph, same weights, one GPU")
        else:
            library_fused = {"unavailable": ref_quant}

    # ---- the other half of the metric: per-projection decode GB/s and prefill TFLOP/s ------------
    per_projection, prefill = None, None
    if rank == 0 and world == 1 and not args.no_tables:
        try:
            per_projection, prefill = projection_tables(dev, peaks)
        except Exception as e:  # noqa: BLE001
            torch.cuda.synchronize()
            per_projection = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    colpar = None
    if dist is not None:
        try:
            colpar = column_parallel_block(dist, [128, 4096], max(5, args.steps // 3), 3)
        except Exception as e:  # noqa: BLE001
            colpar = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu = cpu_baseline(args.rows, args.layers, steps=3, warmup=1)
        except Exception as e:  # noqa: BLE001
            cpu = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f8e4m3xf8e4m3->f32", "data": "synthetic",
            "config": workload_config(args.rows, args.layers, world),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "roofline": roofline,
            "step_roofline": {"algorithmic_bytes": step_bytes,
                              "achieved_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                              "frac_of_hbm": step_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              "tflops": shapes.step_flops(args.rows) * args.layers / shapes.n_layers
                              / (ms_per_step * 1e-3) / 1e12},
            "gates_through_f_linear": {"ms_per_step": ms_fl / args.steps,
                                       "what": "the same step with in_proj_a / in_proj_b through "
                                               "F.linear (two cuBLAS launches per GDN layer), the "
                                               "reference's arm; the headline runs them as 16-bit "
                                               "segments of the grouped launch"},
            "fp8_kernels_only": {"ms_per_step": ms_fp8 / args.steps,
                                 "launches_per_step": fp8_launches,
                                 "what": "the step without the 48 bf16 gate projections"},
            "cpu_baseline": cpu,
            "library_baseline": library,
            "library_baseline_fused_quantizer": library_fused,
            "per_projection": per_projection,
            "prefill": prefill,
            "column_parallel": colpar,
            "device_status": status,
            "fused_state": Q.fused_state(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
