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
on the host cores, on a bounded sample: one layer of each kind, scaled by the layer counts.
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
def cpu_baseline(rows: int, reps: int = 1):
    """The reference's CPU spelling on a bounded sample: one GDN, one attention and one MLP layer
    of projections, timed in full and scaled by the stack's 24 / 8 / 32 layer counts."""
    from braid_b200.projection_set import StackShapes
    from oracle import cpu_spelling as C
    s = StackShapes()
    g = torch.Generator().manual_seed(0)

    def weight(n, k):
        w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
        return C.quantize(w)

    x = torch.randn(rows, s.hidden, generator=g).to(torch.bfloat16)
    core = torch.randn(rows, s.gdn_inner, generator=g).to(torch.bfloat16)
    H, I = s.hidden, s.intermediate
    gdn = [weight(s.gdn_qkv, H), weight(s.gdn_z, H), weight(H, s.gdn_inner)]
    att = [weight(s.attn_q, H), weight(s.attn_kv, H), weight(s.attn_kv, H), weight(H, H)]
    mlp = [weight(I, H), weight(I, H), weight(H, I)]

    def run_gdn():
        C.project(x, gdn[0], gdn[1])
        C.linear(core, *gdn[2])

    def run_att():
        qg, _, _ = C.project(x, att[0], att[1], att[2])
        gate = qg.view(rows, s.attn_heads, 2 * s.attn_head_dim)[..., s.attn_head_dim:]
        C.linear(core * torch.sigmoid(gate.reshape(rows, H)), *att[3])

    def run_mlp():
        C.mlp(x, mlp[0], mlp[1], mlp[2])

    def best(fn):
        fn()
        ts = []
        for _ in range(max(1, reps)):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    n_att = s.n_layers // s.attn_every
    n_gdn = s.n_layers - n_att
    t_step = n_gdn * best(run_gdn) + n_att * best(run_att) + s.n_layers * best(run_mlp)
    return {"value": rows / t_step, "unit": "tok/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": (f"1 GDN + 1 attention + 1 MLP layer of projections at {rows} rows timed in "
                       f"full with the reference's CPU spelling (torch quantizer + fp32 dequant-"
                       f"matmul on {torch.get_num_threads()} threads), scaled by {n_gdn}/{n_att}/"
                       f"{s.n_layers} layers; est. {t_step * 1e3:.0f} ms per step"),
            "host_cpus": os.cpu_count()}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(args.warmup and 1):
        cpu_baseline(args.rows, reps=1)
    vals = [cpu_baseline(args.rows, reps=1) for _ in range(min(args.steps, 3))]
    best = max(vals, key=lambda d: d["value"])
    line = {
        "impl": "reference", "metric": METRIC, "value": best["value"], "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": args.rows / best["value"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f8e4m3xf8e4m3->f32",
        "data": "synthetic",
        "config": {"workload": "decode_step_projection_set", "rows": args.rows, "layers": 32,
                   "hidden": 4096, "intermediate": 12288, "device": "host CPU"},
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


def column_parallel_block(dist, rows_list, steps, warmup):
    """gate_up [2 x 12288, 4096] and down [4096, 12288] N-split over the ranks, bf16 all-gather of
    the h shards and of the output shards (NCCL over NVLink)."""
    from braid_b200 import quant as Q
    from braid_b200.parallel import ColumnParallelMLP
    out = {}
    for rows in rows_list:
        mlp = ColumnParallelMLP.random_init(4096, 12288, torch.device("cuda"), dist.group.WORLD, seed=1)
        x = torch.randn(rows, 4096, device="cuda").to(torch.bfloat16)
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
        # buffers over CUDA IPC, per-rank arrival counters, no collective): decode sizes only
        if rows <= 256:
            try:
                from braid_b200.parallel import FusedColumnParallelMLP
                fmlp = FusedColumnParallelMLP.random_init(4096, 12288, torch.device("cuda"),
                                                          dist.group.WORLD, seed=1)
                fmlp.connect()
                y_fused = fmlp.forward(x).clone()
                torch.cuda.synchronize()
                dist.barrier()
                gf, _ = capture(lambda: fmlp.forward(x))
                msf, _ = timed_replays(gf.replay, steps, warmup, dist=dist)
                entry["fused"] = {"ms_per_call": msf / steps,
                                  "equals_nccl_form": bool(torch.equal(y_fused, y_nccl)),
                                  "wait_status": int(fmlp.buffers.status.item()),
                                  "launches_per_call": 4,
                                  "what": "GEMM epilogues store into every rank's gathered buffer "
                                          "through peer pointers; arrival waits in the consumer / a one-thread kernel; no NCCL"}
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
        if "fused" in entry and "ms_per_call" in entry["fused"]:
            entry["fused"]["speedup_vs_single_gpu"] = (ms1 / steps) / entry["fused"]["ms_per_call"]
            entry["fused"]["speedup_vs_nccl_form"] = (ms / steps) / entry["fused"]["ms_per_call"]
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
    # dram read+write per launch measured by ncu on the three launch shapes of a 2-layer case
    # (profiles/gemm_stream_kernel_decode_M128.md): 1.01-1.04 x the algorithmic bytes, scaled here
    # to the average launch of the full step (traffic grows in proportion to the weights)
    traffic_ratio = 1.02
    roofline = {"bound": "hbm", "kernel": "gemm_stream_kernel", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"],
                "traffic": traffic_ratio * gemm_bytes / max(1, gemm_launches),
                "traffic_source": "ncu dram__bytes_read+write on a 2-layer capture, scaled by weight bytes",
                "launches_per_step": gemm_launches,
                "algorithmic_bytes_per_launch": gemm_bytes / max(1, gemm_launches),
                "avg_launch_us": ms_gemm / args.steps / max(1, gemm_launches) * 1e3}
    step_bytes = gemm_bytes + ps.quant_algorithmic_bytes()
    status = Q.device_status()

    # ---- the step without the 48 bf16 gate projections: this package's kernels only ----------
    n2 = Q.launch_count()
    g_fp8, _ = capture(lambda: ps.step_b200(static_x, bf16_gates=False))
    fp8_launches = (Q.launch_count() - n2) // 4
    ms_fp8, _ = timed_replays(g_fp8.replay, args.steps, args.warmup, dist=None)
    del g_fp8

    # ---- the same step built from the library GEMM + torch-spelling quantizer ---------------
    library = None
    if not args.no_library_arm and rank == 0:
        try:
            g_lib, _ = capture(lambda: ps.step_library(static_x))
            ms_lib, _ = timed_replays(g_lib.replay, args.steps, args.warmup, dist=None)
            library = {"value": args.rows / (ms_lib / args.steps * 1e-3), "unit": "tok/s",
                       "ms_per_step": ms_lib / args.steps,
                       "what": "same step from torch._scaled_mm + torch-spelling quantizer, "
                               "one CUDA graph, same weights, one GPU"}
            del g_lib
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            library = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    colpar = None
    if dist is not None:
        try:
            colpar = column_parallel_block(dist, [128, 4096], max(5, args.steps // 3), 3)
        except Exception as e:  # noqa: BLE001
            colpar = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu = cpu_baseline(args.rows)
        except Exception as e:  # noqa: BLE001
            cpu = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f8e4m3xf8e4m3->f32", "data": "synthetic",
            "config": {"workload": "decode_step_projection_set", "rows": args.rows,
                       "layers": args.layers, "hidden": shapes.hidden,
                       "intermediate": shapes.intermediate, "gdn_layers": 24, "attn_layers": 8,
                       "fp8_weight_bytes": ps.fp8_weight_bytes(), "parallelism": f"dp{world}",
                       "l2": "inputs larger than L2 (6.9 GB of weights streamed per step)",
                       "timing": "CUDA-graph replay, CUDA events, max over ranks",
                       "ab_gates": "bf16 F.linear, as the reference keeps them"},
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
            "fp8_kernels_only": {"ms_per_step": ms_fp8 / args.steps,
                                 "launches_per_step": fp8_launches,
                                 "what": "the step without the 48 bf16 gate GEMMs (F.linear) the "
                                         "reference keeps in bf16: every launch is this library's"},
            "cpu_baseline": cpu,
            "library_baseline": library,
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
