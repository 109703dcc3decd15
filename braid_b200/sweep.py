"""Per-projection sweeps: decode regime in GB/s (M = 1..128), prefill regime in TFLOP/s
(M = 2048 / 8192 / a ragged 16-sequence pack), quantizer GB/s — each beside the library GEMM the
reference calls (`torch._scaled_mm`) on the same GPU.  Run as `python bench.py --sweep`.

Method (the reference's own, braid/bench/noise_floor.py:52-105 and braid/bench/gemm_paths.py:50-74):
`inner` back-to-back calls captured in one CUDA graph, rotating through a bank of distinct weight
copies sized past L2 (>= 1 GiB working set) so every call streams from HBM; median of `reps`
replays timed with CUDA events; never a sync per call.
"""
from __future__ import annotations

import json
import os
import statistics
from pathlib import Path

import torch

from . import quant as Q

PROJECTIONS = {
    # name: (list of N per weight of one grouped launch, K)
    "mlp.gate_up": ([12288, 12288], 4096),
    "mlp.down": ([4096], 12288),
    "gdn.in_proj_qkv_z": ([8192, 4096], 4096),
    "gdn.out_proj": ([4096], 4096),
    "attn.qkv": ([8192, 1024, 1024], 4096),
    "attn.o_proj": ([4096], 4096),
    "attn.k_proj": ([1024], 4096),
    "lm_head": ([248320], 4096),
}


def _bank(ns, k, dev, min_bytes=1 << 30, max_copies=64):
    per = sum(ns) * k
    copies = max(2, min(max_copies, -(-min_bytes // per)))
    g = torch.Generator(device=dev).manual_seed(0)
    bank = []
    for _ in range(copies):
        ws = []
        for n in ns:
            data = torch.randint(0, 120, (n, k), generator=g, device=dev, dtype=torch.uint8).view(Q.FP8)
            ws.append(Q.FP8Weight(data, torch.full((1, 1), 0.01, device=dev), (n, k)))
        bank.append(ws)
    return bank


def _time_graph(fn_of_index, n_bank, inner, reps):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(min(n_bank, 3)):
            fn_of_index(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(inner):
            fn_of_index(i % n_bank)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / inner)
    return statistics.median(times)     # ms per call


def gemm_row(name, ns, k, m, dev, peaks, inner=None, reps=15, library=True):
    bank = _bank(ns, k, dev)
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    xq, sx = Q.quantize_act(x)
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for n in ns]
    flops = 2 * m * sum(ns) * k
    bytes_ = sum(ns) * k + m * k + 2 * m * sum(ns)
    if inner is None:
        inner = max(4, min(64, int(2e9 // max(bytes_, flops // 2000))))
    ms = _time_graph(lambda i: Q.fp8_matmul_grouped(xq, sx, bank[i], out=outs), len(bank), inner, reps)
    launch = Q.last_gemm_launch()
    row = {"proj": name, "M": m, "N": ns, "K": k, "us": ms * 1e3,
           "gbs": bytes_ / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
           "frac_hbm": bytes_ / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "launch": launch}
    if library:
        def lib(i):
            for w, o in zip(bank[i], outs):
                torch._scaled_mm(xq, w.data.t(), scale_a=sx, scale_b=w.scale,
                                 out_dtype=torch.bfloat16, out=o)
        try:
            ms_lib = _time_graph(lib, len(bank), inner, reps)
            row.update({"lib_us": ms_lib * 1e3, "lib_gbs": bytes_ / (ms_lib * 1e-3) / 1e9,
                        "lib_tflops": flops / (ms_lib * 1e-3) / 1e12, "speedup_vs_lib": ms_lib / ms})
        except Exception as e:  # noqa: BLE001
            row["lib_error"] = f"{type(e).__name__}: {str(e)[:100]}"
    del bank
    torch.cuda.empty_cache()
    return row


def lm_head_rows(dev, peaks, ms=(16, 128), vocab=248320, k=4096, reps=7):
    """The `head` group (braid/model/engine.py:349): logits GEMM + `argmax(-1)` as the scheduler
    runs it (braid/serve/scheduler.py:346) against the GEMM with the pick in its epilogue (no
    logits written)."""
    bank = _bank([vocab], k, dev, min_bytes=2 << 30, max_copies=3)
    rows = []
    for m in ms:
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        xq, sx = Q.quantize_act(x)
        pre = Q.QuantizedActivation(xq, sx, x.shape, x.dtype)
        t_logits = _time_graph(lambda i: Q.fp8_matmul(xq, sx, bank[i][0]).argmax(-1), len(bank), 3, reps)
        t_pick = _time_graph(lambda i: Q.lm_head_argmax(pre, bank[i][0]), len(bank), 3, reps)
        bytes_ = vocab * k + m * k
        rows.append({"proj": "lm_head", "M": m, "logits_then_argmax_us": t_logits * 1e3,
                     "argmax_in_epilogue_us": t_pick * 1e3, "speedup": t_logits / t_pick,
                     "gbs": bytes_ / (t_pick * 1e-3) / 1e9,
                     "frac_hbm": bytes_ / (t_pick * 1e-3) / 1e9 / peaks["hbm_gbs"]})
    del bank
    torch.cuda.empty_cache()
    return rows


def quant_row(kind, m, cols, dev, peaks, reps=15):
    n_bank = max(2, min(64, (256 << 20) // (m * cols * 2)))
    if kind == "plain":
        xs = [torch.randn(m, cols, device=dev).to(torch.bfloat16) for _ in range(n_bank)]
        fn = lambda i: Q.quantize_act(xs[i])  # noqa: E731
        bytes_ = 3 * m * cols
    elif kind == "silu_mul":
        xs = [torch.randn(m, 2 * cols, device=dev).to(torch.bfloat16) for _ in range(n_bank)]
        fn = lambda i: Q.silu_mul_quant(xs[i][:, :cols], xs[i][:, cols:])  # noqa: E731
        bytes_ = 5 * m * cols
    elif kind in ("rms_norm", "rms_norm_dense"):
        xs = [torch.randn(m, cols, device=dev).to(torch.bfloat16) for _ in range(n_bank)]
        gamma = 1.0 + 0.02 * torch.randn(cols, device=dev)
        dense = kind == "rms_norm_dense"
        fn = lambda i: Q.rms_norm_quant(xs[i], gamma, 1e-6, keep_dense=dense).q  # noqa: E731
        bytes_ = (5 if dense else 3) * m * cols
    elif kind == "gated_rms_norm":
        xs = [(torch.randn(m, cols, device=dev), torch.randn(m, cols, device=dev).to(torch.bfloat16))
              for _ in range(n_bank)]
        gamma = 1.0 + 0.02 * torch.randn(128, device=dev)
        fn = lambda i: Q.gated_rms_norm_quant(xs[i][0], xs[i][1], gamma, 1e-6, 128).q  # noqa: E731
        bytes_ = 7 * m * cols
    elif kind in ("rms_norm_torch", "gated_rms_norm_torch"):
        # the reference's spelling on the same GPU: norm as torch kernels, then this package's quantizer
        xs = [(torch.randn(m, cols, device=dev).to(torch.bfloat16),
               torch.randn(m, cols, device=dev).to(torch.bfloat16)) for _ in range(n_bank)]
        if kind == "rms_norm_torch":
            gamma = 1.0 + 0.02 * torch.randn(cols, device=dev)
            fn = lambda i: Q.quantize_act(Q.torch_rms_norm(xs[i][0], gamma, 1e-6))  # noqa: E731
        else:
            gamma = 1.0 + 0.02 * torch.randn(128, device=dev)
            fn = lambda i: Q.quantize_act(Q.torch_rms_norm_gated(  # noqa: E731
                xs[i][0].reshape(-1, 128), xs[i][1].reshape(-1, 128), gamma, 1e-6).reshape(m, cols))
        bytes_ = 3 * m * cols
    else:
        raise ValueError(kind)
    inner = max(8, min(128, int(5e8 // bytes_)))
    ms = _time_graph(fn, n_bank, inner, reps)
    return {"quant": kind, "M": m, "cols": cols, "us": ms * 1e3,
            "gbs": bytes_ / (ms * 1e-3) / 1e9, "frac_hbm": bytes_ / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}


def mlp_block_row(m, dev, peaks, hidden=4096, inter=12288, reps=11):
    """The whole quantized MLP block of one layer (BASELINE config 2): quantize -> gate|up GEMM ->
    SiLU*mul fused into the quantization of the intermediate -> down GEMM, beside the reference's
    spelling of the same block on the same GPU (torch quantizer, three `torch._scaled_mm`)."""
    import torch.nn.functional as F
    n_bank = max(2, (1 << 30) // (3 * hidden * inter))
    g = torch.Generator(device=dev).manual_seed(2)

    def w(n, k):
        data = torch.randint(0, 120, (n, k), generator=g, device=dev, dtype=torch.uint8).view(Q.FP8)
        return Q.FP8Weight(data, torch.full((1, 1), 0.01, device=dev), (n, k))

    bank = [(w(inter, hidden), w(inter, hidden), w(hidden, inter)) for _ in range(n_bank)]
    x = torch.randn(m, hidden, device=dev).to(torch.bfloat16)
    inner = 8
    ms = _time_graph(lambda i: Q.mlp_forward(x, *bank[i]), n_bank, inner, reps)

    def lib_quant(t):
        scale = (t.float().abs().amax() / Q.FP8_MAX).clamp(min=Q.EPS).reshape(1, 1)
        return (t.float() / scale).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(Q.FP8), scale

    def lib(i):
        wg, wu, wd = bank[i]
        xq, sx = lib_quant(x)
        mm = lambda a, s, ww: torch._scaled_mm(a, ww.data.t(), scale_a=s, scale_b=ww.scale,  # noqa: E731
                                               out_dtype=torch.bfloat16)
        h = F.silu(mm(xq, sx, wg)) * mm(xq, sx, wu)
        hq, sh = lib_quant(h)
        return mm(hq, sh, wd)

    ms_lib = _time_graph(lib, n_bank, inner, reps)
    weight_bytes = 3 * hidden * inter
    return {"block": "mlp", "M": m, "us": ms * 1e3, "lib_us": ms_lib * 1e3, "speedup_vs_lib": ms_lib / ms,
            "weight_gbs": weight_bytes / (ms * 1e-3) / 1e9,
            "frac_hbm": weight_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "launches": 4}


def fp8_library_peak(dev, seconds=2.0):
    """Dense FP8 peak the way the bf16 peak file was taken: `torch._scaled_mm` 8192^3, best of
    10 (burst) and back to back for `seconds` (sustained)."""
    n = 8192
    a = torch.randn(n, n, device=dev).to(Q.FP8)
    b = torch.randn(n, n, device=dev).to(Q.FP8)
    one = torch.ones(1, 1, device=dev)
    f = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
    for _ in range(3):
        f()
    best = 1e9
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); f(); e.record(); torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e))
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = max(10, int(seconds * 1e3 / best))
    s.record()
    for _ in range(iters):
        f()
    e.record(); torch.cuda.synchronize()
    sustained = s.elapsed_time(e) / iters
    fl = 2 * n ** 3
    return {"fp8_tflops_burst": fl / (best * 1e-3) / 1e12,
            "fp8_tflops_sustained": fl / (sustained * 1e-3) / 1e12}


def _read_phase_ring(lib):
    import ctypes
    import numpy as np
    launches, ctas, words = 1024, 256, 10
    buf = np.zeros(launches * ctas * words, dtype=np.uint64)
    n = ctypes.c_int(0)
    lib.bq_debug_read_phases.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    rc = lib.bq_debug_read_phases(buf.ctypes.data, ctypes.byref(n))
    if rc != 0:
        raise RuntimeError(f"bq_debug_read_phases: status {rc}")
    return buf.reshape(launches, ctas, words).astype(np.int64), int(n.value)


def phase_tables(args, dev, peaks):
    """Per-phase timing of the decode-regime kernels from a development build of the library
    (`python -m braid_b200.build --phases`, loaded through BRAID_B200_LIB).  Every CTA stamps
    %globaltimer at: 0 entry, 1 set-up done, 2 dependency wait returned (producer thread),
    3 first weight tile landed (MMA thread), 4 accumulator complete, 5 staged in shared memory
    and cluster barrier passed, 6 K slices reduced and stored, 7 exit.  Quantizer CTAs stamp
    0, 2, 4 (amax exchanged) and 7.  Times are medians over the CTAs of a launch, in microseconds
    from the launch's first CTA entry; `gap_prev` is entry minus the previous launch's last exit
    (negative = the launches overlapped)."""
    import numpy as np
    from . import _lib
    lib = _lib.load()
    if not hasattr(lib, "bq_debug_phases"):
        raise RuntimeError("this build of the library has no phase stamps: build with "
                           "`python -m braid_b200.build --phases` and set BRAID_B200_LIB")
    lib.bq_debug_phases.argtypes = [__import__("ctypes").c_int]

    def run_chain(body):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        assert lib.bq_debug_phases(1) == 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        for _ in range(4):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        ring, n = _read_phase_ring(lib)
        lib.bq_debug_phases(0)
        rows, prev_end, t_first = [], None, None
        for i in range(min(n, ring.shape[0])):
            meta = ring[i, 0, 9]
            grid, kind = int(meta >> 8), int(meta & 0xFF)
            c = ring[i, :min(grid, ring.shape[1])]
            t0 = int(c[:, 0].min())
            t_first = t0 if t_first is None else t_first
            med = lambda k: (float(np.median(c[:, k][c[:, k] > 0])) - t0) / 1e3 if (c[:, k] > 0).any() else None  # noqa: E731
            row = {"launch": i, "kind": "gemm" if kind == 0 else "quant", "grid": grid,
                   "at_us": (t0 - t_first) / 1e3,
                   "gap_prev_us": None if prev_end is None else (t0 - prev_end) / 1e3,
                   "entry_spread_us": (int(c[:, 0].max()) - t0) / 1e3,
                   "setup": med(1), "dep_wait_done": med(2), "first_tile": med(3),
                   "accum_done": med(4), "staged": med(5), "reduced": med(6), "exit": med(7),
                   "last_exit": (int(c[:, 7].max()) - t0) / 1e3}
            prev_end = int(c[:, 7].max())
            rows.append(row)
        return rows, a.elapsed_time(b) * 1e3

    out = []
    for name in ("mlp.gate_up", "gdn.in_proj_qkv_z", "attn.qkv", "mlp.down", "gdn.out_proj"):
        ns, k = PROJECTIONS[name]
        for m in (16, 128):
            bank = _bank(ns, k, dev, min_bytes=1 << 29, max_copies=8)
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            xq, sx = Q.quantize_act(x)
            outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for n in ns]
            rows, total = run_chain(lambda: [Q.fp8_matmul_grouped(xq, sx, bank[i % len(bank)], out=outs)
                                             for i in range(6)])
            keep = rows[2:]           # the first launches of a replay start from an idle GPU
            avg = lambda key: float(np.mean([r[key] for r in keep if r[key] is not None]))  # noqa: E731
            bytes_ = sum(ns) * k + m * k + 2 * m * sum(ns)
            rec = {"phases": name, "M": m, "us_per_launch": total / 6, "launch": Q.last_gemm_launch(),
                   "stream_floor_us": bytes_ / peaks["hbm_gbs"] / 1e3,
                   **{key: avg(key) for key in ("gap_prev_us", "entry_spread_us", "setup", "dep_wait_done",
                                                 "first_tile", "accum_done", "staged", "reduced", "exit",
                                                 "last_exit")}}
            out.append(rec)
            print(json.dumps(rec), flush=True)
            del bank
            torch.cuda.empty_cache()
    # the launch-by-launch timeline of four layers of the decode step (quantizers and GEMMs)
    from .projection_set import ProjectionSet, StackShapes
    ps = ProjectionSet(StackShapes(), args.rows, dev, seed=0, layers=4)
    x = ps.x.clone()
    rows, total = run_chain(lambda: ps.step_b200(x, bf16_gates=False))
    for r in rows:
        print(json.dumps({"timeline": r}), flush=True)
    print(json.dumps({"timeline_total_us": total, "launches": len(rows)}), flush=True)
    return out


def column_parallel_kernels(rows: int = 4096) -> None:
    """The codes form of `FusedColumnParallelMLP` kernel by kernel, every kernel back to back
    with itself on all ranks at once (max over ranks, CUDA events), and the whole forward from
    one graph.  Run under torchrun, one process per GPU:
        python -m torch.distributed.run --nproc-per-node N bench.py --sweep --only column_parallel --rows 4096
    Rank 0 prints one JSON line."""
    import torch.distributed as dist
    from .parallel import FusedColumnParallelMLP
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    Q.warm_fused(True)
    mlp = FusedColumnParallelMLP.random_init(4096, 12288, dev, dist.group.WORLD, seed=1, rows_max=max(256, rows))
    mlp.connect()
    rank, b = mlp.rank, mlp.buffers
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(rows, 4096, generator=g, device=dev).to(torch.bfloat16)
    xq, sx = Q.quantize_act(x)

    def timed(fn, n=10):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        c.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(c) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    spare = [s + 32 for _, _, s in b.peers]        # counters nobody waits on
    col, hcol = mlp.i_ranges[rank][0], mlp.h_ranges[rank][0]
    h_local, sh = Q.gate_up_silu(xq, sx, mlp.gate, mlp.up, x.dtype)
    hq = b.hq[:rows].view(Q.FP8)
    Q.cast_act_push(h_local, sh, [h + col for h, _, _ in b.peers], mlp.I, spare)
    torch.cuda.synchronize()
    dist.barrier()
    y_local = Q.fp8_matmul(hq, sh, mlp.down, out_dtype=x.dtype)
    out = {"ranks": mlp.world, "rows": rows, "us": {
        "quantize x": timed(lambda: Q.quantize_act(x)),
        "gate/up + SiLU*mul of the shard (local)": timed(lambda: Q.gate_up_silu(xq, sx, mlp.gate, mlp.up, x.dtype)),
        "shard scale word to every rank": timed(lambda: Q.word_push(sh, mlp._slot_ptrs(), spare)),
        "cast of the shard (local)": timed(lambda: Q.cast_act(h_local, sh)),
        "cast + codes to every rank": timed(lambda: Q.cast_act_push(
            h_local, sh, [h + col for h, _, _ in b.peers], mlp.I, spare)),
        "down shard (local)": timed(lambda: Q.fp8_matmul(hq, sh, mlp.down, out_dtype=x.dtype)),
        "down shard, y to every rank from the epilogue": timed(lambda: Q.gemm_push(
            hq, sh, mlp.down, mlp.dtype, [y + hcol * 2 for _, y, _ in b.peers], mlp.H, spare)),
        "y block to every rank (separate kernel)": timed(lambda: Q.rows_push(
            y_local, [y + hcol * 2 for _, y, _ in b.peers], mlp.H, spare)),
    }}
    mlp.forward(x)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        mlp.forward(x)
    out["us"]["whole forward, one graph"] = timed(graph.replay, n=20)
    out["wait_status"] = mlp.last_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    mlp.close()
    dist.destroy_process_group()


def main(args):
    import bench   # peaks reader lives with the benchmark
    if getattr(args, "only", None) == "column_parallel":
        column_parallel_kernels(args.rows if args.rows > 256 else 4096)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Q.warm_fused(True)
    peaks = bench.measured_peaks()
    out_dir = Path(os.environ.get("BQ_SWEEP_OUT", "out"))   # where sweep.json is written
    rows = []
    only = getattr(args, "only", None)
    if only in ("rms_norm", "rms_norm_dense", "gated_rms_norm"):
        print(json.dumps(quant_row(only, args.rows, 4096, dev, peaks, reps=3)), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only == "phases":
        phase_tables(args, dev, peaks)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only == "mlp_block":
        # the whole quantized MLP of one layer at --rows (paired gate/up kernel + down): what the
        # ncu capture of the paired epilogue runs
        print(json.dumps(mlp_block_row(args.rows, dev, peaks, reps=3)), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only == "lm_head_argmax":
        for r in lm_head_rows(dev, peaks):
            print(json.dumps(r), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only == "quant_plain":
        # the plain quantizer at --rows x 4096 (the streaming kernel at prefill sizes): what the
        # ncu capture of quant_stream_kernel runs
        print(json.dumps(quant_row("plain", args.rows, 4096, dev, peaks, reps=3)), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only == "norms":
        for kind in ("rms_norm", "rms_norm_dense", "rms_norm_torch", "gated_rms_norm",
                     "gated_rms_norm_torch"):
            for m in (1, 16, 128):
                print(json.dumps(quant_row(kind, m, 4096, dev, peaks)), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    if only:
        # one projection at one row count (what the ncu captures of single kernels run):
        # a handful of launches, no library arm
        ns, k = PROJECTIONS[only]
        r = gemm_row(only, ns, k, args.rows, dev, peaks, inner=4, reps=3, library=False)
        print(json.dumps(r), flush=True)
        print(json.dumps({"device_status": Q.device_status()}), flush=True)
        return
    peak8 = fp8_library_peak(dev)
    print(json.dumps({"fp8_peak": peak8}), flush=True)
    for name, (ns, k) in PROJECTIONS.items():
        for m in (1, 8, 16, 32, 64, 128):
            r = gemm_row(name, ns, k, m, dev, peaks, inner=6 if name == "lm_head" else None,
                         reps=7 if name == "lm_head" else 15)
            rows.append(r)
            print(json.dumps(r), flush=True)
    for m in (1, 8, 16, 32, 64, 128):
        r = mlp_block_row(m, dev, peaks)
        rows.append(r)
        print(json.dumps(r), flush=True)
    g = torch.Generator().manual_seed(4)
    ragged = int(torch.randint(64, 1025, (16,), generator=g).sum().item())
    for name in ("mlp.gate_up", "mlp.down", "gdn.in_proj_qkv_z", "gdn.out_proj"):
        ns, k = PROJECTIONS[name]
        for m in (2048, 8192, ragged):
            r = gemm_row(name, ns, k, m, dev, peaks, inner=4, reps=7)
            r["frac_fp8_burst"] = r["tflops"] / peak8["fp8_tflops_burst"]
            r["frac_fp8_nominal"] = r["tflops"] / 4500.0
            rows.append(r)
            print(json.dumps(r), flush=True)
    for m, cols in ((1, 4096), (16, 4096), (128, 4096), (128, 12288), (8192, 4096)):
        r = quant_row("plain", m, cols, dev, peaks)
        rows.append(r)
        print(json.dumps(r), flush=True)
    for m in (16, 128, 2048):
        r = quant_row("silu_mul", m, 12288, dev, peaks)
        rows.append(r)
        print(json.dumps(r), flush=True)
    for kind in ("rms_norm", "rms_norm_dense", "rms_norm_torch", "gated_rms_norm", "gated_rms_norm_torch"):
        for m in (1, 16, 128):
            r = quant_row(kind, m, 4096, dev, peaks)
            rows.append(r)
            print(json.dumps(r), flush=True)
    out_dir.mkdir(exist_ok=True)
    (out_dir / "sweep.json").write_text(json.dumps({"fp8_peak": peak8, "rows": rows}, indent=1))
    print(json.dumps({"device_status": Q.device_status()}), flush=True)
