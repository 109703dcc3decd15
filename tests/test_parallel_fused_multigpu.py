"""The peer-memory column-parallel MLP as it really runs: one PROCESS per GPU, buffers mapped
through CUDA IPC, on 2 GPUs of one node.  Skipped where fewer than two GPUs are visible (the
single-GPU emulation in test_parallel_fused_gpu.py covers the kernels there).  The handle
exchange goes over a gloo group, so no NCCL communicator is involved at all."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]

ROOT = str(Path(__file__).resolve().parent.parent)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import torch.nn.functional as F
    from braid_b200 import quant as Q
    from braid_b200.parallel import FusedColumnParallelMLP
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = torch.device("cuda", rank)
    Q.warm_fused(True)
    hidden, inter = 4096, 12288
    mlp = FusedColumnParallelMLP.random_init(hidden, inter, dev, dist.group.WORLD, seed=1, rows_max=1024)
    mlp.connect()
    # every rank can rebuild every shard (same seed): the unfused, gathered spelling, locally
    g = torch.Generator(device=dev).manual_seed(1)
    mk = lambda n, k: Q.quantize_weight((torch.randn(n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16))  # noqa: E731
    full = (mk(inter, hidden), mk(inter, hidden), mk(hidden, inter))
    shards = [FusedColumnParallelMLP(*full, ops=Q, world=world, rank=r) for r in range(world)]
    ok = True
    # decode sizes (weight-streaming kernel) and prefill sizes (CTA-pair kernel), buffers reused
    for call, M in enumerate((1, 16, 128, 128, 300, 1000, 1000, 64)):
        gx = torch.Generator(device=dev).manual_seed(100 + call)      # same x on every rank
        x = torch.randn(M, hidden, generator=gx, device=dev).to(torch.bfloat16)
        y = mlp.forward(x).clone()
        xq, sx = Q.quantize_act(x)
        parts = []
        for s in shards:
            gg, uu = Q.fp8_matmul_grouped(xq, sx, (s.gate, s.up), out_dtype=x.dtype)
            parts.append(F.silu(gg) * uu)
        hq, sh = Q.quantize_act(torch.cat(parts, dim=1))
        y_ref = torch.cat([Q.fp8_matmul(hq, sh, s.down, out_dtype=x.dtype) for s in shards], dim=1)
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(y, y_ref)) and int(mlp.buffers.status.item()) == 0
        dist.barrier()
    ok = ok and Q.device_status() == 0
    for s in shards:
        s.buffers.close()
    mlp.close()
    Path(out_dir, f"rank{rank}.ok" if ok else f"rank{rank}.bad").write_text("x")
    dist.destroy_process_group()


def test_two_processes_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["rank0.ok", "rank1.ok"]


def _worker_nccl(rank: int, world: int, port: int, out_dir: str) -> None:
    """The NCCL form on real ranks: bf16 exchange at decode sizes, e4m3 codes plus a MAX
    all-reduce of the scale at prefill sizes, against the unsharded MLP on this rank's GPU."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from braid_b200 import quant as Q
    from braid_b200.parallel import ColumnParallelMLP
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    Q.warm_fused(True)
    hidden, inter = 4096, 12288
    mlp = ColumnParallelMLP.random_init(hidden, inter, dev, dist.group.WORLD, seed=1)
    g = torch.Generator(device=dev).manual_seed(1)
    mk = lambda n, k: Q.quantize_weight((torch.randn(n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16))  # noqa: E731
    wg, wu, wd = mk(inter, hidden), mk(inter, hidden), mk(hidden, inter)
    notes = []
    ok = True
    for call, M in enumerate((128, 512, 4096, 4100)):
        gx = torch.Generator(device=dev).manual_seed(200 + call)
        x = torch.randn(M, hidden, generator=gx, device=dev).to(torch.bfloat16)
        y = mlp.forward(x)
        want = Q.mlp_forward(x, wg, wu, wd)
        torch.cuda.synchronize()
        if M >= mlp.codes_from:
            # same codes, same scale, and a prefill GEMM sums K in the same order whatever the
            # rows of the weight it is given: bit-equal to the unsharded MLP
            good = bool(torch.equal(y, want))
        else:
            # the decode kernel slices K by the shape of the shard: last-bit differences
            good = float((y.float() - want.float()).abs().max() / want.float().abs().max()) < 2e-2
        notes.append(f"M={M}:{good}")
        ok = ok and good
        dist.barrier()
    ok = ok and Q.device_status() == 0
    Path(out_dir, f"rank{rank}.ok" if ok else f"rank{rank}.bad").write_text(" ".join(notes))
    dist.destroy_process_group()


def test_nccl_form_two_processes_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker_nccl, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = {p.name: p.read_text() for p in tmp_path.iterdir()}
    assert sorted(got) == ["rank0.ok", "rank1.ok"], got
