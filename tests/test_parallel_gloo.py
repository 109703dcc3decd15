"""Column-parallel MLP sharding and gather logic over gloo, world_size 2, on CPU.

The kernels need a GPU, so the compute is a CPU stand-in with the same interface
(oracle/cpu_spelling.py); what is under test is the host logic: row ranges, scale sharing,
gather layout, and that the sharded result equals the unsharded one bit for bit."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_shard_rows_covers_everything_in_units_of_16():
    from braid_b200.parallel import shard_rows
    for n, world in ((12288, 8), (4096, 2), (4096, 3), (48, 4), (16, 2)):
        ranges = [shard_rows(n, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        for (a, b), (c, d) in zip(ranges, ranges[1:]):
            assert b == c
        assert all(lo % 16 == 0 and hi % 16 == 0 for lo, hi in ranges)
        sizes = [hi - lo for lo, hi in ranges]
        assert max(sizes) - min(sizes) <= 16
    with pytest.raises(ValueError):
        shard_rows(100, 2, 0)


class _CpuOps:
    """Stand-in for braid_b200.quant on CPU tensors (tests only)."""

    @dataclass
    class FP8Weight:
        data: torch.Tensor
        scale: torch.Tensor
        shape: tuple

    @staticmethod
    def quantize_weight(w):
        from oracle import cpu_spelling as C
        q, s = C.quantize(w)
        return _CpuOps.FP8Weight(q, s, tuple(w.shape))

    @staticmethod
    def quantize_act(x):
        from oracle import cpu_spelling as C
        return C.quantize(x)

    @staticmethod
    def fp8_matmul_grouped(xq, sx, weights, out_dtype=torch.bfloat16, out=None):
        # exact per-element sums in float64 so that a row slice equals the full product's slice
        ys = [((xq.double() * sx.double()) @ (w.data.double() * w.scale.double()).t()).to(out_dtype)
              for w in weights]
        if out is not None:
            for o, y in zip(out, ys):
                o.copy_(y)
            return list(out)
        return ys

    @staticmethod
    def silu_mul_scale(gate, up):
        import torch.nn.functional as F
        from oracle import cpu_spelling as C
        return C.quantize(F.silu(gate) * up)[1]

    @staticmethod
    def silu_mul_cast(gate, up, scale):
        import torch.nn.functional as F
        from oracle import cpu_spelling as C
        h = F.silu(gate) * up
        return (h.float() / scale).clamp(-C.FP8_MAX, C.FP8_MAX).to(C.FP8)


def _worker(rank, world, port, hidden, inter, rows, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from braid_b200.parallel import ColumnParallelMLP
        import torch.nn.functional as F
        ops = _CpuOps
        g = torch.Generator().manual_seed(5)
        mk = lambda n, k: ops.quantize_weight((torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16))  # noqa: E731
        gate, up, down = mk(inter, hidden), mk(inter, hidden), mk(hidden, inter)
        x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
        mlp = ColumnParallelMLP(gate, up, down, group=None, ops=ops)
        if rows >= 40:                      # exercise the codes exchange (scale MAX all-reduce) on CPU sizes
            mlp.codes_from = 32
        y = mlp(x.view(1, rows, hidden))
        # single-process reference with the same stand-in
        xq, sx = ops.quantize_act(x)
        gg, uu = ops.fp8_matmul_grouped(xq, sx, (gate, up))
        hq, sh = ops.quantize_act(F.silu(gg) * uu)
        (want,) = ops.fp8_matmul_grouped(hq, sh, (down,))
        ok = torch.equal(y.view(rows, hidden), want) and y.shape == (1, rows, hidden)
        ok = ok and mlp.gate.scale is gate.scale and mlp.gate.shape[0] < inter
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,hidden,inter,rows", [(2, 64, 96, 5), (2, 48, 160, 16), (2, 64, 96, 50)])
def test_column_parallel_equals_unsharded(world, hidden, inter, rows):
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, hidden, inter, rows, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
