"""Multi-GPU forms of the projection path on one NVLink/NVSwitch node (one process per GPU).

The reference is single-GPU (no collective anywhere in its tree); these two forms are the ones
the benchmark configuration defines:

  * data-parallel: independent request batches, weights replicated, NO collective — nothing to
    build beyond running one `ProjectionSet` per rank (see bench.py);
  * column-parallel MLP: gate/up and down are split over their output rows (N).  Every rank sees
    the same activation, so `quantize_act(x)` is bit-identical everywhere without communication
    (max is exact).  Rank r computes its slice of SiLU(gate)*up, the bf16 slices are all-gathered
    (NCCL over NVLink) into the full `[M, I]` intermediate, every rank quantizes that (identical
    scale on all ranks and identical to the single-GPU value), computes its slice of the down
    projection, and the bf16 output slices are all-gathered into `[M, H]`.

Weight shards keep the per-tensor scale of the WHOLE weight, so results equal the single-GPU
ones bit for bit.  `ops` is the module providing `quantize_act`, `fp8_matmul_grouped` and
`FP8Weight` (default: `braid_b200.quant`); the CPU tests drive the sharding and gather logic with
a stand-in over gloo.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


def shard_rows(n: int, world: int, rank: int, multiple: int = 16) -> tuple[int, int]:
    """Row range [lo, hi) of rank `rank`; every shard is a multiple of `multiple` rows and
    shards differ by at most one unit."""
    if n % multiple:
        raise ValueError(f"{n} rows cannot be split in units of {multiple}")
    units = n // multiple
    base, rem = divmod(units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo * multiple, hi * multiple


def gather_columns(local: torch.Tensor, group, sizes: list[int]) -> torch.Tensor:
    """All-gather `[M, n_r]` column slices into `[M, sum n_r]` (slices may differ in width)."""
    world = dist.get_world_size(group)
    M = local.shape[0]
    if len(set(sizes)) == 1:
        flat = torch.empty((world * M, sizes[0]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(flat, local.contiguous(), group=group)
        return flat.view(world, M, sizes[0]).permute(1, 0, 2).reshape(M, world * sizes[0])
    # uneven slices: pad every slice to the widest, gather, drop the padding
    widest = max(sizes)
    padded = torch.zeros((M, widest), dtype=local.dtype, device=local.device)
    padded[:, :local.shape[1]] = local
    flat = torch.empty((world * M, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded, group=group)
    parts = flat.view(world, M, widest)
    return torch.cat([parts[r, :, :n] for r, n in enumerate(sizes)], dim=1)


class ColumnParallelMLP:
    """The quantized SwiGLU MLP (braid/model/mlp.py:44-49) with N-split weights."""

    def __init__(self, gate, up, down, group=None, ops=None):
        """`gate`, `up` `[I, H]` and `down` `[H, I]` are FULL FP8Weights; this rank keeps its rows."""
        if ops is None:
            from . import quant as ops
        self.ops, self.group = ops, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        I, H = gate.shape
        self.I, self.H = I, H
        self.i_ranges = [shard_rows(I, self.world, r) for r in range(self.world)]
        self.h_ranges = [shard_rows(H, self.world, r) for r in range(self.world)]
        ilo, ihi = self.i_ranges[self.rank]
        hlo, hhi = self.h_ranges[self.rank]
        W = ops.FP8Weight
        self.gate = W(gate.data[ilo:ihi].contiguous(), gate.scale, (ihi - ilo, H))
        self.up = W(up.data[ilo:ihi].contiguous(), up.scale, (ihi - ilo, H))
        self.down = W(down.data[hlo:hhi].contiguous(), down.scale, (hhi - hlo, I))

    @classmethod
    def random_init(cls, hidden, inter, device, group=None, seed=0, ops=None):
        if ops is None:
            from . import quant as ops
        g = torch.Generator(device=device).manual_seed(seed)   # same weights on every rank
        mk = lambda n, k: ops.quantize_weight(  # noqa: E731
            (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16))
        return cls(mk(inter, hidden), mk(inter, hidden), mk(hidden, inter), group, ops)

    def gather_bytes(self, rows: int) -> dict:
        return {"h": rows * self.I * 2, "y": rows * self.H * 2}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        *lead, K = x.shape
        x2 = x.reshape(-1, K)
        xq, sx = ops.quantize_act(x2)                       # identical on every rank
        g, u = ops.fp8_matmul_grouped(xq, sx, (self.gate, self.up), out_dtype=x.dtype)
        h_local = F.silu(g) * u                             # bf16, as the reference rounds it
        h = gather_columns(h_local, self.group, [hi - lo for lo, hi in self.i_ranges])
        hq, sh = ops.quantize_act(h)                        # full-tensor scale, identical everywhere
        (y_local,) = ops.fp8_matmul_grouped(hq, sh, (self.down,), out_dtype=x.dtype)
        y = gather_columns(y_local, self.group, [hi - lo for lo, hi in self.h_ranges])
        return y.reshape(*lead, self.H)

    __call__ = forward
