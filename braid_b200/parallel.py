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
    projection, and the bf16 output slices are all-gathered into `[M, H]`.  Two forms:
    `ColumnParallelMLP` exchanges through NCCL (bf16 at decode sizes; from 257 rows on e4m3
    codes under the MAX-reduced scale, half the bytes); `FusedColumnParallelMLP` uses no
    collective at all -- every rank's buffers are mapped into every other rank's process and
    the kernels store into them directly (GEMM epilogues at decode sizes; at prefill sizes the
    shard scales travel as 4-byte words and an elementwise kernel stores the codes of the local
    shard into every rank's buffer), with per-rank arrival counters and bounded waits.

Weight shards keep the per-tensor scale of the WHOLE weight, so scales and FP8 codes equal the
single-GPU ones; a GEMM output can differ from the single-GPU one in its last bit because the K
slicing of the weight-streaming kernel follows the shape of the shard it is given (with the
order-independent stand-in used on CPU the results are bit-identical).  `ops` is the module providing `quantize_act`, `fp8_matmul_grouped` and
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
        # [world, M, n] -> [M, world * n].  The copy moves whole 8-byte words where the slice width
        # allows it (it always does for the MLP's shards): a byte-wise strided copy of e4m3 codes
        # runs at a fraction of the memory rate.
        n_bytes = sizes[0] * local.element_size()
        if n_bytes % 8 == 0 and flat.data_ptr() % 8 == 0:
            words = flat.view(torch.uint8).view(world, M, n_bytes).view(torch.int64)
            out = words.permute(1, 0, 2).reshape(M, world * (n_bytes // 8))
            return out.view(torch.uint8).view(M, world * n_bytes).view(local.dtype)
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
    def random_init(cls, hidden, inter, device, group=None, seed=0, ops=None, **kwargs):
        if ops is None:
            from . import quant as ops
        g = torch.Generator(device=device).manual_seed(seed)   # same weights on every rank
        mk = lambda n, k: ops.quantize_weight(  # noqa: E731
            (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16))
        return cls(mk(inter, hidden), mk(inter, hidden), mk(hidden, inter), group, ops, **kwargs)

    def gather_bytes(self, rows: int) -> dict:
        """Bytes every rank ends up holding after each exchange (codes or bf16 for h, bf16 for y)."""
        return {"h": rows * self.I * (1 if rows >= self.codes_from else 2), "y": rows * self.H * 2,
                "h_form": "e4m3 codes + MAX all-reduce of the scale" if rows >= self.codes_from
                else "bf16"}

    # From this many rows on, the h exchange moves FP8 codes instead of bf16 values (half the
    # bytes, and nobody re-quantizes the gathered tensor); below it the exchange is bound by the
    # latency of the collectives, and the codes form needs one more (the 4-byte MAX all-reduce).
    codes_from = 257

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        *lead, K = x.shape
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        i_sizes = [hi - lo for lo, hi in self.i_ranges]
        h_sizes = [hi - lo for lo, hi in self.h_ranges]
        xq, sx = ops.quantize_act(x2)                       # identical on every rank
        n = i_sizes[self.rank]
        fused = ops.gate_up_silu(xq, sx, self.gate, self.up, x.dtype) \
            if (M >= self.codes_from and hasattr(ops, "gate_up_silu")) else None
        if fused is not None:
            # this rank's shard of h and ITS scale straight from the GEMM's epilogue; MAX over the
            # ranks gives the scale of the whole h, then the shard is cast under it
            h_local, sh = fused
            dist.all_reduce(sh, op=dist.ReduceOp.MAX, group=self.group)
            hq_local = ops.cast_act(h_local, sh)
            hq = gather_columns(hq_local.view(torch.uint8), self.group, i_sizes).view(hq_local.dtype)
            (y_local,) = ops.fp8_matmul_grouped(hq, sh, (self.down,), out_dtype=x.dtype)
            return gather_columns(y_local, self.group, h_sizes).reshape(*lead, self.H)
        gu = torch.empty((M, 2 * n), dtype=x.dtype, device=x.device)
        g, u = gu[:, :n], gu[:, n:]
        ops.fp8_matmul_grouped(xq, sx, (self.gate, self.up), out_dtype=x.dtype, out=(g, u))
        if M >= self.codes_from:
            # Scale of this rank's shard of h = silu(gate) * up, MAX over the ranks (the scale is
            # a monotone function of the amax and max is exact, so this IS the scale of the whole
            # h on every rank), then the cast of the shard with it: codes equal, byte for byte,
            # the ones a quantizer of the gathered h would produce.
            sh = ops.silu_mul_scale(g, u)
            dist.all_reduce(sh, op=dist.ReduceOp.MAX, group=self.group)
            hq_local = ops.silu_mul_cast(g, u, sh)
            hq = gather_columns(hq_local.view(torch.uint8), self.group, i_sizes).view(hq_local.dtype)
        else:
            h_local = F.silu(g) * u                         # bf16, as the reference rounds it
            h = gather_columns(h_local, self.group, i_sizes)
            hq, sh = ops.quantize_act(h)                    # full-tensor scale, identical everywhere
        (y_local,) = ops.fp8_matmul_grouped(hq, sh, (self.down,), out_dtype=x.dtype)
        y = gather_columns(y_local, self.group, h_sizes)
        return y.reshape(*lead, self.H)

    __call__ = forward


# ---------------------------------------------------------------------------------------------
# The same MLP without a collective call: the GEMM epilogues store into every rank's gathered
# buffer through peer-mapped pointers and signal per-rank arrival counters.
# ---------------------------------------------------------------------------------------------
class _DeviceBlock:
    """Raw device memory handed to torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerBuffers:
    """One rank's gathered buffers and counters, plus where the other ranks' copies are.

    `h` `[rows_max, I]` and `y` `[rows_max, H]` receive every rank's column slice (`hq`, the
    e4m3 codes of h that prefill sizes exchange instead, shares h's bytes); `sync` holds the
    arrival counters the other ranks increment (word 0: h or the shard scales, 1: y, 2: codes)
    and, from byte 64, one word per rank for that rank's shard scale or max |h|.  The three live in ONE device
    allocation made by the library (`bq_peer_alloc`), because it has to be exported to the other
    processes as a whole; `seen` and `status` are private to the rank.  `peers[r]` is rank r's
    (h, y, sync) device addresses as they are valid on THIS rank."""

    AMAX_OFFSET = 64    # bytes into `sync`: one max |h| word per rank (up to 8)

    def __init__(self, rows_max: int, inter: int, hidden: int, dtype: torch.dtype, device, ops=None):
        import ctypes
        from . import _lib
        self.device = torch.device(device)
        es = torch.empty(0, dtype=dtype).element_size()
        self.off_h = 0
        self.off_y = _align(rows_max * inter * es)
        self.off_sync = self.off_y + _align(rows_max * hidden * es)
        self.nbytes = self.off_sync + 256
        self._lib = _lib.load()
        ptr = ctypes.c_void_p()
        self.handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(self._lib.bq_peer_alloc(self.nbytes, ctypes.byref(ptr), self.handle), "peer_alloc")
        self.base = int(ptr.value)
        raw = torch.as_tensor(_DeviceBlock(self.base, self.nbytes), device=self.device)
        self._raw = raw
        self.h = raw[self.off_h:self.off_h + rows_max * inter * es].view(dtype).view(rows_max, inter)
        # the gathered e4m3 codes of h (prefill sizes exchange codes, not values) share h's bytes
        self.hq = raw[self.off_h:self.off_h + rows_max * inter].view(rows_max, inter)
        self.y = raw[self.off_y:self.off_y + rows_max * hidden * es].view(dtype).view(rows_max, hidden)
        self.sync = raw[self.off_sync:self.off_sync + 256].view(torch.int32)
        self.seen = torch.zeros(3, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.peers: list[tuple[int, int, int]] = []
        self._opened: list[int] = []

    def _addresses(self, base: int) -> tuple[int, int, int]:
        return base + self.off_h, base + self.off_y, base + self.off_sync

    def connect_ipc(self, group) -> None:
        """Exchange the 64-byte handles with every rank of `group` (one process per GPU on one
        node) and map each peer's allocation for THIS rank's device."""
        import ctypes
        from . import _lib
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        everyone: list = [None] * world
        dist.all_gather_object(everyone, bytes(self.handle.raw), group=group)
        self.peers = []
        with torch.cuda.device(self.device):
            for r in range(world):
                if r == rank:
                    self.peers.append(self._addresses(self.base))
                    continue
                p = ctypes.c_void_p()
                buf = ctypes.create_string_buffer(everyone[r], 64)
                _lib.check(self._lib.bq_peer_open(buf, ctypes.byref(p)), "peer_open")
                self._opened.append(int(p.value))
                self.peers.append(self._addresses(int(p.value)))
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def connect_local(self, all_buffers: list["PeerBuffers"]) -> None:
        """Several ranks emulated in ONE process on one GPU (tests): plain addresses."""
        self.peers = [b._addresses(b.base) for b in all_buffers]

    def close(self, group=None) -> None:
        """Unmap the peers' buffers, then (after everyone has) free this rank's own."""
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.bq_peer_close(p)
            self._opened = []
            if group is not None:
                dist.barrier(group=group)
            if self.base:
                self.h = self.hq = self.y = self.sync = self._raw = None
                self._lib.bq_peer_free(self.base)
                self.base = 0
        self.peers = []


class FusedColumnParallelMLP(ColumnParallelMLP):
    """`ColumnParallelMLP` with both all-gathers folded into the producing GEMMs, at decode sizes
    (the weight-streaming kernel) and at prefill sizes (the CTA-pair kernel) up to `rows_max` rows.

    gate/up shard: one paired GEMM whose epilogue forms this rank's slice of SiLU(gate)*up and
    stores it into every rank's `h` buffer; down shard: one GEMM whose epilogue stores its slice
    into every rank's `y` buffer.  The last CTA of a launch signals every rank once.  The wait
    for `h` sits inside the quantizer that consumes it; the wait for `y` is a one-thread kernel.
    Both are bounded (a wait that runs out raises a status word).  Four launches per rank at
    decode sizes (eight at prefill sizes, see the phases below) and no collective.  Buffers are reused from call to call: a rank cannot start writing exchange
    n+1 into a peer before that peer has finished reading exchange n, because its own exchange
    n completes only after every peer has launched past that read."""

    def __init__(self, gate, up, down, group=None, ops=None, rows_max: int = 256,
                 dtype: torch.dtype = torch.bfloat16, world: int | None = None, rank: int | None = None):
        if world is None:
            super().__init__(gate, up, down, group, ops)
        else:                                   # emulated ranks (tests): no process group
            self._init_shards(gate, up, down, ops, world, rank)
        widths = {hi - lo for lo, hi in self.i_ranges} | {hi - lo for lo, hi in self.h_ranges}
        if any(w % 64 for w in widths):
            raise ValueError("shards must be multiples of 64 rows for the paired form")
        dev = self.gate.data.device
        self.rows_max, self.dtype = rows_max, dtype
        self.buffers = PeerBuffers(rows_max, self.I, self.H, dtype, dev)
        # every rank's launch signals each rank once per exchange
        self.count_h = self.count_y = self.world

    def _init_shards(self, gate, up, down, ops, world, rank):
        if ops is None:
            from . import quant as ops
        self.ops, self.group, self.world, self.rank = ops, None, world, rank
        I, H = gate.shape
        self.I, self.H = I, H
        self.i_ranges = [shard_rows(I, world, r) for r in range(world)]
        self.h_ranges = [shard_rows(H, world, r) for r in range(world)]
        (ilo, ihi), (hlo, hhi) = self.i_ranges[rank], self.h_ranges[rank]
        W = ops.FP8Weight
        self.gate = W(gate.data[ilo:ihi].contiguous(), gate.scale, (ihi - ilo, H))
        self.up = W(up.data[ilo:ihi].contiguous(), up.scale, (ihi - ilo, H))
        self.down = W(down.data[hlo:hhi].contiguous(), down.scale, (hhi - hlo, I))

    def connect(self) -> None:
        self.buffers.connect_ipc(self.group)

    def close(self) -> None:
        self.buffers.close(self.group)

    # -- the phases (a test interleaves them over emulated ranks; forward() runs them in order)
    # Prefill sizes (from `amax_from` rows on) exchange h as e4m3 CODES: the gate/up GEMM keeps
    # its shard of h local and returns the shard's scale; the scales go round as 4-byte words;
    # a one-thread kernel waits for them and takes their maximum (the scale of the whole h); an
    # elementwise kernel casts the shard and stores the codes into every rank's buffer, a warp
    # writing 512 contiguous bytes per rank.  Half the bytes of the bf16 exchange and whole
    # lines on the links.  `prefill_form = "epilogue"` selects the other spelling: bf16 pieces
    # pushed from the GEMM's epilogue (overlapped with the GEMM, but 128-byte pieces scattered
    # over rows move at about two thirds of the links' copy rate) and the shard's max |h| ahead
    # of the arrivals.  Decode sizes: bf16 from the epilogue, the quantizer of the gathered h
    # waits in its own kernel (fewest launches).
    amax_from = 257
    prefill_form = "codes"
    _codes = False
    _h_local = None
    _sh = None

    def _slot_ptrs(self):
        return [s + PeerBuffers.AMAX_OFFSET + 4 * self.rank for _, _, s in self.buffers.peers]

    def push_h(self, x2: torch.Tensor) -> None:
        ops, es = self.ops, torch.empty(0, dtype=self.dtype).element_size()
        xq, sx = ops.quantize_act(x2)
        col = self.i_ranges[self.rank][0]
        prefill = x2.shape[0] >= self.amax_from
        self._codes = False
        if prefill and self.prefill_form == "codes":
            got = ops.gate_up_silu(xq, sx, self.gate, self.up, self.dtype)
            if got is not None:
                self._h_local, sh_local = got
                self._codes = True
                ops.word_push(sh_local, self._slot_ptrs(), [s for _, _, s in self.buffers.peers])
                return
        ops.gate_up_silu_push(xq, sx, self.gate, self.up, self.dtype,
                              [h + col * es for h, _, _ in self.buffers.peers], self.I,
                              [s for _, _, s in self.buffers.peers],
                              self._slot_ptrs() if prefill else None)

    def push_codes(self, M: int) -> None:
        """Codes form only: wait for every rank's shard scale, cast this rank's shard under their
        maximum and store the codes into every rank's buffer."""
        if not (M >= self.amax_from and self._codes):
            return
        ops, b = self.ops, self.buffers
        first = PeerBuffers.AMAX_OFFSET // 4
        self._sh = ops.wait_flag_scale(b.sync[0:1], b.seen[0:1], self.count_h, b.status,
                                       b.sync[first:first + self.world], words_are_scales=True)
        col = self.i_ranges[self.rank][0]
        ops.cast_act_push(self._h_local, self._sh, [h + col for h, _, _ in b.peers], self.I,
                          [s + 8 for _, _, s in b.peers])
        self._h_local = None

    def wait_h_push_y(self, M: int) -> None:
        ops, b, es = self.ops, self.buffers, torch.empty(0, dtype=self.dtype).element_size()
        first = PeerBuffers.AMAX_OFFSET // 4
        if M >= self.amax_from and self._codes:
            ops.wait_flag(b.sync[2:3], b.seen[2:3], self.world, b.status)
            hq, sh = b.hq[:M].view(ops.FP8), self._sh
        elif M >= self.amax_from:
            sh = ops.wait_flag_scale(b.sync[0:1], b.seen[0:1], self.count_h, b.status,
                                     b.sync[first:first + self.world])
            hq = ops.cast_act(b.h[:M], sh)
        else:
            # the wait for every rank's h shard is inside the quantizer's kernel
            hq, sh = ops.quantize_act_after(b.h[:M], b.sync[0:1], b.seen[0:1], self.count_h)
        col = self.h_ranges[self.rank][0]
        ops.gemm_push(hq, sh, self.down, self.dtype, [y + col * es for _, y, _ in b.peers], self.H,
                      [s + 4 for _, _, s in b.peers])

    def wait_y(self, M: int) -> torch.Tensor:
        b = self.buffers
        self.ops.wait_flag(b.sync[1:2], b.seen[1:2], self.count_y, b.status)
        return b.y[:M]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """The MLP output `[..., H]`.

        Up to `rows_max` rows the result is a VIEW of this rank's gathered `y` buffer, which every
        rank overwrites during the next call on this object: consume it (or copy it) on the
        launching stream before calling again.  `copy_out = True` returns a fresh tensor instead
        (one device copy).  Larger M takes the NCCL form, which always returns a fresh
        tensor.  Ranks must be barriered, with their warm-up done, before the first call: a peer
        that is more than the wait bound (about half a second) late makes the bounded waits run
        out, which `last_status()` reports."""
        *lead, K = x.shape
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        if M > self.rows_max or x.dtype != self.dtype or not self.buffers.peers:
            return super().forward(x)                    # beyond the buffers: the NCCL form
        self.push_h(x2)
        self.push_codes(M)
        self.wait_h_push_y(M)
        y = self.wait_y(M)
        if self.copy_out:
            y = y.clone()
        return y.reshape(*lead, self.H)

    copy_out = False

    def last_status(self) -> int:
        """Synchronises and returns non-zero if any bounded wait of this object's exchanges (or of
        the kernels that carried them) has run out since the last check; the result of such a
        call is built from incomplete data and must be discarded.  Call it where the host
        already synchronises, never during capture."""
        torch.cuda.synchronize(self.buffers.device)
        bad = int(self.buffers.status.item())
        if bad:
            self.buffers.status.zero_()
        return bad or int(self.ops.device_status(self.buffers.device))

    __call__ = forward
