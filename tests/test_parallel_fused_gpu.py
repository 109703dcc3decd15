"""The column-parallel MLP whose GEMM epilogues store into every rank's gathered buffer
(`FusedColumnParallelMLP`), with the ranks EMULATED on one GPU: every rank's buffers live in this
process, and the launches are enqueued so that no kernel ever waits for one enqueued after it
(all pushes of an exchange precede its first wait).  The multi-process form over CUDA IPC runs in
`bench.py --gpus N` (column_parallel.fused)."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from _util import randn_cpu

pytestmark = pytest.mark.gpu

H, I = 4096, 12288


def _weights(Q):
    mk = lambda n, k, s: Q.quantize_weight(randn_cpu((n, k), seed=s, scale=0.02).cuda())  # noqa: E731
    return mk(I, H, 1), mk(I, H, 2), mk(H, I, 3)


def _emulated(Q, world, weights, rows_max=256):
    from braid_b200.parallel import FusedColumnParallelMLP
    ranks = [FusedColumnParallelMLP(*weights, ops=Q, rows_max=rows_max, world=world, rank=r)
             for r in range(world)]
    for r in ranks:
        r.buffers.connect_local([q.buffers for q in ranks])
    return ranks


def _sharded_reference(Q, ranks, x):
    """The unfused spelling of the same sharded computation, shard by shard on one GPU."""
    xq, sx = Q.quantize_act(x)
    parts = []
    for r in ranks:
        g, u = Q.fp8_matmul_grouped(xq, sx, (r.gate, r.up), out_dtype=x.dtype)
        parts.append(F.silu(g) * u)
    h = torch.cat(parts, dim=1)
    hq, sh = Q.quantize_act(h)
    return h, torch.cat([Q.fp8_matmul(hq, sh, r.down, out_dtype=x.dtype) for r in ranks], dim=1)


@pytest.mark.parametrize("world,M,form", [(w, m, "codes") for w in (2, 4, 8) for m in (1, 16, 128)]
                         + [(2, 300, "codes"), (4, 1000, "codes"), (8, 700, "codes"),
                            (2, 300, "epilogue"), (4, 1000, "epilogue"), (8, 700, "epilogue")])
def test_fused_exchange_equals_the_gathered_spelling(Q, world, M, form):
    """Decode sizes go through the weight-streaming kernel's push epilogues.  M > 256 (ragged row
    counts: clipped last tiles) either exchange e4m3 codes -- shard scales as words, their
    maximum, an elementwise cast-and-store kernel -- or push bf16 pieces from the CTA-pair
    kernel's epilogue with the shard's max |h| ahead of the arrivals."""
    weights = _weights(Q)
    ranks = _emulated(Q, world, weights, rows_max=max(256, M))
    for r in ranks:
        r.prefill_form = form
    for call in range(3):                                   # buffers and counters are reused
        x = randn_cpu((M, H), seed=10 * M + call).cuda()
        for r in ranks:
            r.push_h(x)
        for r in ranks:
            r.push_codes(M)
        for r in ranks:
            r.wait_h_push_y(M)
        outs = [r.wait_y(M).clone() for r in ranks]
        h_ref, y_ref = _sharded_reference(Q, ranks, x)
        hq_ref = Q.quantize_act(h_ref)[0].view(torch.uint8)
        for r, y in zip(ranks, outs):
            if M >= r.amax_from and r.prefill_form == "codes":   # prefill sizes exchange codes
                assert torch.equal(r.buffers.hq[:M], hq_ref), f"rank {r.rank}: gathered codes differ (call {call})"
            else:
                assert torch.equal(r.buffers.h[:M], h_ref), f"rank {r.rank}: gathered h differs (call {call})"
            assert torch.equal(y, y_ref), f"rank {r.rank}: gathered y differs (call {call})"
            assert int(r.buffers.status.item()) == 0
        # against the unsharded MLP: same codes and scales, GEMM sums within the bf16 tolerance
        y_one = Q.mlp_forward(x, *weights)
        err = (outs[0].float() - y_one.float()).abs().max() / y_one.float().abs().max()
        assert float(err) < 1e-2
    assert Q.device_status() == 0
    for r in ranks:
        r.buffers.close()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_block_pushes_store_the_same_rows_on_every_rank_and_signal(Q, dt):
    """`rows_push` (block unchanged) and `cast_act_push` (its e4m3 codes) with three destinations
    in this process: every destination gets the block at the column offset its pointer carries,
    nothing else is touched, and every counter advances by one per launch."""
    M, n, width = 300, 1024, 4096
    x = randn_cpu((M, 2 * n), seed=3, dtype=dt, scale=2.0).cuda()[:, :n]      # strided rows
    flags = torch.zeros(3, dtype=torch.int32, device="cuda")
    dst = [torch.full((M, width), -7.0, dtype=dt, device="cuda") for _ in range(3)]
    col, es = 512, x.element_size()
    Q.rows_push(x, [d.data_ptr() + col * es for d in dst], width, [flags[i:i + 1].data_ptr() for i in range(3)])
    for d in dst:
        assert torch.equal(d[:, col:col + n], x)
        assert bool((d[:, :col] == -7.0).all()) and bool((d[:, col + n:] == -7.0).all())
    scale = Q.quantize_act(x.contiguous())[1]
    want = Q.cast_act(x.contiguous(), scale).view(torch.uint8)
    qd = [torch.full((M, width), 9, dtype=torch.uint8, device="cuda") for _ in range(3)]
    Q.cast_act_push(x, scale, [d.data_ptr() + col for d in qd], width,
                    [flags[i:i + 1].data_ptr() for i in range(3)])
    for d in qd:
        assert torch.equal(d[:, col:col + n], want)
        assert bool((d[:, :col] == 9).all()) and bool((d[:, col + n:] == 9).all())
    assert flags.tolist() == [2, 2, 2]
    assert Q.device_status() == 0


def test_a_wait_that_nothing_satisfies_runs_out_and_reports(Q):
    """A counter no rank increments: the wait kernel gives up after its cycle limit (well under
    a second), raises the status word, and the context stays usable."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    seen = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    Q.wait_flag(flag, seen, 5, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 5                          # BQ_ERR_DEVICE_WAIT
    assert int(seen.item()) == 5                            # the wait still advances its baseline
    x = randn_cpu((8, 4096), seed=1).cuda()
    q, s = Q.quantize_act(x)                                # the device still works
    assert torch.isfinite(s).all()
