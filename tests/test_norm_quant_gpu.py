"""RMSNorm fused into the quantizer, against the reference's torch spelling on the same device.

A sum of squares depends on the order of the additions, so bit identity with `F.rms_norm` is a
property of THIS torch build's CUDA kernel that the fused kernels restate; these tests are the
pin.  Every comparison is `torch.equal` on the dense activation, the scale and the code bytes.
Spec: braid/model/norm.py:31-45 (`rms_norm`), :48-71 (`rms_norm_gated`), consumed at
braid/model/layer.py:49,59 and braid/model/gdn.py:373-387.
"""
from __future__ import annotations

import pytest
import torch

from oracle import torch_spelling as TS
from _util import randn_cpu, u8

pytestmark = pytest.mark.gpu

EPS = 1e-6


def _gamma(n, seed, spread=0.02):
    g = torch.Generator().manual_seed(seed)
    return (1.0 + spread * torch.randn(n, generator=g)).cuda()


def _same(qa, h_ref, what):
    qr, sr = TS.quantize_act(h_ref.reshape(-1, h_ref.shape[-1]))
    assert torch.equal(qa.scale, sr), f"{what}: scale {qa.scale.item():.9e} vs {sr.item():.9e}"
    diff = int((u8(qa.q) != u8(qr)).sum())
    assert diff == 0, f"{what}: {diff} of {qr.numel()} fp8 bytes differ"


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32, torch.float16], ids=["bf16", "fp32", "fp16"])
@pytest.mark.parametrize("shape", [(1, 4096), (8, 4096), (37, 4096), (128, 4096), (128, 2560),
                                   (16, 8192), (5, 512), (3, 64), (256, 4096), (1024, 4096)])
def test_rms_norm_quant_is_bit_identical(Q, dt, shape):
    for seed in range(3):
        x = randn_cpu(shape, seed=seed * 101 + shape[0], dtype=dt, scale=(0.05, 1.0, 30.0)[seed]).cuda()
        gamma = _gamma(shape[1], seed, spread=(0.02, 0.3, 1.0)[seed])
        ref = TS.rms_norm(x, gamma, EPS)
        qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
        assert qa.shape == x.shape and qa.dtype is dt
        bad = int((u8(qa.dense) != u8(ref)).sum())
        assert bad == 0, f"{dt} {shape} seed {seed}: {bad} bytes of the normalised activation differ"
        _same(qa, ref, f"{dt} {shape} seed {seed}")
        assert Q.rms_norm_quant(x, gamma, EPS).dense is None


def test_rms_norm_quant_many_rows_of_real_width(Q):
    """2048 independent rows x 3 magnitudes: a reduction-order mismatch shows up as a last-bit
    difference in a few percent of rows, so this is the statistical net under the exact cases."""
    for seed, scale in enumerate((1e-3, 1.0, 200.0)):
        x = randn_cpu((2048, 4096), seed=40 + seed, scale=scale).cuda()
        x[::7] *= 16.0          # rows of very different energy
        gamma = _gamma(4096, seed)
        ref = TS.rms_norm(x, gamma, EPS)
        qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
        rows_bad = int((qa.dense != ref).any(dim=1).sum())
        assert rows_bad == 0, f"{rows_bad} of 2048 rows differ at scale {scale}"
        _same(qa, ref, f"scale {scale}")


def test_rms_norm_quant_strided_rows_leading_dims_and_fallback(Q):
    gamma = _gamma(4096, 1)
    wide = randn_cpu((16, 8192), seed=2).cuda()
    x = wide[:, :4096]                                  # row stride 8192
    qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
    ref = TS.rms_norm(x, gamma, EPS)
    assert torch.equal(qa.dense, ref)
    _same(qa, ref, "strided")
    x3 = randn_cpu((4, 3, 4096), seed=3).cuda()         # [B, T, H] as the layer sees it
    qa = Q.rms_norm_quant(x3, gamma, EPS, keep_dense=True)
    assert qa.shape == x3.shape and qa.dense.shape == x3.shape and qa.q.shape == (12, 4096)
    _same(qa, TS.rms_norm(x3, gamma, EPS), "3-d")
    big = randn_cpu((4096, 4096), seed=4).cuda()        # more rows than fit at once: two steps
    qa = Q.rms_norm_quant(big, gamma, EPS, keep_dense=True)
    ref = TS.rms_norm(big, gamma, EPS)
    assert torch.equal(qa.dense, ref)
    _same(qa, ref, "4096 rows")


@pytest.mark.parametrize("dt,shape", [(torch.bfloat16, (8192, 4096)), (torch.bfloat16, (2500, 2560)),
                                      (torch.float32, (3000, 4096)), (torch.float16, (4100, 512))],
                         ids=["bf16-8192x4096", "bf16-2500x2560", "fp32-3000x4096", "fp16-4100x512"])
def test_rms_norm_quant_at_prefill_sizes(Q, dt, shape):
    """More rows than one co-resident grid has CTAs: the norm loops rows per CTA and leaves h and
    its scale without a grid-wide wait (`bq_rmsnorm_scale`), the cast pass writes the codes;
    bit-identical to the torch spelling, with and without the dense output, NaN included."""
    x = randn_cpu(shape, seed=shape[0], dtype=dt, scale=3.0).cuda()
    x[::5] *= 9.0
    gamma = _gamma(shape[1], 2, spread=0.3)
    ref = TS.rms_norm(x, gamma, EPS)
    calls = Q.launch_count()
    qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
    assert Q.launch_count() - calls == 2        # the norm (which also leaves the scale), the cast
    assert torch.equal(qa.dense, ref)
    _same(qa, ref, f"{dt} {shape}")
    qb = Q.rms_norm_quant(x, gamma, EPS)
    assert qb.dense is None and torch.equal(u8(qb.q), u8(qa.q)) and torch.equal(qb.scale, qa.scale)
    x[shape[0] // 2, 7] = float("nan")
    qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
    ref = TS.rms_norm(x, gamma, EPS)
    assert torch.isnan(qa.scale).all() and torch.equal(torch.isnan(qa.dense), torch.isnan(ref))
    assert Q.device_status() == 0


def test_rms_norm_quant_degenerate_values(Q):
    gamma = _gamma(4096, 5)
    zeros = torch.zeros(4, 4096, dtype=torch.bfloat16, device="cuda")
    qa = Q.rms_norm_quant(zeros, gamma, EPS, keep_dense=True)
    assert float(qa.dense.float().abs().max()) == 0.0 and qa.scale.item() == pytest.approx(1e-12)
    x = randn_cpu((4, 4096), seed=6).cuda()
    x[2, 100] = float("nan")
    qa = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
    ref = TS.rms_norm(x, gamma, EPS)
    assert torch.isnan(qa.scale).all()
    assert torch.equal(torch.isnan(qa.dense), torch.isnan(ref))
    qr, sr = TS.quantize_act(ref)
    assert int((u8(qa.q) != u8(qr)).sum()) == 0
    huge = torch.full((2, 4096), 60000.0, dtype=torch.bfloat16, device="cuda")
    qa = Q.rms_norm_quant(huge, gamma, EPS, keep_dense=True)
    ref = TS.rms_norm(huge, gamma, EPS)
    assert torch.equal(qa.dense, ref)
    _same(qa, ref, "huge")


@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16], ids=["y_fp32", "y_bf16"])
@pytest.mark.parametrize("rows,heads", [(1, 32), (8, 32), (37, 32), (128, 32), (16, 16), (5, 48), (3, 64)])
def test_gated_rms_norm_quant_is_bit_identical(Q, ydt, rows, heads):
    D = 128
    for seed in range(3):
        scale = (0.01, 1.0, 50.0)[seed]
        y = randn_cpu((rows, heads, D), seed=seed * 17 + rows, dtype=ydt, scale=scale).cuda()
        z = randn_cpu((rows, heads * D), seed=seed * 19 + rows + 1, scale=(1.0, 3.0, 8.0)[seed]).cuda()
        gamma = _gamma(D, seed, spread=(0.02, 0.3, 1.0)[seed])
        core = y.to(torch.bfloat16).reshape(-1, D)            # braid/model/gdn.py:383
        ref = TS.rms_norm_gated(core, z.reshape(-1, D), gamma, EPS).reshape(rows, heads * D)
        qa = Q.gated_rms_norm_quant(y, z, gamma, EPS, D)
        assert qa.shape == (rows, heads * D) and qa.dtype is torch.bfloat16
        _same(qa, ref, f"{ydt} rows {rows} heads {heads} seed {seed}")


def test_gated_rms_norm_quant_many_rows_and_nan(Q):
    D, heads = 128, 32
    y = randn_cpu((1024, heads, D), seed=3, dtype=torch.float32, scale=2.0).cuda()
    y[::5] *= 40.0
    z = randn_cpu((1024, heads * D), seed=4, scale=2.0).cuda()
    gamma = _gamma(D, 9)
    ref = TS.rms_norm_gated(y.to(torch.bfloat16).reshape(-1, D), z.reshape(-1, D), gamma,
                                 EPS).reshape(1024, heads * D)
    _same(Q.gated_rms_norm_quant(y, z, gamma, EPS, D), ref, "1024 rows")
    z[7, 300] = float("nan")
    ref = TS.rms_norm_gated(y.to(torch.bfloat16).reshape(-1, D), z.reshape(-1, D), gamma,
                                 EPS).reshape(1024, heads * D)
    qa = Q.gated_rms_norm_quant(y, z, gamma, EPS, D)
    assert torch.isnan(qa.scale).all()
    qr, _ = TS.quantize_act(ref)
    assert int((u8(qa.q) != u8(qr)).sum()) == 0


@pytest.mark.parametrize("ydt,rows,heads", [(torch.float32, 8192, 32), (torch.bfloat16, 3000, 32),
                                            (torch.float32, 2500, 16)],
                         ids=["f32-scan-8192x32", "bf16-3000x32", "f32-scan-2500x16"])
def test_gated_rms_norm_quant_at_prefill_sizes(Q, ydt, rows, heads):
    """More rows than one co-resident grid has CTAs: warps stride over all (row, head) pairs
    (`bq_gated_rmsnorm_scale`), then the cast pass; bit-identical to the torch spelling."""
    width = heads * 128
    y = randn_cpu((rows, heads, 128), seed=rows, dtype=ydt, scale=2.0).cuda()
    z = randn_cpu((rows, width), seed=rows + 1, scale=1.5).cuda()
    gamma = _gamma(128, 3, spread=0.3)
    ref = TS.rms_norm_gated(y.to(z.dtype).reshape(-1, 128), z.reshape(-1, 128), gamma, EPS).reshape(rows, width)
    calls = Q.launch_count()
    qa = Q.gated_rms_norm_quant(y, z, gamma, EPS, 128)
    assert Q.launch_count() - calls == 2
    _same(qa, ref, f"{ydt} {rows}x{heads}")
    assert Q.device_status() == 0


def test_consumers_take_the_quantized_activation(Q):
    """`project`, `linear` and the MLP on a pre-quantized activation equal the reference order of
    operations (norm, then the consumer quantizes) bit for bit, bf16 weights in the mix included."""
    H, I = 4096, 12288
    x = randn_cpu((16, 1, H), seed=11).cuda()
    gamma = _gamma(H, 12)
    mk = lambda n, k, s: Q.quantize_weight((randn_cpu((n, k), seed=s, scale=0.02)).cuda())  # noqa: E731
    w_qkv, w_z, w_out = mk(8192, H, 13), mk(4096, H, 14), mk(H, 4096, 15)
    w_a = randn_cpu((32, H), seed=16, scale=0.02).cuda()
    h = TS.rms_norm(x, gamma, EPS)
    want = Q.project(h, w_qkv, w_z, w_a)
    got = Q.project(Q.rms_norm_quant(x, gamma, EPS, keep_dense=True), w_qkv, w_z, w_a)
    for a, b in zip(got, want):
        assert a.shape == b.shape and torch.equal(a, b)
    with pytest.raises(ValueError):
        Q.project(Q.rms_norm_quant(x, gamma, EPS), w_qkv, w_a)       # bf16 weight needs the dense form
    assert torch.equal(Q.linear(Q.rms_norm_quant(x, gamma, EPS), w_z), Q.linear(h, w_z))
    wg, wu, wd = mk(I, H, 17), mk(I, H, 18), mk(H, I, 19)
    assert torch.equal(Q.mlp_forward(Q.rms_norm_quant(x, gamma, EPS), wg, wu, wd),
                       Q.mlp_forward(h, wg, wu, wd))
    # GDN readout: gated norm feeding out_proj
    y = randn_cpu((16, 32, 128), seed=20, dtype=torch.float32).cuda()
    z = randn_cpu((16, 1, 4096), seed=21).cuda()
    g128 = _gamma(128, 22)
    core = TS.rms_norm_gated(y.to(torch.bfloat16).reshape(-1, 128), z.reshape(-1, 128), g128, EPS)
    want = Q.linear(core.reshape(16, 1, 4096), w_out)
    got = Q.linear(Q.gated_rms_norm_quant(y, z, g128, EPS, 128), w_out)
    assert got.shape == want.shape and torch.equal(got, want)


def test_norm_quant_survives_capture_and_replays_identically(Q):
    x = randn_cpu((128, 4096), seed=30).cuda()
    gamma = _gamma(4096, 31)
    y = randn_cpu((128, 32, 128), seed=32, dtype=torch.float32).cuda()
    z = randn_cpu((128, 4096), seed=33).cuda()
    g128 = _gamma(128, 34)

    def step():
        a = Q.rms_norm_quant(x, gamma, EPS, keep_dense=True)
        b = Q.gated_rms_norm_quant(y, z, g128, EPS, 128)
        return a.q, a.scale, a.dense, b.q, b.scale

    eager = [t.clone() for t in step()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for e, r in zip(eager, outs):
        assert torch.equal(u8(e), u8(r))
    assert Q.device_status() == 0
