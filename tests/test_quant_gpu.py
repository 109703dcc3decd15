"""The sm_100a quantizer against the reference's torch spelling on the same device (bit identity),
against the CPU oracle, and against the committed golden vectors.  Mirrors the reference's own
gates (tests/test_quant.py:65-70, :146-152, :371-477) and widens them."""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import torch_spelling as TS
from _util import codes_np, f32_bits, from_bits16, randn_cpu, to_np_f32, u8

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float32, torch.float16]
DT_IDS = ["bf16", "fp32", "fp16"]


def _assert_same(q, s, qr, sr, what=""):
    assert torch.equal(s, sr), f"{what} scale differs: {s.item():.9e} vs {sr.item():.9e}"
    diff = int((u8(q) != u8(qr)).sum())
    assert diff == 0, f"{what}: {diff} of {q.numel()} fp8 bytes differ"


@pytest.mark.parametrize("dt", DTYPES, ids=DT_IDS)
@pytest.mark.parametrize("shape", [(1, 4096), (8, 4096), (37, 12288), (128, 12288)],
                         ids=["m1", "m8", "m37", "m128"])
def test_bit_identical_to_the_torch_spelling(Q, dt, shape):
    """The reference's own gate, same generator and seed (tests/test_quant.py:387-401)."""
    g = torch.Generator(device="cuda").manual_seed(17)
    x = (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * 3.5).to(dt)
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    assert q.dtype is Q.FP8 and q.shape == x.shape
    assert s.shape == (1, 1) and s.dtype is torch.float32 and s.is_cuda
    _assert_same(q, s, qr, sr, f"{dt} {shape}")


@pytest.mark.parametrize("shape", [(1, 8), (1, 1), (3, 100), (5, 7), (16, 4096), (64, 4096),
                                   (128, 4096), (333, 12288), (2048, 4096), (8192, 4096)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_ragged_small_and_streaming_sizes(Q, shape, dt):
    """Tails that are not a multiple of 8, single-CTA grids, the register-held regime and the
    streaming regime (8192x4096 = BASELINE's prefill activation)."""
    x = randn_cpu(shape, seed=shape[0] * 31 + shape[1], dtype=dt, scale=2.0).cuda()
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    _assert_same(q, s, qr, sr, f"{dt} {shape}")


@pytest.mark.parametrize("dt,n", [(torch.bfloat16, 4_850_000 + 4099), (torch.bfloat16, 9_000_001),
                                  (torch.bfloat16, 20_000_003), (torch.bfloat16, 296 * 3 * 16384 + 8),
                                  (torch.bfloat16, 296 * 4 * 16384), (torch.float16, 7_777_777),
                                  (torch.float32, 2_500_001), (torch.float32, 9_000_005)],
                         ids=["bf16-8KB-chunks", "bf16-16KB-chunks", "bf16-refetch", "bf16-ring-full+1",
                              "bf16-4-each", "fp16", "fp32-resident", "fp32-refetch"])
def test_ragged_sizes_through_the_shared_memory_ring(Q, dt, n):
    """Plain quantizer beyond the register-held regime: a ring of bulk copies per CTA (96 KB;
    chunks of 8, 16 or 32 KB by input size).  Sizes where every chunk of a CTA stays in the ring
    between the passes, where chunks are fetched again, where the ring is exactly full (three
    32 KB chunks per CTA on 148 SMs), a short last chunk and a tail that is no whole group;
    the cast half alone at the same sizes; and the register-fed streaming kernel on the same
    input (option `quant_ring` off) gives the same bits."""
    x = randn_cpu((n,), seed=n % 1000, dtype=dt, scale=1.7).cuda()
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    _assert_same(q, s, qr, sr, f"{dt} {n}")
    qc = Q.cast_act(x, sr)
    assert torch.equal(u8(qc).reshape(-1), u8(qr).reshape(-1))
    try:
        Q.set_option("quant_ring", 0)
        q0, s0 = Q.quantize_act(x)
        qc0 = Q.cast_act(x, sr)
    finally:
        Q.set_option("quant_ring", 1)
    _assert_same(q0, s0, qr, sr, f"register-fed {dt} {n}")
    assert torch.equal(u8(qc0).reshape(-1), u8(qr).reshape(-1))
    assert Q.device_status() == 0


@pytest.mark.parametrize("cols", [4096, 12288])
def test_config_4_activations_on_the_streaming_kernel(Q, cols):
    """BASELINE config 4: 16 packed sequences (M ~ 8192 rows) of width 4096 (layer input) and
    12288 (MLP intermediate), far beyond what one co-resident grid can hold in registers."""
    g = torch.Generator().manual_seed(4)
    M = int(torch.randint(64, 1025, (16,), generator=g).sum())
    x = randn_cpu((M, cols), seed=cols).cuda()
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    _assert_same(q, s, qr, sr, f"{M}x{cols}")
    if cols == 12288:
        gu = randn_cpu((M, 2 * cols), seed=7, scale=2.0).cuda()
        q, s = Q.silu_mul_quant(gu[:, :cols], gu[:, cols:])
        qr, sr = TS.quantize_act(TS.silu_mul(gu[:, :cols], gu[:, cols:]))
        _assert_same(q, s, qr, sr, "silu_mul prologue at prefill size")
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", DTYPES, ids=DT_IDS)
@pytest.mark.parametrize("shape", [(1, 64), (37, 1536), (128, 12288), (4096, 1536)])
def test_scale_and_cast_halves_equal_the_whole_quantizer(Q, dt, shape):
    """`silu_mul_scale` + `silu_mul_cast` (the column-parallel MLP's exchange) against
    `silu_mul_quant`; and a shard cast under the scale of the whole tensor equals the matching
    columns of the whole tensor's codes."""
    M, I = shape
    gu = randn_cpu((M, 2 * I), seed=M + I, dtype=dt, scale=2.0).cuda()
    g_, u_ = gu[:, :I], gu[:, I:]
    q, s = Q.silu_mul_quant(g_, u_)
    s2 = Q.silu_mul_scale(g_, u_)
    assert torch.equal(s, s2)
    assert torch.equal(u8(Q.silu_mul_cast(g_, u_, s2)), u8(q))
    if I % 32 == 0:
        half = I // 2
        shards = [(g_[:, :half], u_[:, :half]), (g_[:, half:], u_[:, half:])]
        scales = torch.stack([Q.silu_mul_scale(a, b) for a, b in shards])
        smax = scales.max().reshape(1, 1)
        assert torch.equal(smax, s)
        parts = [Q.silu_mul_cast(a, b, smax) for a, b in shards]
        assert torch.equal(u8(torch.cat(parts, dim=1)), u8(q))
    assert Q.device_status() == 0


@pytest.mark.parametrize("shape", [(8, 4096), (37, 12288)])
def test_matches_the_cpu_oracle_with_the_cuda_scale_spelling(Q, shape):
    x = randn_cpu(shape, seed=5, scale=3.5)
    q, s = Q.quantize_act(x.cuda())
    qo, so = oracle.quantize(to_np_f32(x), oracle.SCALE_RCP)
    assert f32_bits(s) == int(np.float32(so).view(np.uint32))
    assert np.array_equal(codes_np(q), qo)


def test_every_bf16_value_through_the_cast(Q):
    """All finite bf16 patterns with |x| <= 448: amax is 448, the scale exactly 1.0."""
    bits = np.arange(65536, dtype=np.uint16)
    x = from_bits16(bits)
    keep = torch.isfinite(x.float()) & (x.float().abs() <= 448.0)
    x = x[keep].contiguous().cuda()
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    _assert_same(q, s, qr, sr, "all bf16")
    assert np.array_equal(codes_np(q), oracle.cast(to_np_f32(x), np.float32(s.item())))


def _code_mismatches(q, want):
    """Indices where two e4m3 code tensors differ; two NaN codes (0x7F, 0xFF) count as equal."""
    a, b = u8(q).reshape(-1), u8(want).reshape(-1)
    both_nan = ((a & 0x7F) == 0x7F) & ((b & 0x7F) == 0x7F)
    return ((a != b) & ~both_nan).nonzero().reshape(-1)


def _division_scales():
    """Scales that stress a division done with one rounded reciprocal: random mantissas over the
    exponents activations produce, mantissas of all ones and 1 + 1 ulp (where 1/scale rounds
    worst), powers of two, the reference's floor 1e-12, both ends of the range the kernel takes
    with the reciprocal, values beyond it (the division instruction), infinity."""
    rng = np.random.default_rng(2024)
    mant = rng.integers(0, 1 << 23, size=160, dtype=np.uint32)
    expo = rng.integers(127 - 45, 127 + 20, size=160, dtype=np.uint32)
    bits = list((expo << 23) | mant)
    for e in (127 - 40, 127 - 7, 127, 127 + 5):
        bits += [(e << 23) | 0x7FFFFF, (e << 23) | 1, (e << 23) | 0x7FFFFE, e << 23,
                 (e << 23) | 0x400000, (e << 23) | 0x555555, (e << 23) | 0x2AAAAB]
    vals = list(np.array(bits, dtype=np.uint32).view(np.float32))
    vals += [np.float32(v) for v in (1e-12, 2.0 ** -60, np.nextafter(np.float32(2.0 ** -60), np.float32(0)),
                                      2.0 ** 60, np.nextafter(np.float32(2.0 ** 60), np.float32(np.inf)),
                                      1e-30, 3e35, 3.0, 1.0 / 3.0, np.inf)]
    return vals


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_cast_under_a_shared_scale_is_the_ieee_division_for_every_16_bit_value(Q, dt):
    """The cast divides by a scale all elements share through one rounded reciprocal and two
    residual corrections; the codes must be those of the IEEE division the reference spells
    (braid/model/quant.py:113) for every one of the 65536 bit patterns (NaN, infinities,
    subnormals and -0 included) under every scale of the list."""
    x = torch.arange(-32768, 32768, dtype=torch.int16).view(dt).cuda()
    for sv in _division_scales():
        scale = torch.full((1, 1), float(sv), dtype=torch.float32, device="cuda")
        q = Q.cast_act(x, scale)
        want = (x.float() / scale).reshape(-1).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(Q.FP8)
        bad = _code_mismatches(q, want)
        assert bad.numel() == 0, (f"scale {float(sv)!r}: {bad.numel()} codes differ, first at bits "
                                  f"{int(x.view(torch.int16)[bad[0]]) & 0xFFFF:#06x}")
    # the oracle's cast agrees with the device's division on a sample of the same grid
    sv = np.float32(0.0123456)
    q = Q.cast_act(x, torch.full((1, 1), float(sv), dtype=torch.float32, device="cuda"))
    fin = torch.isfinite(x.float()).cpu().numpy()
    assert np.array_equal(codes_np(q)[fin], oracle.cast(to_np_f32(x.cpu()), sv)[fin])


def test_cast_of_fp32_values_under_a_shared_scale_is_the_ieee_division(Q):
    """fp32 activations: 2^22 random bit patterns per scale (any exponent, any mantissa)."""
    g = torch.Generator(device="cuda").manual_seed(99)
    bits = torch.randint(-2 ** 31, 2 ** 31 - 1, (1 << 22,), generator=g, device="cuda", dtype=torch.int64)
    x = bits.to(torch.int32).view(torch.float32)
    near = (torch.randn(1 << 22, generator=g, device="cuda") * 3.0)
    for sv in _division_scales()[::5]:
        scale = torch.full((1, 1), float(sv), dtype=torch.float32, device="cuda")
        for t in (x, near * float(sv) if np.isfinite(sv) else near):
            q = Q.cast_act(t, scale)
            want = (t / scale).reshape(-1).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(Q.FP8)
            diff = _code_mismatches(q, want).numel()
            assert diff == 0, f"scale {float(sv)!r}: {diff} codes differ"


def test_golden_vectors_with_the_device_scale(Q, golden):
    """Golden inputs from the reference's CPU run: codes must equal the oracle cast at the scale
    the device computed, and the scale must be the CUDA spelling of the same amax."""
    for key in ("act_bf16_8x4096", "act_bf16_1x4096"):
        x = from_bits16(golden[key + "_x"])
        q, s = Q.quantize_act(x.cuda())
        want_s = oracle.scale_from_amax(oracle.amax(to_np_f32(x)), oracle.SCALE_RCP)
        assert f32_bits(s) == int(want_s.view(np.uint32))
        assert np.array_equal(codes_np(q), oracle.cast(to_np_f32(x), want_s))
        if int(want_s.view(np.uint32)) == int(golden[key + "_scale"].reshape(-1)[0]):
            assert np.array_equal(codes_np(q), golden[key + "_q"])


def test_degenerate_scales(Q):
    for label, fill in (("zeros", 0.0), ("huge", 60000.0), ("tiny", 1e-10)):
        x = torch.full((4, 4096), fill, device="cuda", dtype=torch.bfloat16)
        q, s = Q.quantize_act(x)
        qr, sr = TS.quantize_act(x)
        assert torch.isfinite(s).all(), f"{label}: scale not finite"
        _assert_same(q, s, qr, sr, label)


def test_full_range_is_used(Q):
    x = torch.randn(16, 256, device="cuda", dtype=torch.bfloat16)
    xq, sx = Q.quantize_act(x)
    assert xq.dtype is Q.FP8 and sx.shape == (1, 1)
    assert xq.float().abs().max().item() > Q.FP8_MAX * 0.5


def test_non_contiguous_activation_takes_the_exact_torch_arm(Q):
    base = randn_cpu((64, 4096), seed=5).cuda()
    view = base.t()
    assert not view.is_contiguous()
    q, s = Q.quantize_act(view)
    qc, sc = Q.quantize_act(view.contiguous())
    _assert_same(q, s, qc, sc, "strided")


def test_nan_survives(Q):
    x = randn_cpu((4, 4096), seed=3).cuda()
    x[2, 100] = float("nan")
    q, s = Q.quantize_act(x)
    qr, sr = TS.quantize_act(x)
    assert torch.isnan(s).all() and torch.isnan(sr).all()
    assert torch.equal(u8(q), u8(qr))


def test_warm_fused_switch_selects_the_torch_arm(Q):
    x = randn_cpu((8, 4096), seed=9).cuda()
    fused = Q.quantize_act(x)
    assert Q.fused_state() == "active"
    Q.warm_fused(False)
    try:
        assert Q.fused_state() == "disabled by caller"
        ref = Q.quantize_act(x)
    finally:
        Q.warm_fused(True)
    _assert_same(*fused, *ref, "switch")


def test_back_to_back_calls_leave_the_scratch_clean(Q):
    """The barrier words return to zero: 600 calls (more than the slot pool) stay exact."""
    x = randn_cpu((128, 4096), seed=1).cuda()
    qr, sr = TS.quantize_act(x)
    for _ in range(600):
        q, s = Q.quantize_act(x)
    _assert_same(q, s, qr, sr, "repeat")
    assert Q.device_status() == 0


# ---- prologues ---------------------------------------------------------------------------

@pytest.mark.parametrize("dt", DTYPES, ids=DT_IDS)
@pytest.mark.parametrize("shape", [(1, 12288), (8, 12288), (37, 256), (128, 12288), (512, 12288)])
def test_silu_mul_quant_is_bit_identical(Q, dt, shape):
    gate = randn_cpu(shape, seed=41, dtype=dt, scale=2.0).cuda()
    up = randn_cpu(shape, seed=42, dtype=dt, scale=1.5).cuda()
    q, s = Q.silu_mul_quant(gate, up)
    qr, sr = TS.quantize_act(TS.silu_mul(gate, up))
    _assert_same(q, s, qr, sr, f"silu {dt} {shape}")


def test_silu_mul_quant_reads_column_blocks_in_place(Q):
    """gate and up as the two halves of one [M, 2I] buffer, the layout the grouped GEMM writes."""
    M, I = 16, 1024
    gu = randn_cpu((M, 2 * I), seed=43, scale=2.0).cuda()
    q, s = Q.silu_mul_quant(gu[:, :I], gu[:, I:])
    qr, sr = TS.quantize_act(TS.silu_mul(gu[:, :I].contiguous(), gu[:, I:].contiguous()))
    _assert_same(q, s, qr, sr, "column blocks")


@pytest.mark.parametrize("dt", DTYPES, ids=DT_IDS)
def test_sigmoid_gate_quant_dense_and_per_head_view(Q, dt):
    B, T, H, D = 2, 5, 16, 256
    qg = randn_cpu((B, T, H * 2 * D), seed=44, dtype=dt, scale=2.0).cuda()
    o = randn_cpu((B, T, H * D), seed=45, dtype=dt).cuda()
    _, gate_v = qg.view(B, T, H, 2 * D).chunk(2, dim=-1)        # strided, as in the attention layer
    gate_dense = gate_v.reshape(B, T, H * D)
    qr, sr = TS.quantize_act(TS.sigmoid_gate(o, gate_dense))
    q1, s1 = Q.sigmoid_gate_quant(o, gate_dense)
    _assert_same(q1, s1, qr, sr, "dense gate")
    q2, s2 = Q.sigmoid_gate_quant(o, gate_v)
    _assert_same(q2, s2, qr, sr, "per-head view")
    assert q2.shape == o.shape


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_silu_and_sigmoid_of_every_16_bit_value(Q, dt):
    """The prologues' silu and sigmoid, seen through the dense forms: the result has to be
    torch's (`F.silu(gate) * up`, braid/model/mlp.py:48; `o * torch.sigmoid(gate)`,
    braid/model/attention.py:215) for every one of the 65536 gate bit patterns, NaN and
    infinities included, under several partners."""
    gate = torch.arange(-32768, 32768, dtype=torch.int16).view(dt).cuda().reshape(64, 1024)
    for partner in (1.0, -3.71875, 0.0009765625, 250.0):
        other = torch.full_like(gate, partner)
        for got, want in ((Q.silu_mul(gate, other), F.silu(gate) * other),
                          (Q.sigmoid_mul(other, gate), other * torch.sigmoid(gate))):
            a, b = got.view(torch.int16), want.view(torch.int16)
            both_nan = torch.isnan(got) & torch.isnan(want)
            bad = ((a != b) & ~both_nan).nonzero()
            assert bad.numel() == 0, (f"{dt} partner {partner}: {bad.shape[0]} values differ, first at gate "
                                      f"bits {int(gate.view(torch.int16)[tuple(bad[0])]) & 0xFFFF:#06x}")
    # random partners: the second rounding sees every first-rounding outcome
    g = torch.Generator(device="cuda").manual_seed(8)
    up = (torch.randn(64, 1024, generator=g, device="cuda") * 2.0).to(dt)
    assert torch.equal(Q.silu_mul(gate, up).view(torch.int16)[~torch.isnan(gate)],
                       (F.silu(gate) * up).view(torch.int16)[~torch.isnan(gate)])


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_prologue_quantizers_at_prefill_sizes_take_two_launches(Q, dt):
    """From 2^22 elements on, SiLU*mul and the sigmoid gate run as product + scale (no grid-wide
    wait) followed by the cast pass; same bits as the torch spelling, column blocks and the
    per-head gate view read in place, NaN carried."""
    M, I = 2100, 2048
    gu = randn_cpu((M, 2 * I), seed=51, dtype=dt, scale=2.0).cuda()
    calls = Q.launch_count()
    q, s = Q.silu_mul_quant(gu[:, :I], gu[:, I:])
    assert Q.launch_count() - calls == 2
    qr, sr = TS.quantize_act(TS.silu_mul(gu[:, :I].contiguous(), gu[:, I:].contiguous()))
    _assert_same(q, s, qr, sr, f"silu two-launch {dt}")
    B, T, H, D = 2, 1100, 16, 128
    qg = randn_cpu((B, T, H * 2 * D), seed=52, dtype=dt, scale=2.0).cuda()
    o = randn_cpu((B, T, H * D), seed=53, dtype=dt).cuda()
    _, gate_v = qg.view(B, T, H, 2 * D).chunk(2, dim=-1)
    qr, sr = TS.quantize_act(TS.sigmoid_gate(o, gate_v.reshape(B, T, H * D)))
    calls = Q.launch_count()
    q2, s2 = Q.sigmoid_gate_quant(o, gate_v)
    assert Q.launch_count() - calls == 2
    _assert_same(q2, s2, qr, sr, f"sigmoid two-launch {dt}")
    o[1, 7, 3] = float("nan")
    q3, s3 = Q.sigmoid_gate_quant(o, gate_v)
    assert torch.isnan(s3).all()
    assert Q.device_status() == 0


def test_dense_prologues_in_fp32_and_on_column_blocks(Q):
    x = randn_cpu((33, 2 * 512), seed=12, dtype=torch.float32, scale=3.0).cuda()
    assert torch.equal(Q.silu_mul(x[:, :512], x[:, 512:]), F.silu(x[:, :512]) * x[:, 512:])
    assert torch.equal(Q.sigmoid_mul(x[:, :512].contiguous(), x[:, 512:].contiguous()),
                       x[:, :512] * torch.sigmoid(x[:, 512:]))
    xb = x.to(torch.bfloat16)
    assert torch.equal(Q.silu_mul(xb[:, :512], xb[:, 512:]), F.silu(xb[:, :512]) * xb[:, 512:])


def test_prologues_against_the_golden_vectors(Q, golden):
    """Inputs and outputs of the reference's CPU run.  The device evaluates expf with its own
    library, so agreement with the CPU codes is near-total rather than exact; the bit-exact
    arbiter is the torch-on-device comparison above."""
    gate, up = from_bits16(golden["mlp_gate"]).cuda(), from_bits16(golden["mlp_up"]).cuda()
    q, s = Q.silu_mul_quant(gate, up)
    want = golden["mlp_hq"]
    assert (codes_np(q) != want).mean() < 0.02
    H, D = 4, 64
    qg = from_bits16(golden["sig_qg"]).view(2, 3, H, 2 * D).cuda()
    o = from_bits16(golden["sig_o"]).view(2, 3, H * D).cuda()
    q, s = Q.sigmoid_gate_quant(o, qg[..., D:])
    assert (codes_np(q).reshape(6, H * D) != golden["sig_oq"].reshape(6, H * D)).mean() < 0.02


def test_bad_arguments_raise(Q):
    with pytest.raises(ValueError):
        Q.quantize_act(torch.zeros(4, 8, device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError):
        Q.quantize_act(torch.zeros(0, 8, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        Q.quantize_act(torch.zeros(4, 8, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        Q.silu_mul_quant(torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16),
                         torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16))
    assert Q.device_status() == 0
