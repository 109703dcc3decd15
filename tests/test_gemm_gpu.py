"""The tcgen05 W8A8 GEMM against the CPU oracle (exact dequantize-and-multiply), the library GEMM
the reference calls (`torch._scaled_mm`), the golden vectors, and its own structural properties:
determinism, split-K invariance within tolerance, grouped == separate, untouched canaries.

Tolerance (BASELINE): max|y - ref| / max|ref| <= 1e-2 on bf16 outputs against an fp32
dequant-matmul; fp32 outputs are held to 1e-4."""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import torch_spelling as TS
from _util import codes_np, config1_inputs, from_bits16, from_bits32, max_rel, randn_cpu

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
TOL_F32 = 1e-4


def _operands(Q, M, N, K, seed=0):
    x = randn_cpu((M, K), seed=seed).cuda()
    w = randn_cpu((N, K), seed=seed + 1, scale=0.02).cuda()
    fw = Q.quantize_weight(w)
    xq, sx = Q.quantize_act(x)
    return x, w, xq, sx, fw


def _oracle(xq, sx, fw):
    return torch.from_numpy(oracle.gemm(codes_np(xq), codes_np(fw.data), sx.item(), fw.scale.item()))


@pytest.mark.parametrize("M", [1, 7, 8, 16, 37, 128, 200, 256])
@pytest.mark.parametrize("N,K", [(16, 16), (128, 128), (512, 256), (1040, 272), (4096, 4096)])
def test_decode_regime_against_the_oracle(Q, M, N, K):
    if N * K * M > 4096 * 4096 * 37 and M not in (37, 128):
        pytest.skip("oracle time")
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=M + N)
    y = Q.fp8_matmul(xq, sx, fw)
    assert y.shape == (M, N) and y.dtype is torch.bfloat16
    ref = _oracle(xq, sx, fw)
    assert max_rel(y.cpu(), ref) <= TOL_BF16
    y32 = Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32)
    assert max_rel(y32.cpu(), ref) <= TOL_F32
    assert Q.last_gemm_launch()["kernel"] == "stream"


@pytest.mark.parametrize("M,N,K", [(257, 256, 256), (512, 4096, 4096), (1000, 272, 4096),
                                   (2048, 1024, 128), (2048, 4096, 4096), (4100, 512, 1040)])
def test_prefill_regime_against_fp32_dequant_matmul(Q, M, N, K):
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=M)
    y = Q.fp8_matmul(xq, sx, fw)
    assert Q.last_gemm_launch()["kernel"] in ("tile", "pair")
    ref = TS.dequant_matmul(xq, sx, fw.data, fw.scale)
    assert max_rel(y, ref) <= TOL_BF16
    y32 = Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32)
    assert max_rel(y32, ref) <= TOL_F32
    if M * N * K <= 512 * 4096 * 4096:
        sub = slice(0, M, max(1, M // 16))
        ref_o = torch.from_numpy(oracle.gemm(codes_np(xq[sub]), codes_np(fw.data),
                                             sx.item(), fw.scale.item()))
        assert max_rel(y32[sub].cpu(), ref_o) <= TOL_F32


def ragged_pack_rows(seed: int = 4) -> tuple[list[int], int]:
    """BASELINE config 4: 16 sequence lengths ~U[64, 1024] (seeded), packed into one row block."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(64, 1025, (16,), generator=g).tolist()
    return lens, int(sum(lens))


CONFIG4_GROUPS = {          # the projection groups of the 9B-class stack (one launch each)
    "mlp.gate_up": ((12288, 12288), 4096),
    "gdn.qkv_z": ((8192, 4096), 4096),
    "mlp.down": ((4096,), 12288),
    "gdn.out_proj": ((4096,), 4096),
    "attn.qkv": ((8192, 1024, 1024), 4096),
}


@pytest.mark.parametrize("name", list(CONFIG4_GROUPS))
def test_config_4_ragged_prefill_at_full_size(Q, name):
    """Chunked ragged prefill at BASELINE's size: 16 packed sequences (M ~ 8192 rows, not a
    multiple of any tile) against the exact fp32 dequantize-and-multiply on the device over the
    whole output, and against the CPU oracle on a strided subsample of rows and columns that
    visits every tile row and tile column of the launch."""
    Ns, K = CONFIG4_GROUPS[name]
    lens, M = ragged_pack_rows()
    assert len(lens) == 16 and 16 * 64 <= M <= 16 * 1024
    x = randn_cpu((M, K), seed=41).cuda()
    ws = [Q.quantize_weight(randn_cpu((n, K), seed=42 + i, scale=0.02).cuda()) for i, n in enumerate(Ns)]
    xq, sx = Q.quantize_act(x)
    ys = Q.fp8_matmul_grouped(xq, sx, ws)
    assert Q.last_gemm_launch()["kernel"] in ("pair", "tile")
    ys32 = Q.fp8_matmul_grouped(xq, sx, ws, out_dtype=torch.float32)
    rows = torch.arange(0, M, 61, device="cuda")
    for y, y32, w in zip(ys, ys32, ws):
        ref = TS.dequant_matmul(xq, sx, w.data, w.scale)
        assert max_rel(y, ref) <= TOL_BF16
        assert max_rel(y32, ref) <= TOL_F32
        del ref
        cols = torch.arange(0, w.shape[0], 37, device="cuda")
        ref_o = torch.from_numpy(oracle.gemm(codes_np(xq[rows]), codes_np(w.data[cols]),
                                             sx.item(), w.scale.item()))
        assert max_rel(y32[rows][:, cols].cpu(), ref_o) <= TOL_F32
    # a row of the product does not depend on which rows share its launch: the packed call equals
    # the per-sequence calls (the reference pads sequences to rectangles instead of packing them)
    lo = sum(lens[:5])
    part = Q.fp8_matmul_grouped(xq[lo:lo + lens[5]].contiguous(), sx, ws, out_dtype=torch.float32)
    for y32, yp in zip(ys32, part):
        assert max_rel(yp, y32[lo:lo + lens[5]]) <= 1e-6
    assert Q.device_status() == 0


@pytest.mark.parametrize("M", [1, 128])
def test_lm_head_at_full_vocabulary(Q, M):
    """The `head` group's weight (braid/model/engine.py:348-349): 248,320 x 4096, 1,940 row tiles
    of the weight-streaming kernel in one launch.  Whole output against the library GEMM the
    reference calls; a strided subsample of the vocabulary against the CPU oracle."""
    V, K = 248320, 4096
    g = torch.Generator(device="cuda").manual_seed(43)
    w = (torch.randn(V, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    fw = Q.quantize_weight(w)
    del w
    x = randn_cpu((M, K), seed=44).cuda()
    xq, sx = Q.quantize_act(x)
    y = Q.fp8_matmul(xq, sx, fw)
    assert y.shape == (M, V) and Q.last_gemm_launch()["kernel"] == "stream"
    ref = TS.scaled_mm(xq, sx, fw.data, fw.scale)
    assert max_rel(y, ref) <= TOL_BF16
    assert (y != ref).float().mean().item() < 0.05
    y32 = Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32)
    cols = torch.arange(0, V, 251, device="cuda")
    ref_o = torch.from_numpy(oracle.gemm(codes_np(xq), codes_np(fw.data[cols]), sx.item(),
                                         fw.scale.item()))
    assert max_rel(y32[:, cols].cpu(), ref_o) <= TOL_F32
    assert torch.equal(y, Q.fp8_matmul(xq, sx, fw))            # run-to-run identical
    assert Q.device_status() == 0


@pytest.mark.parametrize("M,N,K,dt", [(4096, 512, 12288, torch.bfloat16), (1000, 1040, 4096, torch.bfloat16),
                                      (300, 144, 512, torch.float32), (2048, 4096, 4096, torch.bfloat16),
                                      (768, 4096, 512, torch.bfloat16)],
                         ids=["down-shard-of-8", "ragged", "tiny-fp32", "wide-weight", "two-rounds-if-narrow"])
def test_prefill_tiles_of_128_columns_give_the_bits_of_256(Q, M, N, K, dt):
    """A lone narrow weight at prefill sizes is tiled 256 x 128 instead of 256 x 256 so that more
    CTA pairs have work; every output element is the same sum in the same order either way."""
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=M + N)
    try:
        Q.set_option("pair_narrow", 0)
        wide = Q.fp8_matmul(xq, sx, fw, out_dtype=dt)
        assert Q.last_gemm_launch()["mma_n"] == 256
        Q.set_option("pair_narrow", 1)
        narrow = Q.fp8_matmul(xq, sx, fw, out_dtype=dt)
        assert Q.last_gemm_launch()["mma_n"] == 128
    finally:
        Q.set_option("pair_narrow", -1)
    assert torch.equal(wide, narrow)
    auto = Q.fp8_matmul(xq, sx, fw, out_dtype=dt)
    tiles_wide = -(-N // 256) * -(-M // 256)
    assert Q.last_gemm_launch()["mma_n"] == (128 if tiles_wide * 2 <= 74 else 256)
    assert torch.equal(auto, wide)
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("M,V,K", [(1, 248320, 4096), (128, 248320, 4096), (37, 1040, 272),
                                   (4, 4096, 256), (256, 16, 16)])
def test_lm_head_argmax_equals_argmax_of_the_logits(Q, dt, M, V, K):
    """braid/model/engine.py:349 + braid/serve/scheduler.py:346: the greedy token of every row,
    taken in the GEMM's epilogue, equals `linear(h, lm_head).argmax(-1)` exactly -- ties between
    equal logits (bf16 rounding makes them common, and duplicated vocabulary rows force them)
    go to the lowest index; the logits, when asked for, are the plain GEMM's bits."""
    if dt is not torch.bfloat16 and V > 5000:
        pytest.skip("dtype variants on the small shapes")
    g = torch.Generator(device="cuda").manual_seed(V + M)
    w = (torch.randn(V, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    fw = Q.quantize_weight(w)
    del w
    if V >= 1040:      # duplicated rows: exact ties far apart in the vocabulary (different tiles)
        codes = fw.data.view(torch.uint8)
        codes[V - 7] = codes[3]
        codes[V // 2 + 1] = codes[V // 2 - 300]
    x = randn_cpu((M, K), seed=M + K, dtype=dt).cuda()
    if V >= 1040:      # make the duplicated rows the winners of two batch rows
        lut = fw.data[3].to(dt)
        x[0] = lut * 8
        if M > 1:
            x[M - 1] = fw.data[V // 2 - 300].to(dt) * 8
    want_logits = Q.linear(x, fw)
    want = want_logits.argmax(-1)
    n0 = Q.launch_count()
    got = Q.lm_head_argmax(x, fw)
    assert Q.launch_count() - n0 == 3                # quantizer, GEMM with the pick, tiny reduction
    assert got.dtype is torch.int64 and got.shape == (M,)
    assert torch.equal(got, want), (got[:4], want[:4])
    if V >= 1040:
        assert int(got[0]) == 3                       # the lower of the two tied indices
    idx2, logits = Q.lm_head_argmax(x, fw, return_logits=True)
    assert torch.equal(idx2, want) and torch.equal(logits, want_logits)
    # a NaN in a row makes every logit of that row NaN: index 0, as torch picks
    if M >= 4:
        x[2, 5] = float("nan")
        assert torch.equal(Q.lm_head_argmax(x, fw), Q.linear(x, fw).argmax(-1))
    # leading dims and a tensor that carries its quantization
    x3 = x.reshape(M, 1, K)
    assert Q.lm_head_argmax(x3, fw).shape == (M, 1)
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
def test_prefill_store_paths_agree_and_stay_in_bounds(Q, dt):
    """The prefill epilogue hands 128-byte row pieces to TMA stores when the output can be
    described to TMA (16-byte aligned base and row pitch) and writes the same staged pieces with
    plain coalesced stores otherwise: same bits either way, ragged M and N clipped, nothing
    outside the output touched."""
    M, N, K = 1000, 4096 + 16, 1040
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=77)
    want = Q.fp8_matmul(xq, sx, fw, out_dtype=dt)                 # contiguous: the TMA path
    assert Q.last_gemm_launch()["kernel"] == "pair"
    ref = TS.dequant_matmul(xq, sx, fw.data, fw.scale)
    assert max_rel(want, ref) <= (TOL_F32 if dt is torch.float32 else TOL_BF16)
    # 16-bit outputs: a pitch of N + 4 elements is 8-byte but not 16-byte aligned (plain stores);
    # fp32 outputs must be 16-byte aligned anyway, so every legal one takes the TMA path
    for off, pitch in ((0, N + 4), (4, N + 4), (8, N + 24)):
        big = torch.full((M + 2, pitch + 16), 7.0, device="cuda", dtype=dt)
        out = big[1:M + 1, off:off + N]
        Q.fp8_matmul_grouped(xq, sx, (fw,), out_dtype=dt, out=(out,))
        assert torch.equal(out, want), (off, pitch)
        mask = torch.ones_like(big, dtype=torch.bool)
        mask[1:M + 1, off:off + N] = False
        assert (big[mask] == 7.0).all(), (off, pitch)
    assert Q.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (128, 4096, 4096), (128, 1024, 4096),
                                   (64, 4096, 12288), (2048, 4096, 4096)])
def test_agrees_with_the_library_gemm_the_reference_calls(Q, M, N, K):
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=3)
    y = Q.fp8_matmul(xq, sx, fw)
    ref = TS.scaled_mm(xq, sx, fw.data, fw.scale)
    assert max_rel(y, ref) <= TOL_BF16
    # both round the same fp32 sums to bf16: almost every element is bit-equal
    assert (y != ref).float().mean().item() < 0.05


def test_config_1_against_the_reference_cpu_output(Q, golden):
    import hashlib
    x, w = config1_inputs(0)
    sha = lambda t: np.frombuffer(hashlib.sha256(t.view(torch.uint8).numpy().tobytes()).digest(), np.uint8)
    if not (np.array_equal(sha(x), golden["c1_xsha"]) and np.array_equal(sha(w), golden["c1_wsha"])):
        pytest.skip("this torch build draws different random numbers")
    fw = Q.quantize_weight(w.cuda())
    xq, sx = Q.quantize_act(x.cuda())
    y = Q.fp8_matmul(xq, sx, fw)
    ref = from_bits16(golden["c1_y"]).float()
    assert max_rel(y.cpu().float(), ref) <= TOL_BF16
    # end to end through the public call, as the reference's test does
    y2 = Q.fp8_linear(x.cuda(), fw)
    assert torch.equal(y, y2)


def test_small_golden_gemm(Q, golden):
    xq = torch.from_numpy(golden["gemm_xq"]).cuda().view(Q.FP8)
    sx = from_bits32(golden["gemm_sx"]).cuda().reshape(1, 1)
    for wq_key, sw_key, y_key in (("weight_q", "weight_scale", "gemm_ya"),
                                  ("gemm_wbq", "gemm_wb_scale", "gemm_yb")):
        wq = torch.from_numpy(golden[wq_key]).cuda().view(Q.FP8)
        fw = Q.FP8Weight(data=wq, scale=from_bits32(golden[sw_key]).cuda().reshape(1, 1),
                         shape=tuple(wq.shape))
        y = Q.fp8_matmul(xq, sx, fw)
        assert max_rel(y.cpu().float(), from_bits16(golden[y_key]).float()) <= TOL_BF16


def test_run_to_run_determinism_and_split_k(Q):
    _, _, xq, sx, fw = _operands(Q, 128, 4096, 4096, seed=8)
    ref = TS.dequant_matmul(xq, sx, fw.data, fw.scale)
    try:
        for split in (1, 2, 4):
            Q.set_option("decode_split_k", split)
            a = Q.fp8_matmul(xq, sx, fw)
            assert Q.last_gemm_launch()["split"] == split
            for _ in range(3):
                assert torch.equal(a, Q.fp8_matmul(xq, sx, fw)), f"split {split} is not deterministic"
            assert max_rel(a, ref) <= TOL_BF16
    finally:
        Q.set_option("decode_split_k", 0)


def test_pipeline_depth_does_not_change_results(Q):
    _, _, xq, sx, fw = _operands(Q, 16, 512, 4096, seed=9)
    try:
        Q.set_option("decode_split_k", 1)
        base = Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32)
        for stages in (1, 2, 3, 5):
            Q.set_option("decode_stages", stages)
            assert torch.equal(base, Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32))
            assert Q.last_gemm_launch()["stages"] <= stages     # never deeper than the work
    finally:
        Q.set_option("decode_split_k", 0)
        Q.set_option("decode_stages", 0)


@pytest.mark.parametrize("M", [4, 128, 1024])
def test_project_matches_linear_per_weight(Q, M):
    """tests/test_quant.py:211-218 — grouped launch equals the separate calls bit for bit."""
    x = randn_cpu((M, 256), seed=12).cuda()
    qa = Q.quantize_weight(randn_cpu((512, 256), seed=13, scale=0.02).cuda())
    qb = Q.quantize_weight(randn_cpu((128, 256), seed=14, scale=0.03).cuda())
    qc = Q.quantize_weight(randn_cpu((272, 256), seed=15, scale=0.01).cuda())
    got = Q.project(x, qa, qb, qc)
    for g, w in zip(got, (qa, qb, qc)):
        assert torch.equal(g, Q.fp8_linear(x, w))


def test_project_leaves_bf16_weights_on_the_bf16_path(Q):
    """tests/test_quant.py:221-242: a weight left in bf16 is multiplied unquantized.  Through
    `F.linear` (the reference's arm, selectable) the result is that call's bits; as a 16-bit
    segment of the one launch (default) it is the same product up to summation order."""
    x = randn_cpu((4, 256), seed=16).cuda()
    a = randn_cpu((512, 256), seed=17, scale=0.02).cuda()
    b = randn_cpu((32, 256), seed=18, scale=0.02).cuda()
    Q.set_dense_segments(False)
    try:
        got_a, got_b = Q.project(x, Q.quantize_weight(a), b)
        assert torch.equal(got_b, F.linear(x, b))
    finally:
        Q.set_dense_segments(True)
    n0 = Q.launch_count()
    seg_a, seg_b = Q.project(x, Q.quantize_weight(a), b)
    assert Q.launch_count() - n0 == 2                       # one quantizer, one GEMM launch
    assert torch.equal(seg_a, got_a)                        # the FP8 member does not change
    assert seg_b.dtype is torch.bfloat16 and seg_b.shape == (4, 32)
    assert max_rel(seg_b, F.linear(x.float(), b.float())) <= 2 ** -8
    ga, gb = Q.project(x, a, b)                             # no FP8 member: untouched torch path
    assert torch.equal(ga, F.linear(x, a)) and torch.equal(gb, F.linear(x, b))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("M", [1, 16, 37, 128, 256])
def test_gdn_input_projection_as_one_launch(Q, dt, M):
    """braid/model/gdn.py:254-255: `project(x, qkv, z, a, b)` with qkv / z in FP8 and the gates
    a / b unquantized (32 x 4096 each, braid/model/gdn.py:73-81), at the 9B widths.  FP8 members
    bit-equal to the grouped FP8 launch; a and b within bf16 rounding of the exact product and
    almost everywhere bit-equal to `F.linear`; run-to-run identical; graph-capturable."""
    H = 4096
    x = randn_cpu((M, H), seed=M, dtype=dt).cuda()
    qkv = Q.quantize_weight(randn_cpu((8192, H), seed=1, scale=0.02).cuda())
    z = Q.quantize_weight(randn_cpu((4096, H), seed=2, scale=0.02).cuda())
    a = randn_cpu((32, H), seed=3, dtype=dt, scale=0.02).cuda()
    b = randn_cpu((32, H), seed=4, dtype=dt, scale=0.05).cuda()
    ys = Q.project(x, qkv, z, a, b)
    assert Q.last_gemm_launch()["kernel"] == "stream"
    xq, sx = Q.quantize_act(x)
    for got, want in zip(ys[:2], Q.fp8_matmul_grouped(xq, sx, (qkv, z), out_dtype=dt)):
        assert torch.equal(got, want)
    for got, w in zip(ys[2:], (a, b)):
        exact = F.linear(x.double(), w.double())
        assert got.dtype is dt and got.shape == (M, 32)
        assert max_rel(got, exact) <= (2 ** -8 if dt is torch.bfloat16 else 2 ** -10)
        assert (got != F.linear(x, w)).float().mean().item() < 0.1
    again = Q.project(x, qkv, z, a, b)
    assert all(torch.equal(p, q) for p, q in zip(ys, again))
    # a pre-quantized activation that kept its dense form takes the same launch
    pre = Q.QuantizedActivation(xq, sx, x.shape, dt, dense=x)
    assert all(torch.equal(p, q) for p, q in zip(ys, Q.project(pre, qkv, z, a, b)))
    assert Q.device_status() == 0


def test_leading_dims_and_dispatch(Q):
    x = randn_cpu((2, 3, 256), seed=19).cuda()
    w = randn_cpu((512, 256), seed=20, scale=0.02).cuda()
    fw = Q.quantize_weight(w)
    out = Q.fp8_linear(x, fw)
    assert out.shape == (2, 3, 512) and out.dtype is torch.bfloat16
    assert torch.equal(Q.linear(x, w), F.linear(x, w))
    ref = F.linear(x, w)
    rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 8e-2
    assert F.cosine_similarity(out.float().flatten(), ref.float().flatten(), dim=0) > 0.99
    (p,) = Q.project(x, fw)
    assert p.shape == (2, 3, 512)


def test_outputs_stay_inside_their_buffers(Q):
    """Canary rows/columns around a strided output must survive (M and N off the tile grid)."""
    for M, N, K in ((37, 272, 256), (300, 272, 256)):
        _, _, xq, sx, fw = _operands(Q, M, N, K, seed=21)
        big = torch.full((M + 2, N + 32), 7.0, device="cuda", dtype=torch.bfloat16)
        out = big[1:M + 1, 16:16 + N]
        Q.fp8_matmul_grouped(xq, sx, (fw,), out=(out,))
        assert torch.equal(out, Q.fp8_matmul(xq, sx, fw))
        mask = torch.ones_like(big, dtype=torch.bool)
        mask[1:M + 1, 16:16 + N] = False
        assert (big[mask] == 7.0).all()


def test_scaling_the_activation_scale_scales_the_output(Q):
    """Linearity at full decode size: doubling sx doubles every output exactly (power of two)."""
    _, _, xq, sx, fw = _operands(Q, 128, 12288, 4096, seed=22)
    y1 = Q.fp8_matmul(xq, sx, fw, out_dtype=torch.float32)
    y2 = Q.fp8_matmul(xq, sx * 2, fw, out_dtype=torch.float32)
    assert torch.equal(y2, y1 * 2)


def test_fused_mlp_equals_the_unfused_sequence(Q):
    """braid/model/mlp.py:44-49 spelled with separate kernels vs `mlp_forward` (4 launches)."""
    M, H, I = 128, 4096, 12288
    x = randn_cpu((M, H), seed=23).cuda()
    wg = Q.quantize_weight(randn_cpu((I, H), seed=24, scale=0.02).cuda())
    wu = Q.quantize_weight(randn_cpu((I, H), seed=25, scale=0.02).cuda())
    wd = Q.quantize_weight(randn_cpu((H, I), seed=26, scale=0.02).cuda())
    xq, sx = Q.quantize_act(x)
    gate = Q.fp8_matmul(xq, sx, wg)
    up = Q.fp8_matmul(xq, sx, wu)
    h = F.silu(gate) * up
    want = Q.linear(h, wd)
    got = Q.mlp_forward(x, wg, wu, wd)
    assert torch.equal(got, want)
    # and it tracks the bf16 MLP the way the reference demands (tests/test_quant.py:157-178)
    wgf, wuf, wdf = (w.data.float() * w.scale for w in (wg, wu, wd))
    ref = F.linear(F.silu(F.linear(x.float(), wgf)) * F.linear(x.float(), wuf), wdf)
    assert F.cosine_similarity(got.float().flatten(), ref.flatten(), dim=0) > 0.99


def test_gated_output_projection(Q):
    B, T, H, D = 4, 1, 16, 256
    qg = randn_cpu((B, T, H * 2 * D), seed=27, scale=2.0).cuda()
    o = randn_cpu((B, T, H * D), seed=28).cuda()
    wo = Q.quantize_weight(randn_cpu((4096, H * D), seed=29, scale=0.02).cuda())
    _, gate = qg.view(B, T, H, 2 * D).chunk(2, dim=-1)
    want = Q.linear(o * torch.sigmoid(gate.reshape(B, T, H * D)), wo)
    assert torch.equal(Q.gated_output_projection(o, gate, wo), want)


def test_eager_equals_graph_replay(Q):
    """tests/test_graph_quant.py:48-87 in miniature: capture quantize + grouped GEMM + fused MLP,
    replay with new contents in the static input, compare with eager bit for bit."""
    M, H, I = 16, 1024, 2048
    wq_ = Q.quantize_weight(randn_cpu((2048, H), seed=30, scale=0.02).cuda())
    wk_ = Q.quantize_weight(randn_cpu((256, H), seed=31, scale=0.02).cuda())
    wg = Q.quantize_weight(randn_cpu((I, H), seed=32, scale=0.02).cuda())
    wu = Q.quantize_weight(randn_cpu((I, H), seed=33, scale=0.02).cuda())
    wd = Q.quantize_weight(randn_cpu((H, I), seed=34, scale=0.02).cuda())

    def step(x):
        q, k = Q.project(x, wq_, wk_)
        return q[:, :H] + Q.mlp_forward(x + k.sum(dim=1, keepdim=True) * 0, wg, wu, wd)

    static_x = randn_cpu((M, H), seed=35).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step(static_x)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_y = step(static_x)
    for seed in (36, 37):
        new = randn_cpu((M, H), seed=seed, scale=float(seed - 34)).cuda()
        eager = step(new).clone()
        static_x.copy_(new)
        graph.replay()
        assert torch.equal(static_y, eager)
    assert Q.device_status() == 0


def test_shape_guards(Q):
    with pytest.raises(ValueError, match="multiples of 16"):
        Q.quantize_weight(torch.randn(30, 256, device="cuda", dtype=torch.bfloat16))
    w = torch.randn(512, 250, device="cuda", dtype=torch.bfloat16)
    assert Q.maybe_quantize(w, True) is w
    _, _, xq, sx, fw = _operands(Q, 4, 64, 128, seed=40)
    bad = Q.FP8Weight(data=fw.data[:, :64].contiguous(), scale=fw.scale, shape=(64, 64))
    with pytest.raises(ValueError):
        Q.fp8_matmul(xq, sx, bad)
    assert Q.device_status() == 0


# -- residual add in the epilogue ---------------------------------------------------------------
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("M", [1, 8, 37, 128, 256, 512])
@pytest.mark.parametrize("N,K", [(4096, 4096), (4096, 12288), (1024, 4096), (272, 256), (16, 16)])
def test_residual_epilogue_equals_gemm_then_add(Q, dt, M, N, K):
    """`residual + fp8_matmul(...)` as torch evaluates it (GEMM output rounded to the output type,
    then the add rounds again) against the add done in the GEMM epilogue: bit-equal for every K
    split (1, 2, 4), ragged M, and the prefill sizes that fall back to a separate add."""
    if dt is not torch.bfloat16 and (N, K) not in ((4096, 4096), (272, 256)):
        pytest.skip("dtype variants on two shapes")
    _, _, xq, sx, fw = _operands(Q, M, N, K, seed=M + N)
    res = randn_cpu((M, N), seed=7, dtype=dt, scale=0.5).cuda()
    want = res + Q.fp8_matmul(xq, sx, fw, out_dtype=dt)
    got = Q.fp8_matmul(xq, sx, fw, out_dtype=dt, residual=res)
    assert got.dtype is dt and got.shape == (M, N)
    assert torch.equal(got, want), f"{int((got != want).sum())} of {got.numel()} differ"


def test_residual_strided_scoped_and_through_the_sublayers(Q):
    H, I, M = 4096, 12288, 16
    x = randn_cpu((M, 1, H), seed=1).cuda()
    mk = lambda n, k, s: Q.quantize_weight(randn_cpu((n, k), seed=s, scale=0.02).cuda())  # noqa: E731
    w_out, wg, wu, wd = mk(H, H, 2), mk(I, H, 3), mk(I, H, 4), mk(H, I, 5)
    wide = randn_cpu((M, 2 * H), seed=6).cuda()
    res = wide[:, H:]                                           # row stride 2H
    xq, sx = Q.quantize_act(x.reshape(M, H))
    assert torch.equal(Q.fp8_matmul(xq, sx, w_out, residual=res), res + Q.fp8_matmul(xq, sx, w_out))
    r3 = randn_cpu((M, 1, H), seed=8).cuda()
    assert torch.equal(Q.linear(x, w_out, residual=r3), r3 + Q.linear(x, w_out))
    assert torch.equal(Q.mlp_forward(x, wg, wu, wd, residual=r3), r3 + Q.mlp_forward(x, wg, wu, wd))
    # the scoped form: only the named weight takes the residual, and only once
    with Q.residual_into(w_out, r3) as slot:
        a = Q.linear(x, wd_t := mk(H, H, 9))                    # another weight: untouched
        assert not slot.taken
        b = Q.linear(x, w_out)
        assert slot.taken
        c = Q.linear(x, w_out)                                  # second call: plain again
    assert torch.equal(a, Q.linear(x, wd_t))
    assert torch.equal(b, r3 + Q.linear(x, w_out)) and torch.equal(c, Q.linear(x, w_out))
    with Q.residual_into(None, r3) as slot:
        assert torch.equal(Q.linear(x, w_out), c) and not slot.taken
    with pytest.raises(ValueError):
        Q.fp8_matmul(xq, sx, w_out, residual=r3.reshape(M, H)[:, :128])


# -- gate and up as one paired GEMM with SiLU*mul + quantization in the epilogue -----------------------
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("M", [1, 8, 37, 128, 200, 256])
@pytest.mark.parametrize("I,K", [(12288, 4096), (9216, 2560), (1024, 512), (64, 128), (2048, 4096)],
                         ids=["9B", "4B", "small", "one_tile", "split4"])
def test_paired_gate_up_epilogue_equals_the_separate_kernels(Q, dt, M, I, K):
    """Codes and scale of h from the one-launch form against grouped GEMM + `silu_mul_quant`:
    every K split the shape rule produces (1, 2, 4), ragged M, three activation types."""
    if dt is not torch.bfloat16 and (I, K) not in ((9216, 2560), (1024, 512)):
        pytest.skip("dtype variants on two shapes")
    x = randn_cpu((M, K), seed=M + I, dtype=dt).cuda()
    gate = Q.quantize_weight(randn_cpu((I, K), seed=1, scale=0.02).cuda())
    up = Q.quantize_weight(randn_cpu((I, K), seed=2, scale=0.05).cuda())      # a different scale
    xq, sx = Q.quantize_act(x)
    g, u = Q.fp8_matmul_grouped(xq, sx, (gate, up), out_dtype=dt)
    hq_ref, sh_ref = Q.silu_mul_quant(g, u)
    got = Q.gate_up_silu_quant(xq, sx, gate, up, dt)
    if got is None:
        # the exchange needs the whole grid resident: with M > 128 the staging buffer allows one
        # CTA per SM, which tiles x K slices of the larger shapes exceed (192 for the 9B MLP,
        # 288 for the 4B one) -- the caller then runs 4 launches
        assert M > 128 and 2 * I // 128 > 74, "paired form refused a launch that fits"
        pytest.skip("grid not co-resident at this M: four-launch path")
    hq, sh = got
    assert torch.equal(sh, sh_ref), f"scale {sh.item():.9e} vs {sh_ref.item():.9e}"
    bad = int((hq.view(torch.uint8) != hq_ref.view(torch.uint8)).sum())
    assert bad == 0, f"{bad} of {hq.numel()} codes differ"
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("M,I,K", [(300, 1024, 512), (1000, 12288, 4096), (2048, 1536, 4096),
                                   (4100, 272, 1040)],
                         ids=["small", "9B", "shard_of_8", "ragged"])
def test_prefill_gate_up_silu_equals_the_separate_kernels(Q, dt, M, I, K):
    """M > 256: h = silu(gate) * up and its scale written by the CTA-pair GEMM's epilogue, then
    `cast_act`, against the grouped GEMM + torch's SiLU*mul + the quantizer: h, scale and codes
    bit for bit (three activation types, I off the tile grid, ragged M)."""
    if dt is not torch.bfloat16 and (M, I) not in ((300, 1024), (4100, 272)):
        pytest.skip("dtype variants on two shapes")
    x = randn_cpu((M, K), seed=M + I, dtype=dt).cuda()
    gate = Q.quantize_weight(randn_cpu((I, K), seed=1, scale=0.02).cuda())
    up = Q.quantize_weight(randn_cpu((I, K), seed=2, scale=0.05).cuda())
    xq, sx = Q.quantize_act(x)
    g, u = Q.fp8_matmul_grouped(xq, sx, (gate, up), out_dtype=dt)
    h_ref = F.silu(g) * u
    hq_ref, sh_ref = Q.quantize_act(h_ref)
    got = Q.gate_up_silu(xq, sx, gate, up, dt)
    assert got is not None and Q.last_gemm_launch()["kernel"] == "pair"
    h, sh = got
    assert torch.equal(h, h_ref), f"{int((h != h_ref).sum())} of {h.numel()} h values differ"
    assert torch.equal(sh, sh_ref), f"scale {sh.item():.9e} vs {sh_ref.item():.9e}"
    assert torch.equal(Q.cast_act(h, sh).view(torch.uint8), hq_ref.view(torch.uint8))
    h2, sh2 = Q.gate_up_silu(xq, sx, gate, up, dt)          # the scratch words were returned to zero
    assert torch.equal(h2, h) and torch.equal(sh2, sh)
    assert Q.device_status() == 0


def test_paired_mlp_equals_the_four_launch_mlp_and_replays(Q):
    H, I = 4096, 12288
    mk = lambda n, k, s: Q.quantize_weight(randn_cpu((n, k), seed=s, scale=0.02).cuda())  # noqa: E731
    wg, wu, wd = mk(I, H, 3), mk(I, H, 4), mk(H, I, 5)
    for M in (1, 16, 128, 300):
        x = randn_cpu((M, H), seed=M).cuda()
        r = randn_cpu((M, H), seed=M + 1).cuda()
        Q.set_paired_mlp(False)
        want, want_r = Q.mlp_forward(x, wg, wu, wd), Q.mlp_forward(x, wg, wu, wd, residual=r)
        Q.set_paired_mlp(True)
        n0 = Q.launch_count()
        got = Q.mlp_forward(x, wg, wu, wd)
        assert Q.launch_count() - n0 == (3 if M <= 128 else 4)
        assert torch.equal(got, want) and torch.equal(Q.mlp_forward(x, wg, wu, wd, residual=r), want_r)
    # the one-launch form reads the two weights in place: no copy of either is made or kept
    free0 = torch.cuda.mem_get_info()[0]
    Q.mlp_forward(randn_cpu((16, H), seed=2).cuda(), wg, wu, wd)
    torch.cuda.synchronize()
    assert free0 - torch.cuda.mem_get_info()[0] < 32 << 20
    # capture + replay
    x = randn_cpu((128, H), seed=9).cuda()
    eager = Q.mlp_forward(x, wg, wu, wd).clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            Q.mlp_forward(x, wg, wu, wd)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = Q.mlp_forward(x, wg, wu, wd)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager) and Q.device_status() == 0
