"""The reference's own engine, decode step and graph capture, running on these kernels.

Port of the reference's capture gate (tests/test_graph_quant.py:51-91: every quant group must
survive CUDA-graph capture and replay bit-identically) onto a random-init stack of the 9B shape
(`braid_b200.engine_dropin.random_checkpoint`; the published checkpoints are not available
offline), plus the comparison the reference cannot make: the same engine stock and on these
kernels, on the same weights.

Needs the install of the reference under baseline/_ref (not part of the repository); skipped
without it.  The mixers use the reference's CUDA kernels when a prebuilt extension is present
(baseline/ref_kernels.py), its torch path otherwise.
"""
from __future__ import annotations

import gc
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "braid" / "model" / "engine.py").exists(),
                                 reason="no reference install under baseline/_ref")]

LAYERS, VOCAB, B, MAX_LEN = 8, 4096, 4, 96


def _purge():
    for name in [m for m in sys.modules if m == "braid" or m.startswith("braid.")]:
        del sys.modules[name]


@pytest.fixture(scope="module")
def ref_engine_env(Q):
    """Reference modules imported fresh, its kernels attached if prebuilt, one shared checkpoint."""
    from braid_b200 import engine_dropin as E
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(ROOT / "baseline"))
    _purge()
    import ref_kernels
    use_kernels = ref_kernels.available()
    if use_kernels:
        ref_kernels.attach()
    ckpt = E.random_checkpoint(E.text_config(LAYERS, VOCAB), torch.device("cuda", 0), seed=3)
    yield E, ckpt, use_kernels
    E.deactivate()
    del ckpt
    _purge()
    sys.path.remove(str(REF))
    sys.path.remove(str(ROOT / "baseline"))
    gc.collect()
    torch.cuda.empty_cache()


def _prefilled(E, eng, rows):
    cache = eng.allocate_cache(MAX_LEN, max_slots=rows + 1)
    g = torch.Generator(device="cuda").manual_seed(5)
    for slot in range(rows + 1):
        cache.reset_slot(slot)
    # differing state per row, as the reference's gate does: zeros would hide a slot mix-up
    for row in range(rows):
        eng.forward(torch.randint(0, 1000, (1, 6 + row), generator=g, device="cuda"),
                    cache.select([row]))
    return cache


@pytest.mark.parametrize("fuse_norms", [True, False], ids=["norms_fused", "norms_torch"])
@pytest.mark.parametrize("quant", ["mlp", "attn", "gdn", "head", "all"])
def test_every_quant_group_captures_and_replays_identically(Q, ref_engine_env, quant, fuse_norms):
    E, ckpt, use_kernels = ref_engine_env
    import importlib
    graph_mod = importlib.import_module("braid.model.graph")
    E.activate(fuse_norms=fuse_norms)
    eng = cache = dec = None
    try:
        eng = E.build_engine(ckpt, quant=quant, use_kernels=use_kernels)
        assert eng.quant, f"{quant} resolved to no groups"
        assert "active" in eng.quant_report().splitlines()[-1]
        n0 = Q.launch_count()
        cache = _prefilled(E, eng, B)
        snapshot = cache.snapshot()
        tokens = torch.arange(100, 100 + B, device="cuda")[:, None]
        slots = torch.arange(B, device="cuda")

        eager = eng.decode_step(tokens, cache.select(slots.tolist())).clone()
        assert Q.launch_count() > n0, "the decode step launched none of this library's kernels"
        cache.restore(snapshot)
        dec = graph_mod.GraphedDecoder(eng, cache, buckets=(B,))
        cache.restore(snapshot)
        replay = dec.step(tokens, slots)
        assert torch.isfinite(eager.float()).all()
        assert torch.equal(eager, replay), (
            f"quant={quant}: replay differs from eager by "
            f"{(eager.float() - replay.float()).abs().max():.3e}")
        assert Q.device_status() == 0
    finally:
        E.deactivate()
        del eng, cache, dec
        gc.collect()
        torch.cuda.empty_cache()


# ---- the reference's group-wiring gates (tests/test_quant.py:264-358) on the random-init stack ----
GROUP_NAMES = ("mlp", "attn", "gdn", "head")


def _wired_engine(E, ckpt, quant, use_kernels):
    E.activate()
    return E.build_engine(ckpt, quant=quant, use_kernels=use_kernels)


def _drop(eng):
    del eng
    gc.collect()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("group", GROUP_NAMES)
def test_a_group_quantizes_itself_and_nothing_else(Q, ref_engine_env, group):
    """tests/test_quant.py:264-283: asking for one group must not quantize a neighbour; `attn`
    and `gdn` sit on alternating layers of the same stack."""
    E, ckpt, use_kernels = ref_engine_env
    eng = _wired_engine(E, ckpt, group, use_kernels)
    try:
        got = {g: [isinstance(w, Q.FP8Weight) for w in ws] for g, ws in eng._projections().items()}
        assert all(len(v) for v in got.values()), "the random stack must hold every group"
        assert all(got[group]) or group == "gdn", f"{group} was not quantized"
        if group == "gdn":      # a and b are excluded by design; everything else in the group goes
            assert sum(got["gdn"]) == len(got["gdn"]) * 3 // 5
        for other in set(GROUP_NAMES) - {group}:
            assert not any(got[other]), f"asking for {group} also quantized {other}"
    finally:
        E.deactivate()
        _drop(eng)


def test_gates_stay_bf16_and_the_embedding_is_never_quantized(Q, ref_engine_env):
    """tests/test_quant.py:286-320: `in_proj_a` / `in_proj_b` stay bf16 even under "all";
    `embed_tokens` is gathered per token and is never quantized."""
    E, ckpt, use_kernels = ref_engine_env
    eng = _wired_engine(E, ckpt, "all", use_kernels)
    try:
        gdn = [lyr.mixer for lyr in eng.layers if lyr.is_gdn]
        assert gdn, "no linear-attention layers in this stack"
        for m in gdn:
            assert not isinstance(m.in_proj_a, Q.FP8Weight) and m.in_proj_a.dtype is torch.bfloat16
            assert not isinstance(m.in_proj_b, Q.FP8Weight) and m.in_proj_b.dtype is torch.bfloat16
            assert all(isinstance(w, Q.FP8Weight) for w in (m.in_proj_qkv, m.in_proj_z, m.out_proj))
        assert isinstance(eng.embed_tokens, torch.Tensor) and eng.embed_tokens.dtype is torch.bfloat16
        assert isinstance(eng.lm_head, Q.FP8Weight)
    finally:
        E.deactivate()
        _drop(eng)


def test_each_group_removes_its_own_bytes_and_the_report_states_the_result(Q, ref_engine_env):
    """tests/test_quant.py:323-358: FP8 is worth exactly the bytes it removes from `step_bytes`,
    group by group, and `quant_report` shows what WAS quantized (3 of 5 for gdn), not the request."""
    E, ckpt, use_kernels = ref_engine_env
    base = _wired_engine(E, ckpt, "", use_kernels)
    want = base.step_bytes()
    E.deactivate()
    _drop(base)
    for group in GROUP_NAMES:
        eng = _wired_engine(E, ckpt, group, use_kernels)
        try:
            got = eng.step_bytes()
            assert got[group] < want[group] * 0.75, f"{group}: {got[group]} vs bf16 {want[group]}"
            for other in set(GROUP_NAMES) - {group}:
                assert got[other] == want[other], f"{group} moved {other}'s bytes"
            if group == "gdn":
                rep = eng.quant_report()
                assert "[on]" in rep and "[off]" in rep
                line = next(x for x in rep.splitlines() if x.strip().startswith("gdn"))
                n_q, n = line.split()[1].split("/")
                assert int(n_q) == int(n) * 3 // 5, line
                assert "active" in rep.splitlines()[-1]
        finally:
            E.deactivate()
            _drop(eng)


def _truncated(ckpt, layers):
    """The first `layers` layers of the shared checkpoint (same tensors, shorter schedule)."""
    import importlib
    from braid_b200 import engine_dropin as E
    config = importlib.import_module("braid.model.config")
    loader = importlib.import_module("braid.model.loader")
    cfg = config.ModelConfig.from_dict({"text_config": E.text_config(layers, VOCAB)})
    return loader.Checkpoint(config=cfg, tensors=ckpt.tensors)


def _first_step_logits(E, ckpt, use_kernels):
    tokens = torch.arange(100, 100 + B, device="cuda")[:, None]
    logits = {}
    for name, quant, ours in (("stock", "all", False), ("bf16", "", False), ("b200", "all", True),
                              ("b200_norms_torch", "all", True)):
        E.activate(fuse_norms=(name == "b200")) if ours else E.deactivate()
        eng = E.build_engine(ckpt, quant=quant, use_kernels=use_kernels)
        cache = _prefilled(E, eng, B)
        logits[name] = eng.decode_step(tokens, cache.select(list(range(B)))).clone()
        del eng, cache
        gc.collect()
        torch.cuda.empty_cache()
    E.deactivate()
    return logits


def test_engine_on_these_kernels_tracks_the_stock_engine(Q, ref_engine_env):
    """Same weights, same tokens: FP8 through `torch._scaled_mm` against FP8 through this library.
    Activation codes and scales are bit-identical by construction; the two GEMMs differ in
    accumulation order, so a bf16 output can land one ulp apart, which the next quantizer turns
    into an occasional different code.  With random-init weights a deep stack amplifies any such
    difference, so the yardstick is what FP8 itself does to the same logits (stock FP8 against
    the stock bf16 engine): measured on B200, the swap moves the 8-layer logits by 0.33 of that
    (rel-L2 0.136 against 0.413), a single layer by 0.019 against 0.134."""
    E, ckpt, use_kernels = ref_engine_env
    one = _first_step_logits(E, _truncated(ckpt, 1), use_kernels)
    near = E.logits_agreement(one["b200"], one["stock"])
    assert near["cosine"] > 0.999 and near["rel_l2"] < 0.05, near
    assert near["argmax_match"] == 1.0, near

    # fusing the norms changes no bit anywhere in the engine
    assert torch.equal(one["b200"], one["b200_norms_torch"])

    deep = _first_step_logits(E, ckpt, use_kernels)
    assert torch.equal(deep["b200"], deep["b200_norms_torch"])
    ours_vs_stock = E.logits_agreement(deep["b200"], deep["stock"])
    stock_vs_bf16 = E.logits_agreement(deep["stock"], deep["bf16"])
    ours_vs_bf16 = E.logits_agreement(deep["b200"], deep["bf16"])
    assert ours_vs_stock["rel_l2"] < 0.5 * stock_vs_bf16["rel_l2"], (ours_vs_stock, stock_vs_bf16)
    assert ours_vs_bf16["rel_l2"] < 1.1 * stock_vs_bf16["rel_l2"], (ours_vs_bf16, stock_vs_bf16)


def test_activate_is_reversible(Q, ref_engine_env):
    E, _, _ = ref_engine_env
    import importlib
    rq = importlib.import_module("braid.model.quant")
    mlp = importlib.import_module("braid.model.mlp")
    E.deactivate()
    layer = importlib.import_module("braid.model.layer")
    gdn = importlib.import_module("braid.model.gdn")

    def state():
        return (rq.quantize_act, rq.fp8_matmul, mlp.fp8_matmul, mlp.MLP.forward, rq.FP8Weight,
                layer.DecoderLayer.forward, layer.DecoderLayer.__call__, gdn.GatedDeltaNet._readout)

    stock = state()
    done = E.activate()
    assert "braid.model.mlp.MLP.forward" in done and rq.fp8_matmul is Q.fp8_matmul
    assert "braid.model.layer.DecoderLayer.forward" in done
    assert "braid.model.gdn.GatedDeltaNet._readout" in done
    assert mlp.fp8_matmul is Q.fp8_matmul and rq.FP8Weight is Q.FP8Weight
    assert all(a is not b for a, b in zip(state(), stock))
    E.deactivate()
    assert state() == stock


@pytest.mark.parametrize("case", ["fp32_engine", "4b_widths"])
def test_other_engine_shapes_capture_and_replay_identically(Q, case):
    """The same gate on (a) an fp32 engine (fp32 activations through every fused kernel: the
    reference keeps fp32 engines for its identity gates) and (b) the 4B member's widths
    (hidden 2560, MLP 9216), both with every group quantized and all fusions on."""
    import importlib
    from braid_b200 import engine_dropin as E
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(ROOT / "baseline"))
    _purge()
    eng = cache = dec = ckpt = None
    try:
        import ref_kernels
        use_kernels = ref_kernels.available()
        if use_kernels:
            ref_kernels.attach()
        graph_mod = importlib.import_module("braid.model.graph")
        dtype = torch.float32 if case == "fp32_engine" else torch.bfloat16
        cfg = E.text_config(4, VOCAB) if case == "fp32_engine" else \
            E.text_config(4, VOCAB, hidden_size=2560, intermediate_size=9216)
        ckpt = E.random_checkpoint(cfg, torch.device("cuda", 0), dtype=dtype, seed=4)
        E.activate()
        eng = E.build_engine(ckpt, quant="all", use_kernels=use_kernels, dtype=dtype,
                             state_dtype=torch.float32)
        n0 = Q.launch_count()
        cache = _prefilled(E, eng, B)
        snapshot = cache.snapshot()
        tokens = torch.arange(100, 100 + B, device="cuda")[:, None]
        slots = torch.arange(B, device="cuda")
        eager = eng.decode_step(tokens, cache.select(slots.tolist())).clone()
        assert eager.dtype is dtype and Q.launch_count() > n0
        cache.restore(snapshot)
        dec = graph_mod.GraphedDecoder(eng, cache, buckets=(B,))
        cache.restore(snapshot)
        replay = dec.step(tokens, slots)
        assert torch.isfinite(eager.float()).all() and torch.equal(eager, replay)
        assert Q.device_status() == 0
    finally:
        E.deactivate()
        del eng, cache, dec, ckpt
        _purge()
        sys.path.remove(str(REF))
        sys.path.remove(str(ROOT / "baseline"))
        gc.collect()
        torch.cuda.empty_cache()
