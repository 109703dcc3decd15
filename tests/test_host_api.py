"""Host-side logic and the C-ABI surface, without a GPU: group parsing, shape guards, symbol
export, argument validation that returns before any CUDA call, and the loud failure modes."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_group_names_round_trip():
    from braid_b200.quant import GROUPS, parse_groups
    assert parse_groups("") == frozenset()
    assert parse_groups(None) == frozenset()
    assert parse_groups("mlp") == {"mlp"}
    assert parse_groups("mlp, attn") == {"mlp", "attn"}
    assert parse_groups(["gdn", "head"]) == {"gdn", "head"}
    assert parse_groups("all") == frozenset(GROUPS)


def test_an_unknown_group_raises():
    from braid_b200.quant import parse_groups
    with pytest.raises(ValueError, match="unknown quant group"):
        parse_groups("mpl")
    with pytest.raises(ValueError, match="unknown quant group"):
        parse_groups("mlp,attention")


def test_public_names_match_the_reference_module():
    """Everything other reference modules import from braid.model.quant exists here."""
    from braid_b200 import quant
    for name in ("GROUPS", "parse_groups", "FP8", "FP8_MAX", "EPS", "FP8Weight", "quantize_weight",
                 "warm_fused", "fused_state", "quantize_act", "fp8_matmul", "fp8_linear", "linear",
                 "project", "maybe_quantize", "_act_scale", "_weight_scale", "_CAST_CHUNK_BYTES"):
        assert hasattr(quant, name), name
    assert quant.FP8 is torch.float8_e4m3fn and quant.FP8_MAX == 448.0 and quant.EPS == 1e-12


def test_weight_quantization_on_cpu_follows_the_reference_spelling(golden):
    """Load-time work keeps the torch spelling; on a CPU it reproduces the golden weight exactly."""
    from _util import from_bits16
    from braid_b200.quant import FP8Weight, maybe_quantize, quantize_weight
    import numpy as np
    w = from_bits16(golden["weight_w"])
    fw = quantize_weight(w)
    assert isinstance(fw, FP8Weight) and fw.shape == (256, 128) and fw.nbytes == 256 * 128 + 4
    assert fw.scale.shape == (1, 1) and fw.scale.dtype is torch.float32
    assert np.array_equal(fw.data.view(torch.uint8).numpy(), golden["weight_q"])
    assert int(fw.scale.view(torch.int32).item()) & 0xFFFFFFFF == int(golden["weight_scale"].reshape(-1)[0])
    # banding invariance (tests/test_quant.py:81-96)
    from braid_b200 import quant as Q
    old = Q._CAST_CHUNK_BYTES
    Q._CAST_CHUNK_BYTES = 128 * 4 * 3
    try:
        banded = quantize_weight(w)
    finally:
        Q._CAST_CHUNK_BYTES = old
    assert torch.equal(banded.data.view(torch.uint8), fw.data.view(torch.uint8))
    assert maybe_quantize(w, False) is w
    z = quantize_weight(torch.zeros(64, 32, dtype=torch.bfloat16))
    assert torch.isfinite(z.data.float()).all() and (z.scale > 0).all()
    for a in (w, -w.abs(), w * 100):
        assert torch.equal(Q._weight_scale(a), Q._act_scale(a))


@pytest.mark.parametrize("shape", [(30, 256), (512, 250)])
def test_shapes_the_gemm_cannot_take_are_refused(shape):
    from braid_b200.quant import maybe_quantize, quantize_weight
    w = torch.randn(*shape, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="multiples of 16"):
        quantize_weight(w)
    assert maybe_quantize(w, True) is w


def test_the_library_exports_every_declared_symbol(lib):
    """Each `bq_*` function declared in include/braid_b200.h resolves in the built library and has
    a ctypes signature."""
    from braid_b200 import _lib
    header = (ROOT / "include" / "braid_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(bq_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.bq_version() >= 100
    assert lib.bq_quant_workspace_bytes() == 16
    assert lib.bq_gemm_workspace_bytes(128, 4096, 4096) >= 16


def test_argument_validation_returns_before_any_cuda_call(lib):
    from braid_b200 import _lib
    assert lib.bq_quantize_act(None, 1, 8, None, None, None, 0, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_quantize_act(16, 9, 8, 16, 16, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_quantize_act(16, 1, 0, 16, 16, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_quantize_act(16, 1, 8, 16, 16, None, 0, None) == _lib.BQ_ERR_WORKSPACE
    assert lib.bq_quantize_act(24, 1, 8, 16, 16, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_silu_mul_quant(16, 16, 1, 4, 12, 12, 12, 16, 16, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_gemm_w8a8(16, 16, 16, 16, 16, 1, 8, 64, 24, 64, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_gemm_w8a8(16, 16, 16, 16, 16, 1, 8, 60, 32, 64, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_gemm_w8a8(16, 16, 16, 16, 16, 7, 8, 64, 32, 64, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_gemm_w8a8(16, 16, 16, 16, 16, 1, 8, 64, 32, 64, None, 0, None) == _lib.BQ_ERR_WORKSPACE
    # the prefill-size and column-parallel entry points: every check precedes any CUDA call
    assert lib.bq_cast_act(None, 1, 8, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_cast_act(24, 1, 8, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_rmsnorm_scale(16, 1, 4, 64, 64, 16, 1e-6, None, 64, 16, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_rmsnorm_scale(16, 1, 4, 64, 64, 16, 1e-6, 16, 64, 16, None, 0, None) == _lib.BQ_ERR_WORKSPACE
    assert lib.bq_rmsnorm_scale(16, 1, 4, 62, 64, 16, 1e-6, 16, 64, 16, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_gated_rmsnorm_scale(16, 0, 256, 16, 1, 256, 16, 1e-6, 4, 2, 64, 16, 256, 16, 16, 16,
                                      None) == _lib.BQ_ERR_UNSUPPORTED          # head_dim must be 128
    assert lib.bq_silu_mul_dense_scale(16, 16, 1, 4, 16, 16, 16, None, 16, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_silu_mul(16, 16, 1, 4, 12, 12, 12, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_sigmoid_mul(16, 16, 1, 4, 16, 16, 16, 0, 0, 16, None) == _lib.BQ_ERR_BAD_ARG
    ptrs = (ctypes.c_void_p * 2)(16, 32)
    bad = (ctypes.c_void_p * 2)(16, None)
    assert lib.bq_word_push(None, 2, ptrs, ptrs, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_word_push(16, 9, ptrs, ptrs, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_word_push(16, 2, bad, ptrs, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_wait_flag_scale(16, 16, 0, 16, 16, 2, 0, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_wait_flag_scale(16, 16, 2, 16, 16, 9, 0, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_cast_act_push(16, 1, 4, 16, 16, None, 2, ptrs, 64, ptrs, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_cast_act_push(16, 1, 4, 12, 16, 16, 2, ptrs, 64, ptrs, 16, 16, None) == _lib.BQ_ERR_UNSUPPORTED
    assert lib.bq_rows_push(16, 1, 4, 16, 16, 2, bad, 64, ptrs, 16, 16, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_rows_push(16, 1, 4, 16, 16, 2, ptrs, 64, ptrs, None, 0, None) == _lib.BQ_ERR_WORKSPACE
    assert lib.bq_scratchless_status(None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_set_option(b"no_such_option", 1) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_set_option(b"quant_ring", 1) == _lib.BQ_OK and lib.bq_set_option(b"push_tma", 1) == _lib.BQ_OK
    assert lib.bq_set_option(b"decode_split_k", 0) == _lib.BQ_OK
    for code in range(0, 9):
        assert _lib.status_string(code)
    with pytest.raises(ValueError):
        _lib.check(_lib.BQ_ERR_UNSUPPORTED, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.BQ_ERR_DEVICE_WAIT, "x")


def test_a_missing_library_is_loud(monkeypatch, tmp_path):
    from braid_b200 import _lib, quant
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libbraid_b200.so")
    monkeypatch.setattr(quant, "_FUSED", None)
    monkeypatch.setattr(quant, "_FUSED_STATE", "not tried")
    with pytest.raises(_lib.LibraryMissing):
        quant.warm_fused(True)
    assert quant.fused_state().startswith("unavailable: LibraryMissing")


def test_cpu_tensors_are_refused_not_emulated():
    from braid_b200 import quant
    x = torch.zeros(4, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        quant.quantize_act(x)
    with pytest.raises(RuntimeError, match="no CPU path"):
        quant.silu_mul_quant(x, x)
    fw = quant.quantize_weight(torch.randn(16, 16, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU path"):
        quant.fp8_matmul(x.to(quant.FP8), torch.ones(1, 1), fw)
    # weights left in bf16 never touch the kernels
    w = torch.randn(8, 16, dtype=torch.bfloat16)
    assert torch.equal(quant.project(x, w)[0], torch.nn.functional.linear(x, w))
    assert torch.equal(quant.linear(x, w), torch.nn.functional.linear(x, w))


def test_the_product_package_never_imports_the_oracle():
    for path in (ROOT / "braid_b200").rglob("*.py"):
        text = path.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), path


def test_install_into_rebinds_a_reference_shaped_module():
    """`install_into` on a stand-in with the reference's attribute names (no reference needed)."""
    import sys
    import types
    from braid_b200 import quant
    from braid_b200.integrate import adopt_weight, install_into
    ref = types.ModuleType("fake_ref_quant")
    for name in ("quantize_act", "fp8_matmul", "fp8_linear", "linear", "project", "warm_fused",
                 "fused_state", "FP8Weight", "quantize_weight", "maybe_quantize"):
        setattr(ref, name, object())
    user = types.ModuleType("fake_ref_mlp")
    user.fp8_matmul = user.quantize_act = object()
    sys.modules["fake_ref_mlp"] = user
    try:
        done = install_into(ref, extra_modules=("fake_ref_mlp", "not.loaded"))
    finally:
        del sys.modules["fake_ref_mlp"]
    assert ref.fp8_matmul is quant.fp8_matmul and ref.project is quant.project
    assert user.fp8_matmul is quant.fp8_matmul and user.quantize_act is quant.quantize_act
    assert "fake_ref_mlp.fp8_matmul" in done and ref._FUSED_STATE == "active"
    w = quant.quantize_weight(torch.randn(16, 16, dtype=torch.bfloat16))
    assert adopt_weight(w).data is w.data


# -- engine drop-in helpers (host side; the reference install is optional) ---------------------------
def _ref_install():
    from pathlib import Path
    ref = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
    return ref if (ref / "braid" / "model" / "engine.py").exists() else None


def test_text_config_is_the_9b_shape():
    from braid_b200.engine_dropin import text_config
    from braid_b200.projection_set import StackShapes
    c, s = text_config(), StackShapes()
    assert (c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"]) == (s.hidden, s.intermediate, s.n_layers)
    assert c["layer_types"].count("full_attention") == 8 and c["layer_types"][3] == "full_attention"
    assert 2 * c["num_attention_heads"] * c["head_dim"] == s.attn_q
    assert c["num_key_value_heads"] * c["head_dim"] == s.attn_kv
    assert c["linear_num_value_heads"] * c["linear_value_head_dim"] == s.gdn_inner
    assert (2 * c["linear_num_key_heads"] * c["linear_key_head_dim"]
            + c["linear_num_value_heads"] * c["linear_value_head_dim"]) == s.gdn_qkv
    assert text_config(layers=8, vocab=4096)["vocab_size"] == 4096


@pytest.mark.skipif(_ref_install() is None, reason="no reference install under baseline/_ref")
def test_random_checkpoint_runs_through_the_reference_engine_on_cpu():
    """A CPU-sized stack of the same structure: the reference's loader validation accepts the
    tensors and its engine decodes with every group quantized (stock torch arm)."""
    import sys
    ref = _ref_install()
    sys.path.insert(0, str(ref))
    try:
        from braid_b200 import engine_dropin as E
        cfg = E.text_config(layers=4, vocab=1024, hidden_size=64, intermediate_size=128,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                            linear_num_value_heads=4, linear_num_key_heads=2,
                            linear_value_head_dim=16, linear_key_head_dim=16,
                            rope_parameters={"rope_type": "default", "rope_theta": 1e7,
                                             "partial_rotary_factor": 0.25, "mrope_section": [2, 1, 1],
                                             "mrope_interleaved": True})
        ck = E.random_checkpoint(cfg, "cpu", torch.bfloat16)
        assert ck.config.gdn_layers == (0, 1, 2) and ck.config.attention_layers == (3,)
        eng = E.build_engine(ck, quant="all", use_kernels=False, state_dtype=torch.float32)
        cache = eng.allocate_cache(32, max_slots=3)
        E.seed_cache(eng, cache, 3, 5)
        out = eng.decode_step(torch.tensor([[1], [2], [3]]), cache.select([0, 1, 2]))
        assert out.shape == (3, 1024) and torch.isfinite(out.float()).all()
        assert " 3/3 " in eng.quant_report() or "fp8" in eng.quant_report()
    finally:
        sys.path.remove(str(ref))
        for name in [m for m in sys.modules if m == "braid" or m.startswith("braid.")]:
            del sys.modules[name]


def test_push_entry_points_check_their_arguments():
    """Host-only: the column-parallel entry points refuse missing pointers before any CUDA call."""
    from braid_b200 import _lib
    lib = _lib.load()
    assert lib.bq_wait_flag(None, None, 1, None, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_gemm_w8a8_push(None, None, None, None, 1, 8, 4096, 4096, 0, None, 4096, None,
                                 None, 0, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_peer_open(None, None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_peer_alloc(0, None, None) == _lib.BQ_ERR_BAD_ARG
