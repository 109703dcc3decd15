"""The reference's whole decode step on these kernels: a random-init checkpoint of the
Qwen3.5-9B shape, the reference's own `Engine`, and the two arms that are compared.

Nothing here restates the engine: `braid.model.engine.Engine`, `braid.model.graph.GraphedDecoder`
and the mixers are imported from an install of the reference (it must be importable as `braid`)
and run unmodified.  What this module adds is

  * `text_config()` / `random_checkpoint()` — a `braid.model.loader.Checkpoint` with the tensor
    names, shapes, dtypes and load-time transforms `load_checkpoint` would have produced
    (braid/model/loader.py:71-84 names, :167-209 transforms, :303-342 shapes), filled from a
    seeded generator because no published checkpoint is available offline;
  * `activate()` / `deactivate()` — rebinding the reference's quant API onto this package
    (`integrate.install_into`) plus the class-level swap of `MLP.forward` for the four-launch
    fused form, and back;
  * `decode_arm()` — one arm of the reference's decode-speed measurement
    (braid/bench/decode_speed.py:138-186: seed KV under every row, capture
    `Engine.decode_step` with `GraphedDecoder`, time replays with events around the whole run).
"""
from __future__ import annotations

import importlib
import sys
from dataclasses import dataclass

import torch

from . import integrate
from . import quant as Q

_PATCHED = ("braid.model.quant", "braid.model.mlp", "braid.model.gdn", "braid.model.attention",
            "braid.model.engine")


def text_config(layers: int = 32, vocab: int = 248320, **overrides) -> dict:
    """`text_config` of the 9B member of the family (braid/model/config.py:177-205 reads these
    keys).  `layers` truncates the stack keeping the period-4 schedule; `vocab` may be reduced for
    tests (it only sizes embed_tokens / lm_head); `overrides` replace single keys (CPU-sized
    stacks in the host tests)."""
    cfg = {
        "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": layers,
        "layer_types": ["full_attention" if i % 4 == 3 else "linear_attention"
                        for i in range(layers)],
        "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 256,
        "attn_output_gate": True, "attention_bias": False, "rms_norm_eps": 1e-6,
        "vocab_size": vocab, "tie_word_embeddings": False, "hidden_act": "silu",
        "dtype": "bfloat16",
        "rope_parameters": {"rope_type": "default", "rope_theta": 1e7,
                            "partial_rotary_factor": 0.25, "mrope_section": [11, 11, 10],
                            "mrope_interleaved": True},
        "linear_num_value_heads": 32, "linear_num_key_heads": 16,
        "linear_value_head_dim": 128, "linear_key_head_dim": 128, "linear_conv_kernel_dim": 4,
        "mlp_only_layers": [], "mamba_ssm_dtype": "float32", "mtp_num_hidden_layers": 0,
    }
    cfg.update(overrides)
    return cfg


def random_checkpoint(cfg_dict: dict, device, dtype: torch.dtype = torch.bfloat16, seed: int = 0):
    """A `Checkpoint` as the reference's loader would hand to `Engine.from_checkpoint`.

    Projection weights ~ N(0, 0.02) in `dtype`; plain norms are the folded fp32 `1 + W` with
    W ~ N(0, 0.02); the gated norm's gamma is stored directly (fp32, near 1); `A` is fp32 and
    strictly negative (`-exp(A_log)`, A_log ~ U(-4, -1) as in the published files); `dt_bias`
    fp32; `conv1d` is `[C, K]`.  The loader's own `_validate` is run on the result."""
    loader = importlib.import_module("braid.model.loader")
    config = importlib.import_module("braid.model.config")
    cfg = config.ModelConfig.from_dict({"text_config": cfg_dict})
    g = torch.Generator(device=device).manual_seed(seed)
    h, gd = cfg.hidden_size, cfg.gdn

    def proj(n, k):
        return (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

    def norm(n):
        return 1.0 + torch.randn(n, generator=g, device=device, dtype=torch.float32) * 0.02

    t: dict[str, torch.Tensor] = {"embed_tokens": proj(cfg.vocab_size, h), "norm": norm(h),
                                  "lm_head": proj(cfg.vocab_size, h)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        t[p + "input_layernorm"] = norm(h)
        t[p + "post_attention_layernorm"] = norm(h)
        if cfg.is_gdn(i):
            t[p + "linear_attn.in_proj_qkv"] = proj(gd.conv_channels, h)
            t[p + "linear_attn.in_proj_z"] = proj(gd.inner_size, h)
            t[p + "linear_attn.in_proj_a"] = proj(gd.n_heads, h)
            t[p + "linear_attn.in_proj_b"] = proj(gd.n_heads, h)
            t[p + "linear_attn.out_proj"] = proj(h, gd.inner_size)
            t[p + "linear_attn.conv1d"] = (torch.randn(gd.conv_channels, gd.conv_kernel, generator=g,
                                                       device=device) * 0.2).to(dtype)
            a_log = torch.rand(gd.n_heads, generator=g, device=device) * 3.0 - 4.0
            t[p + "linear_attn.A"] = -torch.exp(a_log.float())
            t[p + "linear_attn.dt_bias"] = torch.randn(gd.n_heads, generator=g, device=device) * 0.5
            t[p + "linear_attn.norm"] = 1.0 + torch.randn(gd.head_dim, generator=g, device=device) * 0.02
        else:
            t[p + "self_attn.q_proj"] = proj(cfg.q_proj_out, h)
            t[p + "self_attn.k_proj"] = proj(cfg.kv_dim, h)
            t[p + "self_attn.v_proj"] = proj(cfg.kv_dim, h)
            t[p + "self_attn.o_proj"] = proj(h, cfg.q_dim)
            t[p + "self_attn.q_norm"] = norm(cfg.head_dim)
            t[p + "self_attn.k_norm"] = norm(cfg.head_dim)
        t[p + "mlp.gate_proj"] = proj(cfg.intermediate_size, h)
        t[p + "mlp.up_proj"] = proj(cfg.intermediate_size, h)
        t[p + "mlp.down_proj"] = proj(h, cfg.intermediate_size)
    loader._validate(cfg, t, list(range(cfg.num_hidden_layers)))
    report = loader.LoadReport(total_in_index=len(t), text=len(t), loaded=len(t),
                               layers_loaded=tuple(range(cfg.num_hidden_layers)))
    return loader.Checkpoint(config=cfg, tensors=t, report=report)


# -- switching the reference between its stock path and these kernels ---------------------------
_SAVED: dict[tuple[str, str], object] = {}


def _swap(mod_name: str, cls_name: str, attrs: tuple[str, ...], fn, done: list[str]) -> None:
    cls = getattr(sys.modules[mod_name], cls_name)
    key = (mod_name, f"{cls_name}.{attrs[0]}")
    if key not in _SAVED:
        _SAVED[key] = (cls_name, attrs, tuple(getattr(cls, a) for a in attrs))
    for a in attrs:
        setattr(cls, a, fn)
    done.append(f"{mod_name}.{cls_name}.{attrs[0]}")


def activate(fuse_mlp: bool = True, fuse_norms: bool = True) -> list[str]:
    """Rebind every module of the reference that holds quant names onto this package.  With
    `fuse_mlp`, `MLP.forward` (braid/model/mlp.py:34-49) becomes the fused four-launch form; with
    `fuse_norms`, `DecoderLayer.forward` (braid/model/layer.py:37-60) and
    `GatedDeltaNet._readout` (braid/model/gdn.py:373-387) become the forms whose norms run inside
    the quantizer of the consumer.  Engines must be BUILT after activating: their weights are
    then this package's `FP8Weight`."""
    fuse_mlp = fuse_mlp or fuse_norms      # the fused layer hands the MLP a quantized activation
    for name in _PATCHED + ("braid.model.layer",):
        importlib.import_module(name)
    names = integrate._REBOUND + ("FP8Weight", "quantize_weight", "maybe_quantize", "_FUSED",
                                  "_FUSED_STATE")
    for mod_name in _PATCHED:
        mod = sys.modules[mod_name]
        for n in names:
            if hasattr(mod, n) and (mod_name, n) not in _SAVED:
                _SAVED[(mod_name, n)] = getattr(mod, n)
    done = integrate.install_into(sys.modules["braid.model.quant"], _PATCHED[1:])
    if fuse_mlp:
        _swap("braid.model.mlp", "MLP", ("forward", "__call__"), integrate.fused_mlp_forward, done)
    if fuse_norms:
        _swap("braid.model.layer", "DecoderLayer", ("forward", "__call__"),
              integrate.fused_layer_forward, done)
        _swap("braid.model.gdn", "GatedDeltaNet", ("_readout",), integrate.fused_gdn_readout, done)
        # the final norm in front of lm_head (braid/model/engine.py:263,348): the engine module
        # holds `rms_norm` by name and uses it nowhere else
        eng_mod = sys.modules["braid.model.engine"]
        if ("braid.model.engine", "rms_norm") not in _SAVED:
            _SAVED[("braid.model.engine", "rms_norm")] = eng_mod.rms_norm
        eng_mod.rms_norm = integrate.fused_final_norm
        done.append("braid.model.engine.rms_norm")
    return done


def deactivate() -> None:
    """Undo `activate()`: the reference is stock again (engines built meanwhile keep their weights)."""
    for (mod_name, n), value in list(_SAVED.items()):
        mod = sys.modules.get(mod_name)
        if mod is None:
            continue
        if isinstance(value, tuple) and len(value) == 3 and isinstance(value[1], tuple):
            cls_name, attrs, originals = value
            for a, fn in zip(attrs, originals):
                setattr(getattr(mod, cls_name), a, fn)
        else:
            setattr(mod, n, value)
    _SAVED.clear()


# -- one arm of the decode-speed measurement -----------------------------------------------------
@dataclass
class ArmResult:
    name: str
    batch: int
    ms_per_step: float
    tok_per_s: float
    steps: int
    quantizer: str
    kernels: bool


def build_engine(ckpt, quant: str = "all", use_kernels: bool = False,
                 state_dtype: torch.dtype = torch.float16, dtype: torch.dtype = torch.bfloat16):
    """`dtype` must be the dtype the checkpoint's projection weights were created in."""
    engine_mod = importlib.import_module("braid.model.engine")
    return engine_mod.Engine.from_checkpoint(ckpt, device=ckpt["norm"].device, dtype=dtype,
                                             use_kernels=use_kernels, quant=quant,
                                             state_dtype=state_dtype)


def seed_cache(engine, cache, batch: int, prompt_len: int, seed: int = 11) -> None:
    """`prompt_len` tokens of KV and recurrent state under every row (decode_speed.py:63-74)."""
    g = torch.Generator(device=engine.device).manual_seed(seed)
    for slot in range(cache.max_slots):
        cache.reset_slot(slot)
    ids = torch.randint(0, 1000, (batch, prompt_len), generator=g, device=engine.device)
    engine.forward(ids, cache.select(list(range(batch))))


def decode_arm(name: str, engine, batch: int, steps: int, prompt_len: int = 128,
               max_len: int = 512, warm: int = 16) -> tuple[ArmResult, torch.Tensor]:
    """Graphed decode at `batch` rows, the KV bucket chosen from the live length as a scheduler
    would (the `graphed-kvbucket` arm, decode_speed.py:165-186).  Returns the timing and the
    logits of the first replayed step (for comparing arms)."""
    graph_mod = importlib.import_module("braid.model.graph")
    quant_mod = importlib.import_module("braid.model.quant")
    dev = engine.device
    cache = engine.allocate_cache(max_len, max_slots=batch)
    seed_cache(engine, cache, batch, prompt_len)
    snap = cache.snapshot()
    dec = graph_mod.GraphedDecoder(engine, cache, buckets=(batch,))
    cache.restore(snap)
    tokens = torch.full((batch, 1), 42, dtype=torch.long, device=dev)
    slots = torch.arange(batch, device=dev)

    first = dec.step(tokens, slots, live_len=prompt_len + 1).clone()
    cache.restore(snap)
    for i in range(warm):
        dec.step(tokens, slots, live_len=prompt_len + 1 + i)
    torch.cuda.synchronize(dev)
    cache.restore(snap)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        dec.step(tokens, slots, live_len=prompt_len + 1 + i)
    end.record()
    end.synchronize()
    s = start.elapsed_time(end) / 1e3 / steps
    res = ArmResult(name, batch, s * 1e3, batch / s, steps, quant_mod.fused_state(),
                    bool(engine.use_kernels))
    del dec, cache, snap
    return res, first


def logits_agreement(a: torch.Tensor, b: torch.Tensor) -> dict:
    """How close two arms' first-step logits are: the GEMM bits differ between libraries (fp32
    accumulation order), so this is a tolerance, not an identity."""
    af, bf = a.float().flatten(), b.float().flatten()
    return {"cosine": float(torch.nn.functional.cosine_similarity(af, bf, dim=0)),
            "rel_l2": float((af - bf).norm() / bf.norm()),
            "argmax_match": float((a.argmax(-1) == b.argmax(-1)).float().mean())}


def compare_arms(device, layers: int = 32, vocab: int = 248320, batch: int = 128, steps: int = 64,
                 prompt_len: int = 128, max_len: int = 512, use_kernels: bool = False,
                 bf16_arm: bool = True, seed: int = 0) -> dict:
    """The reference engine's graphed decode at `batch` rows, three ways on one GPU and one set of
    random-init weights: stock FP8 (`torch._scaled_mm` + its own quantizer), stock bf16, and FP8
    through this package.  Engines are built one after another so only one is resident."""
    import gc
    ckpt = random_checkpoint(text_config(layers, vocab), device, seed=seed)
    out: dict = {"arms": {
        "reference_fp8": "stock reference, quant=all: torch._scaled_mm + its own fused quantizer",
        "reference_bf16": "stock reference, no quantization",
        "b200_fp8_projections_only": "quantizer, prologues, grouped GEMMs and fused MLP from this "
                                     "package; norms stay torch kernels",
        "b200_fp8": "as above, plus the pre-norms and the gated readout norm fused into the "
                    "quantizer of the sublayer they feed"},
        "config": {"layers": layers, "vocab": vocab, "batch": batch, "steps": steps,
                            "prompt_len": prompt_len, "max_len": max_len, "state_dtype": "fp16",
                            "mixer_kernels": "reference CUDA kernels" if use_kernels else "torch path",
                            "weights": "random init N(0,0.02), 9B shape", "arm": "graphed-kvbucket"}}
    logits = {}

    def run(name, quant):
        eng = build_engine(ckpt, quant=quant, use_kernels=use_kernels)
        n0 = Q.launch_count()
        res, first = decode_arm(name, eng, batch, steps, prompt_len, max_len)
        out[name] = {"tok_per_s": res.tok_per_s, "ms_per_step": res.ms_per_step,
                     "quantizer": res.quantizer if quant else "n/a",
                     "step_weight_bytes": sum(eng.step_bytes().values()),
                     "b200_launches": Q.launch_count() - n0}
        logits[name] = first
        del eng
        gc.collect()
        torch.cuda.empty_cache()

    deactivate()
    run("reference_fp8", "all")
    if bf16_arm:
        run("reference_bf16", "")
    try:
        activate(fuse_norms=False)
        run("b200_fp8_projections_only", "all")
        deactivate()
        activate(fuse_norms=True)
        run("b200_fp8", "all")
    finally:
        deactivate()
    out["speedup_vs_reference_fp8"] = out["b200_fp8"]["tok_per_s"] / out["reference_fp8"]["tok_per_s"]
    out["agreement_with_reference_fp8"] = logits_agreement(logits["b200_fp8"], logits["reference_fp8"])
    if bf16_arm:
        out["speedup_vs_reference_bf16"] = out["b200_fp8"]["tok_per_s"] / out["reference_bf16"]["tok_per_s"]
        out["reference_fp8_vs_bf16_agreement"] = logits_agreement(logits["reference_fp8"],
                                                                  logits["reference_bf16"])
        out["b200_fp8_vs_bf16_agreement"] = logits_agreement(logits["b200_fp8"], logits["reference_bf16"])
    return out
