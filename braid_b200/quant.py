"""FP8 W8A8 projections on B200 — the host-side mirror of `braid/model/quant.py`.

Same names, signatures and return conventions as the reference module
(braid/model/quant.py:61-298), so the sublayers that import from it
(braid/model/mlp.py:16, gdn.py:35, attention.py:27, engine.py:30-37) run
unchanged; what is underneath is replaced:

  * `quantize_act`  -> one launch of the sm_100a quantizer (`bq_quantize_act`)
    instead of nine torch kernels / the reference's two-launch kernel;
  * `fp8_matmul`    -> the hand-written tcgen05 GEMM (`bq_gemm_w8a8`) instead of
    `torch._scaled_mm`;
  * `project`       -> one quantization plus ONE grouped GEMM launch for all FP8
    weights of the call (per-weight scales kept, results identical to separate
    calls);
  * new: `silu_mul_quant`, `sigmoid_gate_quant`, `fp8_matmul_grouped`,
    `mlp_forward`, `gated_output_projection` — the fused prologues the reference
    leaves as separate bf16 kernels (braid/model/mlp.py:48, attention.py:215).

Weights are quantized with the reference's own torch spelling (load-time work,
braid/model/quant.py:118-154), on whatever device the weight lives on.

There is no CPU implementation of the kernels: activations must be CUDA
tensors, and a missing library is an error, not a silent slow path.  The only
torch arm kept is the one the reference keeps as API behaviour: a
non-contiguous (or misaligned) activation is quantized by the torch spelling,
which is exact, and `warm_fused(False)` selects that spelling on purpose for the
parity gate.
"""
from __future__ import annotations

import ctypes
import threading
from collections.abc import Iterable, Sequence
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib

GROUPS = ("mlp", "attn", "gdn", "head")


def parse_groups(spec: str | Iterable[str] | None) -> frozenset[str]:
    """`"mlp,attn"` / `("mlp", "attn")` / `"all"` / `""` -> a set of group names.

    Unknown names raise `ValueError` (braid/model/quant.py:64-80): a typo must
    not yield a run that is labelled quantized and is not.
    """
    if not spec:
        return frozenset()
    names = spec.split(",") if isinstance(spec, str) else list(spec)
    names = [n.strip() for n in names if n.strip()]
    if "all" in names:
        return frozenset(GROUPS)
    bad = sorted(set(names) - set(GROUPS))
    if bad:
        raise ValueError(f"unknown quant group(s) {bad}; known: {list(GROUPS)}")
    return frozenset(names)


FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
EPS = 1e-12

_DTYPE_CODE = {torch.float32: _lib.BQ_DTYPE_F32, torch.bfloat16: _lib.BQ_DTYPE_BF16,
               torch.float16: _lib.BQ_DTYPE_F16}


@dataclass
class FP8Weight:
    """A `[N, K]` weight held as e4m3 with one dequant scale (braid/model/quant.py:90-105).

    `scale` is a `[1, 1]` fp32 DEVICE tensor: the kernels read it through a
    pointer, so a captured graph stays valid and nothing is boxed per call.
    """

    data: torch.Tensor       # [N, K] float8_e4m3fn, row-major (K contiguous)
    scale: torch.Tensor      # [1, 1] float32
    shape: tuple[int, int]

    @property
    def nbytes(self) -> int:
        return self.data.numel() + 4


def _act_scale(t: torch.Tensor) -> torch.Tensor:
    """Per-tensor dequant scale, the obvious way (braid/model/quant.py:108-115)."""
    return (t.detach().float().abs().amax() / FP8_MAX).clamp(min=EPS).reshape(1, 1)


def _weight_scale(t: torch.Tensor) -> torch.Tensor:
    """Same value without an fp32 image of the weight (braid/model/quant.py:118-130)."""
    t = t.detach()
    return ((torch.maximum(t.amax().abs(), t.amin().abs()).float() / FP8_MAX)
            .clamp(min=EPS).reshape(1, 1))


# Largest fp32 temporary `quantize_weight` builds at once (braid/model/quant.py:136).
_CAST_CHUNK_BYTES = 256 * 2 ** 20


def quantize_weight(w: torch.Tensor) -> FP8Weight:
    """`[N, K]` -> e4m3 + one per-tensor scale, once, at load (braid/model/quant.py:139-154)."""
    if w.dim() != 2:
        raise ValueError(f"expected a 2-D weight, got {tuple(w.shape)}")
    N, K = w.shape
    if K % 16 or N % 16:
        raise ValueError(
            f"_scaled_mm needs both weight dims to be multiples of 16; got "
            f"[{N}, {K}]. Leave this projection in bf16.")
    scale = _weight_scale(w)
    data = torch.empty((N, K), dtype=FP8, device=w.device)
    rows = max(1, min(N, _CAST_CHUNK_BYTES // (K * 4)))
    for i in range(0, N, rows):
        band = w[i:i + rows]
        data[i:i + rows] = (band.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return FP8Weight(data=data, scale=scale, shape=(N, K))


# ---------------------------------------------------------------------------
# library state
# ---------------------------------------------------------------------------
_FUSED = None                 # the loaded ctypes library, or None when switched off
_FUSED_STATE = "not tried"
_LOCK = threading.Lock()

# Scratch for the kernels: 16-byte slots (amax word, two barrier counters, a
# sticky status word), zeroed once and returned to zero by the kernels.  Calls
# take slots round-robin so that launches in flight on different streams do not
# share barrier words.
_SLOTS = 256
# From this many elements on (beyond what the one-launch prologue quantizers hold in registers)
# the SiLU*mul and sigmoid-gate quantizers run as two launches: product + scale, then the cast.
_TWO_LAUNCH_FROM = 1 << 22
_SLOT_BYTES = 64
_scratch: dict[int, torch.Tensor] = {}
_next_slot: dict[int, int] = {}
_launches = 0      # kernels of this library launched (or captured) so far


def launch_count() -> int:
    """How many kernels of this library have been launched or captured by this process."""
    return _launches


def warm_fused(enable: bool = True) -> bool:
    """Load the kernel library (and its scratch) up front, or switch it off.

    Same contract as braid/model/quant.py:161-201: call it before any CUDA-graph
    capture; `warm_fused(False)` forces the torch spelling for the parity gate;
    the return value says whether the kernels are active and `fused_state()`
    gives the one-line report.  Unlike the reference, a library that cannot be
    loaded RAISES: there is no slower arm that would make a benchmark look
    plausible without the kernels.
    """
    global _FUSED, _FUSED_STATE
    if not enable:
        _FUSED, _FUSED_STATE = None, "disabled by caller"
        return False
    if _FUSED is not None:
        return True
    try:
        lib = _lib.load()
    except Exception as e:
        _FUSED = None
        _FUSED_STATE = f"unavailable: {type(e).__name__}: {str(e).split(chr(10), 1)[0][:120]}"
        raise
    _FUSED, _FUSED_STATE = lib, "active"
    if torch.cuda.is_available():
        _scratch_for(torch.cuda.current_device())
    return True


def fused_state() -> str:
    """One line on whether the kernels are running (braid/model/quant.py:204-206)."""
    return _FUSED_STATE


def _require_lib():
    """The loaded library; loading is attempted on first use and failure raises.

    `warm_fused(False)` only selects the torch spelling of the QUANTIZERS (the
    parity arm); the GEMM has no torch arm here and always needs the library.
    """
    if _FUSED is not None:
        return _FUSED
    if _FUSED_STATE == "disabled by caller":
        lib = _lib.load()
        if torch.cuda.is_available():
            _scratch_for(torch.cuda.current_device())
        return lib
    warm_fused(True)
    return _FUSED


def _quantizers_off() -> bool:
    return _FUSED is None and _FUSED_STATE == "disabled by caller"


def _scratch_for(device_index: int) -> torch.Tensor:
    buf = _scratch.get(device_index)
    if buf is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("braid_b200: call warm_fused() before CUDA-graph capture "
                               "(the kernel scratch cannot be created inside a capture)")
        with _LOCK:
            buf = _scratch.get(device_index)
            if buf is None:
                buf = torch.zeros(_SLOTS * _SLOT_BYTES, dtype=torch.uint8,
                                  device=torch.device("cuda", device_index))
                torch.cuda.synchronize(device_index)
                _scratch[device_index] = buf
                _next_slot[device_index] = 0
    return buf


def _take_slot(device: torch.device) -> int:
    """Device address of the next scratch slot of this device."""
    global _launches
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _scratch_for(idx)
    with _LOCK:
        _launches += 1
        slot = _next_slot[idx]
        _next_slot[idx] = (slot + 1) % _SLOTS
    return buf.data_ptr() + slot * _SLOT_BYTES


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def device_status(device: torch.device | int | None = None) -> int:
    """Synchronise and return the sticky status of every scratch slot (0 = clean).

    A non-zero value means a bounded device-side wait ran out at some point
    since the last check.  Never call this during capture.
    """
    if device is None:
        idx = torch.cuda.current_device()
    elif isinstance(device, int):
        idx = device
    else:
        idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _scratch.get(idx)
    if buf is None:
        return 0
    torch.cuda.synchronize(idx)
    words = buf.view(torch.int32).view(_SLOTS, _SLOT_BYTES // 4)[:, 3]
    bad = int(words.max().item())
    if bad:
        words.zero_()
    # launches that take no scratch (the cast pass) raise a word inside the library
    own = ctypes.c_int(0)
    with torch.cuda.device(idx):
        _lib.check(_require_lib().bq_scratchless_status(ctypes.byref(own)), "scratchless_status")
    return bad or int(own.value)


def set_option(key: str, value: int) -> None:
    """Tuning switch of the library (`decode_split_k`, `decode_stages`, `quant_block`, ...)."""
    _lib.check(_require_lib().bq_set_option(key.encode(), int(value)), f"set_option({key})")


def last_gemm_launch() -> dict:
    """What the last GEMM call of this thread launched (kernel, grid, split, stages, smem, tile)."""
    out = (ctypes.c_int64 * 6)()
    _lib.check(_require_lib().bq_last_gemm_launch(out), "last_gemm_launch")
    return {"kernel": {0: "stream", 2: "pair"}.get(int(out[0]), "?"),
            "grid": out[1], "split": out[2],
            "stages": out[3], "smem": out[4], "mma_n": out[5]}


# ---------------------------------------------------------------------------
# activation quantization
# ---------------------------------------------------------------------------
def _torch_quantize(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The reference spelling, braid/model/quant.py:228-229."""
    scale = _act_scale(x)
    return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8), scale


def _check_cuda(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda:
        raise RuntimeError(f"{what}: braid_b200 kernels run on CUDA tensors only "
                           f"(got a {x.device.type} tensor); there is no CPU path")


def quantize_act(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """`[M, K]` (any shape) -> e4m3 codes of the same shape plus a `[1, 1]` fp32 scale.

    Dynamic, per call; bit-identical to the torch spelling on the same device
    (braid/model/quant.py:209-229).  Contiguous CUDA activations of fp32 / bf16 /
    fp16 take the one-launch kernel; a non-contiguous or 16-byte-misaligned view
    takes the torch spelling, as the reference does (`tests/test_quant.py:424-449`).
    """
    _check_cuda(x, "quantize_act")
    if _quantizers_off():
        return _torch_quantize(x)
    lib = _require_lib()
    code = _DTYPE_CODE.get(x.dtype)
    if code is None:
        raise ValueError(f"activation must be fp32, bf16 or fp16, got {x.dtype}")
    if x.numel() == 0:
        raise ValueError("x must not be empty")
    if not x.is_contiguous() or x.data_ptr() % 16:
        return _torch_quantize(x)
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    scale = torch.empty((1, 1), dtype=torch.float32, device=x.device)
    rc = lib.bq_quantize_act(x.data_ptr(), code, x.numel(), q.data_ptr(), scale.data_ptr(),
                             _take_slot(x.device), 16, _stream_ptr(x.device))
    _lib.check(rc, "quantize_act")
    return q, scale


def quantize_act_after(x: torch.Tensor, flag: torch.Tensor, seen: torch.Tensor,
                       count: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`quantize_act` of a gathered buffer that other ranks store into: the kernel itself waits
    (bounded) until the one-word counter `flag` has advanced by `count` beyond `seen`, then
    quantizes, and advances `seen`.  A wait that runs out shows in `device_status()`."""
    _check_cuda(x, "quantize_act_after")
    lib = _require_lib()
    code = _DTYPE_CODE.get(x.dtype)
    if code is None or not x.is_contiguous() or x.data_ptr() % 16 or x.numel() == 0:
        raise ValueError("the gathered buffer must be a contiguous, 16-byte aligned fp32/bf16/fp16 tensor")
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    scale = torch.empty((1, 1), dtype=torch.float32, device=x.device)
    rc = lib.bq_quantize_act_after(x.data_ptr(), code, x.numel(), q.data_ptr(), scale.data_ptr(),
                                   flag.data_ptr(), seen.data_ptr(), count,
                                   _take_slot(x.device), 16, _stream_ptr(x.device))
    _lib.check(rc, "quantize_act_after")
    return q, scale


def silu_mul_quant(gate: torch.Tensor, up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """`quantize_act(F.silu(gate) * up)` in one launch, without materialising the product.

    Bit-identical to the two-kernel bf16 spelling followed by the quantizer
    (braid/model/mlp.py:48-49).  `gate` and `up` are `[..., I]` with a contiguous
    last axis; they may be two column blocks of one `[M, 2I]` buffer.
    """
    _check_cuda(gate, "silu_mul_quant")
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    if _quantizers_off():
        return _torch_quantize(F.silu(gate) * up)
    lib = _require_lib()
    code = _DTYPE_CODE.get(gate.dtype)
    if code is None:
        raise ValueError(f"activation must be fp32, bf16 or fp16, got {gate.dtype}")
    cols = gate.shape[-1]
    g2, u2 = _as_rows(gate, cols), _as_rows(up, cols)
    rows = g2.shape[0]
    scale = torch.empty((1, 1), dtype=torch.float32, device=gate.device)
    if rows * cols >= _TWO_LAUNCH_FROM:
        # prefill sizes: the product and its scale in one launch (no grid-wide wait), then the
        # cast pass -- the one-launch form would evaluate silu twice over its two passes
        h = torch.empty((rows, cols), dtype=gate.dtype, device=gate.device)
        rc = lib.bq_silu_mul_dense_scale(g2.data_ptr(), u2.data_ptr(), code, rows, cols, g2.stride(0),
                                         u2.stride(0), h.data_ptr(), scale.data_ptr(),
                                         _take_slot(gate.device), 16, _stream_ptr(gate.device))
        _lib.check(rc, "silu_mul_dense_scale")
        return cast_act(h, scale).reshape(*gate.shape[:-1], cols), scale
    q = torch.empty((rows, cols), dtype=FP8, device=gate.device)
    rc = lib.bq_silu_mul_quant(g2.data_ptr(), u2.data_ptr(), code, rows, cols,
                               g2.stride(0), u2.stride(0), q.data_ptr(), scale.data_ptr(),
                               _take_slot(gate.device), 16, _stream_ptr(gate.device))
    _lib.check(rc, "silu_mul_quant")
    return q.reshape(*gate.shape[:-1], cols), scale


def _silu_mul_args(gate: torch.Tensor, up: torch.Tensor, what: str):
    _check_cuda(gate, what)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    code = _DTYPE_CODE.get(gate.dtype)
    if code is None:
        raise ValueError(f"activation must be fp32, bf16 or fp16, got {gate.dtype}")
    cols = gate.shape[-1]
    return code, cols, _as_rows(gate, cols), _as_rows(up, cols)


def silu_mul_scale(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The `[1, 1]` scale `quantize_act(F.silu(gate) * up)` would return, without the codes.

    First half of the column-parallel MLP's exchange: every rank takes the scale of its own
    column shard, a MAX all-reduce over the ranks turns it into the scale of the whole
    intermediate (max is exact), and `silu_mul_cast` casts the shard with it."""
    code, cols, g2, u2 = _silu_mul_args(gate, up, "silu_mul_scale")
    if _quantizers_off():
        return _act_scale(F.silu(gate) * up)
    lib = _require_lib()
    scale = torch.empty((1, 1), dtype=torch.float32, device=gate.device)
    rc = lib.bq_silu_mul_scale(g2.data_ptr(), u2.data_ptr(), code, g2.shape[0], cols,
                               g2.stride(0), u2.stride(0), scale.data_ptr(),
                               _take_slot(gate.device), 16, _stream_ptr(gate.device))
    _lib.check(rc, "silu_mul_scale")
    return scale


def silu_mul_cast(gate: torch.Tensor, up: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 codes of `F.silu(gate) * up` under a scale decided elsewhere (a `[1, 1]` fp32 device
    tensor): `clamp(h / scale, +-448)` cast, the second half of `silu_mul_quant`."""
    code, cols, g2, u2 = _silu_mul_args(gate, up, "silu_mul_cast")
    if scale.dtype is not torch.float32 or scale.numel() != 1 or not scale.is_cuda:
        raise ValueError("scale must be a one-element fp32 CUDA tensor")
    if _quantizers_off():
        h = F.silu(gate) * up
        return (h.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    lib = _require_lib()
    global _launches
    _launches += 1
    q = torch.empty((g2.shape[0], cols), dtype=FP8, device=gate.device)
    rc = lib.bq_silu_mul_cast(g2.data_ptr(), u2.data_ptr(), code, g2.shape[0], cols,
                              g2.stride(0), u2.stride(0), scale.data_ptr(), q.data_ptr(),
                              _stream_ptr(gate.device))
    _lib.check(rc, "silu_mul_cast")
    return q.reshape(*gate.shape[:-1], cols)


def sigmoid_gate_quant(o: torch.Tensor, gate: torch.Tensor,
                       heads: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """`quantize_act(o * torch.sigmoid(gate))` in one launch (braid/model/attention.py:215-216).

    `o` is `[..., H*D]`.  `gate` is either a dense tensor of the same shape or the
    strided per-head view `[..., H, D]` the attention layer gets from
    `qg.view(B, T, H, 2*D).chunk(2, dim=-1)` (braid/model/attention.py:177), which
    is read in place — no `reshape` copy.
    """
    _check_cuda(o, "sigmoid_gate_quant")
    if _quantizers_off():
        return _torch_quantize(o * torch.sigmoid(gate.reshape(o.shape)))
    lib = _require_lib()
    code = _DTYPE_CODE.get(o.dtype)
    if code is None or gate.dtype != o.dtype:
        raise ValueError("o and gate must share one of fp32, bf16, fp16")
    cols = o.shape[-1]
    o2 = _as_rows(o, cols)
    rows = o2.shape[0]
    if gate.dim() == o.dim() + 1 and gate.shape[-1] * gate.shape[-2] == cols:
        # [..., H, D] view: rows must be uniformly strided, D contiguous
        D = gate.shape[-1]
        g3 = gate.reshape(rows, gate.shape[-2], D) if gate.is_contiguous() else \
            _rows_view_3d(gate, rows)
        if g3.stride(2) != 1:
            g3 = g3.contiguous()
        ld_gate, chunk, chunk_stride, gptr = g3.stride(0), D, g3.stride(1), g3.data_ptr()
        keep = g3
    else:
        if gate.shape != o.shape:
            raise ValueError(f"gate shape {tuple(gate.shape)} does not match o {tuple(o.shape)}")
        g2 = _as_rows(gate, cols)
        ld_gate, chunk, chunk_stride, gptr = g2.stride(0), cols, 0, g2.data_ptr()
        keep = g2
    scale = torch.empty((1, 1), dtype=torch.float32, device=o.device)
    if rows * cols >= _TWO_LAUNCH_FROM:
        # prefill sizes: product and scale in one launch, then the cast pass (see silu_mul_quant)
        h = torch.empty((rows, cols), dtype=o.dtype, device=o.device)
        rc = lib.bq_sigmoid_mul_dense_scale(o2.data_ptr(), gptr, code, rows, cols, o2.stride(0), ld_gate,
                                            chunk, chunk_stride, h.data_ptr(), scale.data_ptr(),
                                            _take_slot(o.device), 16, _stream_ptr(o.device))
        del keep
        _lib.check(rc, "sigmoid_mul_dense_scale")
        return cast_act(h, scale).reshape(*o.shape[:-1], cols), scale
    q = torch.empty((rows, cols), dtype=FP8, device=o.device)
    rc = lib.bq_sigmoid_gate_quant(o2.data_ptr(), gptr, code, rows, cols, o2.stride(0), ld_gate,
                                   chunk, chunk_stride, q.data_ptr(), scale.data_ptr(),
                                   _take_slot(o.device), 16, _stream_ptr(o.device))
    del keep
    _lib.check(rc, "sigmoid_gate_quant")
    return q.reshape(*o.shape[:-1], cols), scale


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """`F.silu(gate) * up` (braid/model/mlp.py:48) as one kernel, bit for bit: silu in fp32
    rounded to the activation type, product in fp32 rounded again.  For the places that want the
    product dense (an unquantized down projection); the quantized path never materialises it."""
    code, cols, g2, u2 = _silu_mul_args(gate, up, "silu_mul")
    if _quantizers_off():
        return F.silu(gate) * up
    rows = g2.shape[0]
    h = torch.empty((rows, cols), dtype=gate.dtype, device=gate.device)
    _lib.check(_require_lib().bq_silu_mul(g2.data_ptr(), u2.data_ptr(), code, rows, cols, g2.stride(0),
                                          u2.stride(0), h.data_ptr(), _stream_ptr(gate.device)),
               "silu_mul")
    return h.reshape(*gate.shape[:-1], cols)


def sigmoid_mul(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """`o * torch.sigmoid(gate)` (braid/model/attention.py:215) as one kernel, bit for bit;
    `gate` dense and of `o`'s shape."""
    _check_cuda(o, "sigmoid_mul")
    code = _DTYPE_CODE.get(o.dtype)
    if code is None or gate.dtype != o.dtype or gate.shape != o.shape:
        raise ValueError("o and gate must share shape and one of fp32, bf16, fp16")
    if _quantizers_off():
        return o * torch.sigmoid(gate)
    cols = o.shape[-1]
    o2, g2 = _as_rows(o, cols), _as_rows(gate, cols)
    rows = o2.shape[0]
    out = torch.empty((rows, cols), dtype=o.dtype, device=o.device)
    _lib.check(_require_lib().bq_sigmoid_mul(o2.data_ptr(), g2.data_ptr(), code, rows, cols, o2.stride(0),
                                             g2.stride(0), cols, 0, out.data_ptr(),
                                             _stream_ptr(o.device)), "sigmoid_mul")
    return out.reshape(*o.shape[:-1], cols)


# ---------------------------------------------------------------------------
# norms fused into the quantizer of their consumer
# ---------------------------------------------------------------------------
class QuantizedActivation:
    """An activation that arrives already quantized: e4m3 codes `[rows, K]`, its `[1, 1]` scale
    and, when a consumer still needs it unquantized (bf16 weights in a mixed `project`), the dense
    tensor.  Carries `shape` / `dtype` / `device` of the activation it stands for, which is all
    the reference's mixers read from their input before handing it to `project`
    (braid/model/gdn.py:239-255, braid/model/attention.py:168-173)."""

    __slots__ = ("q", "scale", "dense", "shape", "dtype", "device")

    def __init__(self, q, scale, shape, dtype, dense=None):
        self.q, self.scale, self.dense = q, scale, dense
        self.shape, self.dtype, self.device = torch.Size(shape), dtype, q.device

    def dim(self) -> int:
        return len(self.shape)

    def require_dense(self) -> torch.Tensor:
        if self.dense is None:
            raise ValueError("this activation was produced without its dense form "
                             "(ask the norm for it: keep_dense=True)")
        return self.dense


def attach_quantized(dense: torch.Tensor, qa: "QuantizedActivation") -> torch.Tensor:
    """Let an ordinary tensor carry its own quantization: `linear(dense, fp8_weight)` then skips
    the quantizer and multiplies the attached codes.  For call sites that cannot be handed a
    `QuantizedActivation` because other code reads the tensor too (the engine's final norm,
    braid/model/engine.py:263,348).  The attachment is ignored once the tensor has been modified
    in place."""
    dense._bq_quantized = (qa.q, qa.scale, dense._version)
    return dense


def _attached(x) -> tuple | None:
    pre = getattr(x, "_bq_quantized", None)
    if pre is None or pre[2] != x._version or pre[0].shape[-1] != x.shape[-1] \
            or pre[0].numel() != x.numel():
        return None
    return pre


def torch_rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """The reference's spelling (braid/model/norm.py:31-45): fp32 norm, one cast back."""
    return F.rms_norm(x.float(), (x.shape[-1],), gamma, eps).type_as(x)


def torch_rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, gamma: torch.Tensor,
                         eps: float) -> torch.Tensor:
    """The reference's gated form (braid/model/norm.py:48-71): normalise, round, gamma, silu(gate)."""
    dt = x.dtype
    xf = F.rms_norm(x.float(), (x.shape[-1],), None, eps)
    return ((gamma * xf.to(dt)) * F.silu(gate.float())).to(dt)


def rms_norm_quant(x: torch.Tensor, gamma: torch.Tensor, eps: float,
                   keep_dense: bool = False) -> QuantizedActivation:
    """`quantize_act(rms_norm(x, gamma, eps))` in one launch (braid/model/layer.py:49,59 feeding
    `project` / the MLP).  Bit-identical to the two steps.  More rows than fit on the device at
    once (prefill) take two launches: the norm with rows looped per CTA, which also leaves the
    scale, and the cast pass; inputs with odd strides run the two torch-spelled steps."""
    _check_cuda(x, "rms_norm_quant")
    K = x.shape[-1]
    code = _DTYPE_CODE.get(x.dtype)
    if code is None:
        raise ValueError(f"activation must be fp32, bf16 or fp16, got {x.dtype}")
    if gamma.dtype is not torch.float32 or gamma.numel() != K:
        raise ValueError("gamma must be an fp32 vector of the activation's width")
    if not _quantizers_off() and x.numel() and K % 4 == 0 and gamma.is_contiguous():
        lib = _require_lib()
        x2 = _as_rows(x, K)
        rows = x2.shape[0]
        q = torch.empty((rows, K), dtype=FP8, device=x.device)
        scale = torch.empty((1, 1), dtype=torch.float32, device=x.device)
        h = torch.empty((rows, K), dtype=x.dtype, device=x.device) if keep_dense else None
        rc = lib.bq_rmsnorm_quant(x2.data_ptr(), code, rows, K, x2.stride(0), gamma.data_ptr(),
                                  float(eps), h.data_ptr() if keep_dense else None, K, q.data_ptr(),
                                  scale.data_ptr(), _take_slot(x.device), 16, _stream_ptr(x.device))
        if rc not in (_lib.BQ_ERR_TOO_LARGE, _lib.BQ_ERR_UNSUPPORTED):
            _lib.check(rc, "rms_norm_quant")
            return QuantizedActivation(q, scale, x.shape, x.dtype,
                                       h.reshape(x.shape) if keep_dense else None)
        if rc == _lib.BQ_ERR_TOO_LARGE:
            global _launches
            _launches -= 1            # the refused call launched nothing
            # prefill: more rows than CTAs can wait for one another -- rows looped per CTA, h and
            # its scale from one launch with no grid-wide wait, then the cast pass
            if h is None:
                h = torch.empty((rows, K), dtype=x.dtype, device=x.device)
            rc = lib.bq_rmsnorm_scale(x2.data_ptr(), code, rows, K, x2.stride(0), gamma.data_ptr(),
                                      float(eps), h.data_ptr(), K, scale.data_ptr(),
                                      _take_slot(x.device), 16, _stream_ptr(x.device))
            if rc != _lib.BQ_ERR_UNSUPPORTED:
                _lib.check(rc, "rms_norm_scale")
                q = cast_act(h, scale)
                return QuantizedActivation(q, scale, x.shape, x.dtype,
                                           h.reshape(x.shape) if keep_dense else None)
    h = torch_rms_norm(x, gamma, eps)
    q, scale = quantize_act(h.reshape(-1, K))
    return QuantizedActivation(q, scale, x.shape, x.dtype, h if keep_dense else None)


def gated_rms_norm_quant(y: torch.Tensor, z: torch.Tensor, gamma: torch.Tensor, eps: float,
                         head_dim: int) -> QuantizedActivation:
    """`quantize_act(rms_norm_gated(y.to(z.dtype), z, gamma, eps))` in one launch: the GDN readout
    feeding out_proj (braid/model/gdn.py:373-387).  `y` is `[..., H, D]` or `[..., H*D]`, the fp32
    scan output or already of `z`'s type; `z` is `[..., H*D]`.  Returns the `[..., H*D]` activation."""
    _check_cuda(z, "gated_rms_norm_quant")
    width = z.shape[-1]
    heads = width // head_dim
    lead = z.shape[:-1]
    code = _DTYPE_CODE.get(z.dtype)
    ycode = _DTYPE_CODE.get(y.dtype)
    if code is None or ycode is None or (y.dtype != z.dtype and y.dtype is not torch.float32):
        raise ValueError("z must be fp32/bf16/fp16 and y either fp32 or z's type")
    if gamma.dtype is not torch.float32 or gamma.numel() != head_dim:
        raise ValueError("gamma must be an fp32 vector of head_dim entries")
    y2 = _as_rows(y.reshape(*lead, width) if y.shape[-1] != width else y, width)
    z2 = _as_rows(z, width)
    rows = z2.shape[0]
    if (not _quantizers_off() and rows and head_dim == 128 and heads * head_dim == width
            and heads <= 64 and gamma.is_contiguous()):
        lib = _require_lib()
        q = torch.empty((rows, width), dtype=FP8, device=z.device)
        scale = torch.empty((1, 1), dtype=torch.float32, device=z.device)
        rc = lib.bq_gated_rmsnorm_quant(y2.data_ptr(), ycode, y2.stride(0), z2.data_ptr(), code,
                                        z2.stride(0), gamma.data_ptr(), float(eps), rows, heads,
                                        head_dim, q.data_ptr(), scale.data_ptr(),
                                        _take_slot(z.device), 16, _stream_ptr(z.device))
        if rc not in (_lib.BQ_ERR_TOO_LARGE, _lib.BQ_ERR_UNSUPPORTED):
            _lib.check(rc, "gated_rms_norm_quant")
            return QuantizedActivation(q, scale, (*lead, width), z.dtype)
        if rc == _lib.BQ_ERR_TOO_LARGE:
            global _launches
            _launches -= 1            # the refused call launched nothing
            # prefill: warps stride over all (row, head) pairs, the gated activation and its
            # scale from one launch with no grid-wide wait, then the cast pass
            core = torch.empty((rows, width), dtype=z.dtype, device=z.device)
            rc = lib.bq_gated_rmsnorm_scale(y2.data_ptr(), ycode, y2.stride(0), z2.data_ptr(), code,
                                            z2.stride(0), gamma.data_ptr(), float(eps), rows, heads,
                                            head_dim, core.data_ptr(), width, scale.data_ptr(),
                                            _take_slot(z.device), 16, _stream_ptr(z.device))
            if rc != _lib.BQ_ERR_UNSUPPORTED:
                _lib.check(rc, "gated_rms_norm_scale")
                return QuantizedActivation(cast_act(core, scale), scale, (*lead, width), z.dtype)
    core = torch_rms_norm_gated(y2.to(z.dtype).reshape(-1, head_dim), z2.reshape(-1, head_dim),
                                gamma, eps).reshape(rows, width)
    q, scale = quantize_act(core)
    return QuantizedActivation(q, scale, (*lead, width), z.dtype)


def _as_rows(t: torch.Tensor, cols: int) -> torch.Tensor:
    """A `[rows, cols]` view with a contiguous last axis and one row stride (copy if needed)."""
    if t.dim() == 2 and t.stride(1) == 1:
        return t
    if t.is_contiguous():
        return t.view(-1, cols)
    try:
        v = t.view(-1, cols)
        if v.stride(1) == 1:
            return v
    except RuntimeError:
        pass
    return t.reshape(-1, cols).contiguous()


def _rows_view_3d(g: torch.Tensor, rows: int) -> torch.Tensor:
    try:
        return g.view(rows, g.shape[-2], g.shape[-1])
    except RuntimeError:
        return g.reshape(rows, g.shape[-2], g.shape[-1])


# ---------------------------------------------------------------------------
# the GEMM
# ---------------------------------------------------------------------------
def _check_gemm_inputs(xq: torch.Tensor, sx: torch.Tensor) -> None:
    _check_cuda(xq, "fp8_matmul")
    if xq.dtype is not FP8 or xq.dim() != 2:
        raise ValueError(f"xq must be a 2-D {FP8} tensor, got {xq.dtype} {tuple(xq.shape)}")
    if sx.dtype is not torch.float32 or sx.numel() != 1 or not sx.is_cuda:
        raise ValueError("sx must be a one-element fp32 CUDA tensor")


def fp8_matmul(xq: torch.Tensor, sx: torch.Tensor, w: FP8Weight,
               out_dtype: torch.dtype = torch.bfloat16,
               residual: torch.Tensor | None = None) -> torch.Tensor:
    """The GEMM alone on an already-quantized `[M, K]` activation (braid/model/quant.py:232-241).

    `(xq * sx) @ (w.data * w.scale)^T`, fp32 accumulation, `out_dtype` result.  With `residual`
    (`[M, N]`, `out_dtype`) the result is `residual + that`, the add running in the GEMM's
    epilogue with the two roundings of the separate kernels (decode sizes; larger M adds after).
    """
    if residual is None:
        return fp8_matmul_grouped(xq, sx, (w,), out_dtype=out_dtype)[0]
    _check_gemm_inputs(xq, sx)
    M, K = xq.shape
    N = w.data.shape[0]
    if residual.shape != (M, N) or residual.dtype != out_dtype or not residual.is_cuda:
        raise ValueError(f"residual must be a [{M}, {N}] {out_dtype} CUDA tensor")
    code = _DTYPE_CODE.get(out_dtype)
    if (M == 0 or code is None or residual.stride(1) != 1 or w.data.shape[1] != K
            or not w.data.is_contiguous()):
        return residual + fp8_matmul_grouped(xq, sx, (w,), out_dtype=out_dtype)[0]
    lib = _require_lib()
    if not xq.is_contiguous():
        xq = xq.contiguous()
    y = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    ws_ptr, ws_bytes = _take_slot(xq.device), 16
    rc = lib.bq_gemm_w8a8_residual(xq.data_ptr(), w.data.data_ptr(), sx.data_ptr(), w.scale.data_ptr(),
                                   residual.data_ptr(), residual.stride(0), y.data_ptr(), code,
                                   M, N, K, N, ws_ptr, ws_bytes, _stream_ptr(xq.device))
    if rc == _lib.BQ_ERR_UNSUPPORTED:
        return residual + fp8_matmul_grouped(xq, sx, (w,), out_dtype=out_dtype)[0]
    _lib.check(rc, "fp8_matmul")
    return y


def fp8_matmul_grouped(xq: torch.Tensor, sx: torch.Tensor, weights: Sequence[FP8Weight],
                       out_dtype: torch.dtype = torch.bfloat16,
                       out: Sequence[torch.Tensor] | None = None) -> list[torch.Tensor]:
    """Several weights against one quantized activation in ONE launch.

    Each weight keeps its own scale, so every result equals the separate
    `fp8_matmul` call bit for bit.  `out`, if given, holds one `[M, N_i]` tensor
    per weight (last axis contiguous; column blocks of a wider buffer are fine).
    More than 8 weights are split over several launches.
    """
    _check_gemm_inputs(xq, sx)
    lib = _require_lib()
    code = _DTYPE_CODE.get(out_dtype)
    if code is None:
        raise ValueError(f"out_dtype must be fp32, bf16 or fp16, got {out_dtype}")
    if not xq.is_contiguous():
        xq = xq.contiguous()
    M, K = xq.shape
    outs: list[torch.Tensor] = []
    for i, w in enumerate(weights):
        if not isinstance(w, FP8Weight):
            raise TypeError("fp8_matmul_grouped takes FP8Weight operands")
        if w.data.shape[1] != K:
            raise ValueError(f"weight {i} has K={w.data.shape[1]}, activation has K={K}")
        if not w.data.is_contiguous():
            raise ValueError("FP8Weight.data must be contiguous [N, K]")
        if out is not None:
            y = out[i]
            if y.shape != (M, w.data.shape[0]) or y.dtype != out_dtype or y.stride(1) != 1:
                raise ValueError(f"out[{i}] must be [{M}, {w.data.shape[0]}] {out_dtype}")
        else:
            y = torch.empty((M, w.data.shape[0]), dtype=out_dtype, device=xq.device)
        outs.append(y)
    if M == 0:
        return outs
    stream = _stream_ptr(xq.device)
    for lo in range(0, len(weights), _lib.BQ_MAX_SEGMENTS):
        ws_, ys = weights[lo:lo + _lib.BQ_MAX_SEGMENTS], outs[lo:lo + _lib.BQ_MAX_SEGMENTS]
        n = len(ws_)
        wq = (ctypes.c_void_p * n)(*[w.data.data_ptr() for w in ws_])
        sw = (ctypes.c_void_p * n)(*[w.scale.data_ptr() for w in ws_])
        yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
        Ns = (ctypes.c_int64 * n)(*[w.data.shape[0] for w in ws_])
        ld = (ctypes.c_int64 * n)(*[y.stride(0) for y in ys])
        ws_ptr, ws_bytes = _take_slot(xq.device), 16
        rc = lib.bq_gemm_w8a8_grouped(xq.data_ptr(), sx.data_ptr(), M, K, n, wq, sw, yp, Ns, ld,
                                      code, ws_ptr, ws_bytes, stream)
        _lib.check(rc, "fp8_matmul")
    return outs


def lm_head_argmax(x, w: FP8Weight, return_logits: bool = False):
    """Greedy tokens straight from the lm_head GEMM: `linear(x, w).argmax(-1)` with the per-row
    argmax taken in the GEMM's epilogue (braid/model/engine.py:349 + braid/serve/scheduler.py:346).
    `x` is `[..., K]` (a tensor, a tensor carrying its quantization, or a `QuantizedActivation`).
    Returns int64 indices of shape `x.shape[:-1]`; with `return_logits` also the logits, which are
    otherwise never written.  Exactly equal to the argmax of the logits `linear` would return."""
    *lead, K = x.shape
    if isinstance(x, QuantizedActivation):
        xq, sx, dt = x.q, x.scale, x.dtype
    else:
        pre = _attached(x)
        dt = x.dtype
        xq, sx = (pre[0].reshape(-1, K), pre[1]) if pre is not None else quantize_act(x.reshape(-1, K))
    _check_gemm_inputs(xq, sx)
    M, N = xq.shape[0], w.data.shape[0]
    code = _DTYPE_CODE.get(dt)
    if M == 0 or M > 256 or code is None or w.data.shape[1] != K or not w.data.is_contiguous():
        logits = fp8_matmul(xq, sx, w, out_dtype=dt)
        idx = logits.argmax(-1).reshape(lead)
        return (idx, logits.reshape(*lead, N)) if return_logits else idx
    lib = _require_lib()
    if not xq.is_contiguous():
        xq = xq.contiguous()
    global _launches
    _launches += 1                      # the second-stage reduction
    need = int(lib.bq_lm_head_argmax_workspace_bytes(M, N))
    partial = torch.empty(need // 8, dtype=torch.int64, device=xq.device)
    idx = torch.empty(M, dtype=torch.int64, device=xq.device)
    logits = torch.empty((M, N), dtype=dt, device=xq.device) if return_logits else None
    rc = lib.bq_lm_head_argmax(xq.data_ptr(), w.data.data_ptr(), sx.data_ptr(), w.scale.data_ptr(), code,
                               M, N, K, logits.data_ptr() if return_logits else None, N, idx.data_ptr(),
                               partial.data_ptr(), need, _take_slot(xq.device), 16,
                               _stream_ptr(xq.device))
    _lib.check(rc, "lm_head_argmax")
    idx = idx.reshape(lead)
    return (idx, logits.reshape(*lead, N)) if return_logits else idx


# A residual waiting for the output projection of a mixer: set by the caller of the mixer
# (`residual_into`), taken by the first `fp8_linear` on exactly that weight.
_PENDING_RESIDUAL: list | None = None


class residual_into:
    """`with residual_into(w, r) as slot:` — the next `linear(·, w)` inside the block returns
    `r + linear(·, w)` with the add in the GEMM epilogue, and `slot.taken` says whether it did.
    Lets the decoder layer fuse its residual add into a projection that is called deep inside the
    reference's mixer code (braid/model/gdn.py:387, braid/model/attention.py:216) without
    touching that code."""

    def __init__(self, w, residual: torch.Tensor):
        self.w, self.residual, self.taken = w, residual, False

    def __enter__(self):
        global _PENDING_RESIDUAL
        self._outer, _PENDING_RESIDUAL = _PENDING_RESIDUAL, self
        return self

    def __exit__(self, *exc):
        global _PENDING_RESIDUAL
        _PENDING_RESIDUAL = self._outer
        return False


def _claim_residual(w, lead, n, dtype):
    slot = _PENDING_RESIDUAL
    if (slot is None or slot.taken or slot.w is not w or slot.residual.dtype != dtype
            or tuple(slot.residual.shape) != (*lead, n)):
        return None
    slot.taken = True
    return slot.residual.reshape(-1, n)


def fp8_linear(x: torch.Tensor, w: FP8Weight, residual: torch.Tensor | None = None) -> torch.Tensor:
    """`F.linear(x, w)` for a single call site; leading dims preserved (braid/model/quant.py:244-252).
    `residual` (same shape as the result) is added in the GEMM epilogue."""
    *lead, K = x.shape
    N = w.shape[0]
    res2 = residual.reshape(-1, N) if residual is not None else _claim_residual(w, lead, N, x.dtype)
    if isinstance(x, QuantizedActivation):
        return fp8_matmul(x.q, x.scale, w, out_dtype=x.dtype, residual=res2).reshape(*lead, N)
    pre = _attached(x)
    xq, sx = (pre[0].reshape(-1, K), pre[1]) if pre is not None else quantize_act(x.reshape(-1, K))
    return fp8_matmul(xq, sx, w, out_dtype=x.dtype, residual=res2).reshape(*lead, N)


def linear(x: torch.Tensor, w: torch.Tensor | FP8Weight,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """Dispatch on the weight's type (braid/model/quant.py:255-257)."""
    if isinstance(w, FP8Weight):
        return fp8_linear(x, w, residual)
    y = F.linear(x.require_dense() if isinstance(x, QuantizedActivation) else x, w)
    return y if residual is None else residual + y


_DENSE_SEGMENTS = True


def set_dense_segments(enable: bool) -> None:
    """Whether `project` runs the unquantized 16-bit members of a mixed set (the GDN gates the
    reference keeps in bf16) as extra segments of its one launch (default) or through
    `F.linear`, as the reference does.  The FP8 members do not change; a 16-bit member differs
    from `F.linear` only by the summation order of its tensor-core GEMM."""
    global _DENSE_SEGMENTS
    _DENSE_SEGMENTS = bool(enable)


def _project_mixed(xq, sx, dense: torch.Tensor, weights, lead, K):
    """One launch for FP8 and 16-bit weights together, or None when the set does not qualify."""
    M = xq.shape[0]
    dt = dense.dtype
    if (not _DENSE_SEGMENTS or M == 0 or M > 256 or dt not in (torch.bfloat16, torch.float16)
            or len(weights) > _lib.BQ_MAX_SEGMENTS):
        return None
    d2 = dense.reshape(-1, K)
    if not d2.is_contiguous() or d2.data_ptr() % 16:
        return None
    for w in weights:
        if isinstance(w, FP8Weight):
            if w.data.shape[1] != K or not w.data.is_contiguous():
                return None
        elif (w.dtype != dt or w.dim() != 2 or w.shape[1] != K or w.shape[0] % 16
              or not w.is_contiguous() or w.data_ptr() % 16 or not w.is_cuda):
            return None
    lib = _require_lib()
    n = len(weights)
    raw = [w.data if isinstance(w, FP8Weight) else w for w in weights]
    outs = [torch.empty((M, r.shape[0]), dtype=dt, device=xq.device) for r in raw]
    wp = (ctypes.c_void_p * n)(*[r.data_ptr() for r in raw])
    sw = (ctypes.c_void_p * n)(*[w.scale.data_ptr() if isinstance(w, FP8Weight) else None
                                 for w in weights])
    kind = (ctypes.c_int * n)(*[0 if isinstance(w, FP8Weight) else 1 for w in weights])
    yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in outs])
    Ns = (ctypes.c_int64 * n)(*[r.shape[0] for r in raw])
    ld = (ctypes.c_int64 * n)(*[y.stride(0) for y in outs])
    if not xq.is_contiguous():
        xq = xq.contiguous()
    rc = lib.bq_project_mixed(xq.data_ptr(), sx.data_ptr(), d2.data_ptr(), _DTYPE_CODE[dt], M, K, n,
                              wp, sw, kind, yp, Ns, ld, _DTYPE_CODE[dt], _take_slot(xq.device), 16,
                              _stream_ptr(xq.device))
    if rc == _lib.BQ_ERR_UNSUPPORTED:
        return None
    _lib.check(rc, "project")
    return [y.reshape(*lead, y.shape[1]) for y in outs]


def project(x: torch.Tensor, *weights: torch.Tensor | FP8Weight) -> list[torch.Tensor]:
    """`F.linear(x, w)` for several projections that share one activation.

    The activation is quantized once (braid/model/quant.py:260-286) and all FP8 weights of
    the call go through one grouped launch.  Weights left in bf16 (GDN's a/b gates beside its
    FP8 qkv/z) ride in the same launch at decode sizes, as 16-bit tensor-core segments over
    the unquantized activation; where that does not apply (larger M, fp32 engines,
    `set_dense_segments(False)`) they take `F.linear`, as in the reference.
    """
    pre = x if isinstance(x, QuantizedActivation) else None
    if not any(isinstance(w, FP8Weight) for w in weights):
        dense = pre.require_dense() if pre is not None else x
        return [F.linear(dense, w) for w in weights]
    *lead, K = x.shape
    fp8 = [w for w in weights if isinstance(w, FP8Weight)]
    if len(fp8) < len(weights) and (pre is None or pre.dense is not None):
        if pre is not None:
            xq, sx, dense = pre.q, pre.scale, pre.dense
        else:
            dense = x
            xq, sx = quantize_act(x.reshape(-1, K))
        mixed = _project_mixed(xq, sx, dense, weights, lead, K)
        if mixed is not None:
            return mixed
        pre = QuantizedActivation(xq, sx, x.shape, x.dtype, dense)     # do not quantize twice
    if pre is not None:
        ys = iter(fp8_matmul_grouped(pre.q, pre.scale, fp8, out_dtype=pre.dtype))
    else:
        xq, sx = quantize_act(x.reshape(-1, K))
        ys = iter(fp8_matmul_grouped(xq, sx, fp8, out_dtype=x.dtype))
    out = []
    for w in weights:
        if isinstance(w, FP8Weight):
            out.append(next(ys).reshape(*lead, w.shape[0]))
        else:
            out.append(F.linear(pre.require_dense() if pre is not None else x, w))
    return out


def maybe_quantize(w: torch.Tensor, enabled: bool) -> torch.Tensor | FP8Weight:
    """Quantize if asked and if the shape allows it (braid/model/quant.py:289-298)."""
    if not enabled or w.dim() != 2:
        return w
    N, K = w.shape
    return w if (K % 16 or N % 16) else quantize_weight(w)


# ---------------------------------------------------------------------------
# gate and up in ONE launch: every MMA tile is put together from 64 gate rows and the 64 up rows
# of the same output columns (two TMA boxes per stage, read from the two weights where they lie),
# so the epilogue can form silu(gate) * up, its amax and its FP8 codes without either half ever
# being written.  The reference keeps `gate_proj` and `up_proj` as two tensors with two scales
# (braid/model/mlp.py:27-29) and so does this: nothing is repacked or copied.
# ---------------------------------------------------------------------------
_PAIR_MLP = True


def set_paired_mlp(enable: bool) -> None:
    """Use (default) or not the one-launch gate/up form and the 3-launch MLP (results are
    identical either way; off gives the four-launch form at every size)."""
    global _PAIR_MLP
    _PAIR_MLP = bool(enable)


def _pairable(gate: FP8Weight, up: FP8Weight, K: int) -> bool:
    I = gate.data.shape[0]
    return (up.data.shape == gate.data.shape and I % 64 == 0 and gate.data.shape[1] == K
            and gate.data.is_contiguous() and up.data.is_contiguous())


def gate_up_silu_quant(xq: torch.Tensor, sx: torch.Tensor, gate: FP8Weight, up: FP8Weight,
                       act_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor] | None:
    """`quantize_act(F.silu(xq @ gate^T) * (xq @ up^T))` in ONE launch (decode sizes): the two
    GEMMs run as one over the paired weight, the product and its quantization happen in the
    epilogue (braid/model/mlp.py:46-49 up to the input of down_proj).  Codes and scale are
    bit-identical to the separate GEMMs + `silu_mul_quant`.  `None` when not applicable."""
    M, K = xq.shape
    code = _DTYPE_CODE.get(act_dtype)
    if not _PAIR_MLP or _quantizers_off() or code is None or M == 0 or M > 256:
        return None
    if not _pairable(gate, up, K):
        return None
    lib = _require_lib()
    I = gate.data.shape[0]
    hq = torch.empty((M, I), dtype=FP8, device=xq.device)
    sh = torch.empty((1, 1), dtype=torch.float32, device=xq.device)
    if not xq.is_contiguous():
        xq = xq.contiguous()
    rc = lib.bq_gate_up_silu_quant_w8a8(xq.data_ptr(), sx.data_ptr(), gate.data.data_ptr(),
                                        up.data.data_ptr(), gate.scale.data_ptr(), up.scale.data_ptr(), M, I, K, code,
                                        hq.data_ptr(), sh.data_ptr(), _take_slot(xq.device), 16,
                                        _stream_ptr(xq.device))
    if rc == _lib.BQ_ERR_UNSUPPORTED:
        return None
    _lib.check(rc, "gate_up_silu_quant")
    return hq, sh


def cast_act(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 codes of `x` under a scale decided elsewhere (a `[1, 1]` fp32 device tensor): the
    cast half of `quantize_act`."""
    _check_cuda(x, "cast_act")
    code = _DTYPE_CODE.get(x.dtype)
    if _quantizers_off() or code is None or not x.is_contiguous() or x.data_ptr() % 16 or not x.numel():
        return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    lib = _require_lib()
    global _launches
    _launches += 1
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    _lib.check(lib.bq_cast_act(x.data_ptr(), code, x.numel(), scale.data_ptr(), q.data_ptr(),
                               _stream_ptr(x.device)), "cast_act")
    return q


def gate_up_silu(xq: torch.Tensor, sx: torch.Tensor, gate: FP8Weight, up: FP8Weight,
                 act_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor] | None:
    """`h = F.silu(xq @ gate^T) * (xq @ up^T)` and the quantization scale of h in ONE launch at
    prefill sizes (M > 256): gate and up never reach memory, SiLU*mul runs in the GEMM's epilogue
    (braid/model/mlp.py:46-48).  Returns `(h [M, I], scale [1, 1])`, bit-identical to the separate
    GEMMs, `F.silu(gate) * up` and `_act_scale(h)`; `None` when not applicable."""
    M, K = xq.shape
    code = _DTYPE_CODE.get(act_dtype)
    if not _PAIR_MLP or _quantizers_off() or code is None or M <= 256:
        return None
    I = gate.data.shape[0]
    if (up.data.shape != gate.data.shape or I % 16 or gate.data.shape[1] != K
            or not gate.data.is_contiguous() or not up.data.is_contiguous()):
        return None
    lib = _require_lib()
    h = torch.empty((M, I), dtype=act_dtype, device=xq.device)
    sh = torch.empty((1, 1), dtype=torch.float32, device=xq.device)
    if not xq.is_contiguous():
        xq = xq.contiguous()
    rc = lib.bq_gate_up_silu_w8a8(xq.data_ptr(), sx.data_ptr(), gate.data.data_ptr(), up.data.data_ptr(),
                                  gate.scale.data_ptr(), up.scale.data_ptr(), M, I, K, code, h.data_ptr(),
                                  I, sh.data_ptr(), _take_slot(xq.device), 16, _stream_ptr(xq.device))
    if rc == _lib.BQ_ERR_UNSUPPORTED:
        return None
    _lib.check(rc, "gate_up_silu")
    return h, sh


# ---------------------------------------------------------------------------
# column-parallel forms: the GEMM epilogue stores into every rank's gathered buffer
# ---------------------------------------------------------------------------
def _ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def enable_peer_access(local_device: torch.device, peer_index: int) -> None:
    """Allow kernels on `local_device` to touch memory of GPU `peer_index` mapped into this process."""
    lib = _require_lib()
    with torch.cuda.device(local_device):
        _lib.check(lib.bq_enable_peer_access(int(peer_index)), "enable_peer_access")


def gemm_push(xq: torch.Tensor, sx: torch.Tensor, w: FP8Weight, out_dtype: torch.dtype,
              dst_ptrs: Sequence[int], ld: int, flag_ptrs: Sequence[int]) -> None:
    """`fp8_matmul` of this rank's weight shard whose epilogue stores the `[M, N_shard]` result
    into every rank's gathered buffer (`dst_ptrs`: device addresses of this rank's first column
    in each buffer, row stride `ld`) and then signals every rank's arrival counter."""
    _check_gemm_inputs(xq, sx)
    lib = _require_lib()
    M, K = xq.shape
    rc = lib.bq_gemm_w8a8_push(xq.data_ptr(), w.data.data_ptr(), sx.data_ptr(), w.scale.data_ptr(),
                               _DTYPE_CODE[out_dtype], M, w.data.shape[0], K, len(dst_ptrs),
                               _ptr_array(dst_ptrs), ld, _ptr_array(flag_ptrs),
                               _take_slot(xq.device), 16, _stream_ptr(xq.device))
    _lib.check(rc, "gemm_push")


def gate_up_silu_push(xq: torch.Tensor, sx: torch.Tensor, gate: FP8Weight, up: FP8Weight,
                      act_dtype: torch.dtype, dst_ptrs: Sequence[int], ld: int,
                      flag_ptrs: Sequence[int], amax_ptrs: Sequence[int] | None = None) -> None:
    """This rank's slice of `F.silu(xq @ gate^T) * (xq @ up^T)` in one launch over its gate and
    up shards, stored into every rank's gathered `h` buffer, followed by the signals.  At prefill
    sizes (M > 256) `amax_ptrs` (this rank's word on every rank) also receive the slice's
    max |h| ahead of the signals, for `wait_flag_scale`."""
    _check_gemm_inputs(xq, sx)
    lib = _require_lib()
    M, K = xq.shape
    if not _pairable(gate, up, K):
        raise ValueError("gate/up shards must be two contiguous [I, K] weights, I a multiple of 64")
    rc = lib.bq_gate_up_silu_push_w8a8(xq.data_ptr(), sx.data_ptr(), gate.data.data_ptr(),
                                       up.data.data_ptr(), gate.scale.data_ptr(), up.scale.data_ptr(), M,
                                       gate.data.shape[0], K, _DTYPE_CODE[act_dtype], len(dst_ptrs),
                                       _ptr_array(dst_ptrs), ld, _ptr_array(flag_ptrs),
                                       _ptr_array(amax_ptrs) if amax_ptrs is not None else None,
                                       _take_slot(xq.device), 16, _stream_ptr(xq.device))
    _lib.check(rc, "gate_up_silu_push")


def wait_flag(flag: torch.Tensor, seen: torch.Tensor, count: int, status: torch.Tensor) -> None:
    """Stream-ordered bounded wait until the one-word counter `flag` has advanced by `count`
    beyond `seen` (then `seen += count`).  A wait that runs out sets `status` non-zero."""
    global _launches
    lib = _require_lib()
    _launches += 1
    rc = lib.bq_wait_flag(flag.data_ptr(), seen.data_ptr(), count, status.data_ptr(),
                          _stream_ptr(flag.device))
    _lib.check(rc, "wait_flag")


def wait_flag_scale(flag: torch.Tensor, seen: torch.Tensor, count: int, status: torch.Tensor,
                    words: torch.Tensor, words_are_scales: bool = False) -> torch.Tensor:
    """`wait_flag`, then the `[1, 1]` quantization scale of the gathered `h` from the ranks'
    words (one int32 per rank): max |h| of each shard (written by `gate_up_silu_push` ahead of
    its signals) or, with `words_are_scales`, each shard's scale (`word_push`) -- either way the
    scale `quantize_act` of the whole tensor returns."""
    global _launches
    lib = _require_lib()
    _launches += 1
    scale = torch.empty((1, 1), dtype=torch.float32, device=flag.device)
    rc = lib.bq_wait_flag_scale(flag.data_ptr(), seen.data_ptr(), count, status.data_ptr(),
                                words.data_ptr(), words.numel(), 1 if words_are_scales else 0,
                                scale.data_ptr(), _stream_ptr(flag.device))
    _lib.check(rc, "wait_flag_scale")
    return scale


def word_push(word: torch.Tensor, dst_ptrs: Sequence[int], flag_ptrs: Sequence[int]) -> None:
    """The 4-byte `word` (a `[1, 1]` scale) into every rank's slot for this rank, then one
    arrival on every rank's counter."""
    global _launches
    _launches += 1
    rc = _require_lib().bq_word_push(word.data_ptr(), len(dst_ptrs), _ptr_array(dst_ptrs),
                                     _ptr_array(flag_ptrs), _stream_ptr(word.device))
    _lib.check(rc, "word_push")


def cast_act_push(x: torch.Tensor, scale: torch.Tensor, dst_ptrs: Sequence[int], ld: int,
                  flag_ptrs: Sequence[int]) -> None:
    """e4m3 codes of this rank's `[M, n]` block under `scale`, stored at the same rows of every
    rank's gathered code buffer (`dst_ptrs`: device addresses of this rank's first column, row
    pitch `ld` bytes), then one arrival per rank."""
    _check_cuda(x, "cast_act_push")
    M, n = x.shape
    rc = _require_lib().bq_cast_act_push(x.data_ptr(), _DTYPE_CODE[x.dtype], M, n, x.stride(0),
                                         scale.data_ptr(), len(dst_ptrs), _ptr_array(dst_ptrs), ld,
                                         _ptr_array(flag_ptrs), _take_slot(x.device), 16,
                                         _stream_ptr(x.device))
    _lib.check(rc, "cast_act_push")


def rows_push(x: torch.Tensor, dst_ptrs: Sequence[int], ld: int, flag_ptrs: Sequence[int]) -> None:
    """This rank's `[M, n]` block, unchanged, to the same rows of every rank's gathered buffer
    (row pitch `ld` elements), then one arrival per rank."""
    _check_cuda(x, "rows_push")
    M, n = x.shape
    rc = _require_lib().bq_rows_push(x.data_ptr(), _DTYPE_CODE[x.dtype], M, n, x.stride(0),
                                     len(dst_ptrs), _ptr_array(dst_ptrs), ld, _ptr_array(flag_ptrs),
                                     _take_slot(x.device), 16, _stream_ptr(x.device))
    _lib.check(rc, "rows_push")


# ---------------------------------------------------------------------------
# fused sublayer tails (what the reference spells as separate bf16 kernels)
# ---------------------------------------------------------------------------
def mlp_forward(x: torch.Tensor, gate_proj: FP8Weight, up_proj: FP8Weight,
                down_proj: FP8Weight, residual: torch.Tensor | None = None) -> torch.Tensor:
    """The quantized branch of `MLP.forward` (braid/model/mlp.py:44-49) in 3 launches at decode
    sizes: quantize(x) -> gate and up as one GEMM (tiles put together from both weights) with
    SiLU*mul and the quantization of h in its epilogue -> down GEMM (with `residual` added in its epilogue).
    Larger M: 4 launches (quantize -> gate and up as one CTA-pair GEMM that writes h = silu(gate)*up
    and its scale -> cast of h -> down).  Unpaired shapes or `set_paired_mlp(False)`: 4 launches
    (quantize -> grouped GEMM writing gate|up into one `[M, 2I]` buffer -> SiLU*mul inside the
    quantizer of h -> down).
    Either way the result is bit-identical to the reference's nine-plus-kernel sequence built
    from the same primitives.
    """
    *lead, K = x.shape
    pre = x if isinstance(x, QuantizedActivation) else None
    x2 = None if pre is not None else x.reshape(-1, K)
    M = pre.q.shape[0] if pre is not None else x2.shape[0]
    I = gate_proj.shape[0]
    res2 = residual.reshape(-1, down_proj.shape[0]) if residual is not None else None
    if _PAIR_MLP and M <= 256 and x.device.type == "cuda":
        xq, sx = (pre.q, pre.scale) if pre is not None else quantize_act(x2)
        paired = gate_up_silu_quant(xq, sx, gate_proj, up_proj, x.dtype)
        if paired is not None:
            y = fp8_matmul(paired[0], paired[1], down_proj, out_dtype=x.dtype, residual=res2)
            return y.reshape(*lead, down_proj.shape[0])
        pre = QuantizedActivation(xq, sx, x.shape, x.dtype)     # do not quantize twice
    if _PAIR_MLP and M > 256 and x.device.type == "cuda":
        xq, sx = (pre.q, pre.scale) if pre is not None else quantize_act(x2)
        fused = gate_up_silu(xq, sx, gate_proj, up_proj, x.dtype)
        if fused is not None:
            h, sh = fused
            y = fp8_matmul(cast_act(h, sh), sh, down_proj, out_dtype=x.dtype, residual=res2)
            return y.reshape(*lead, down_proj.shape[0])
        pre = QuantizedActivation(xq, sx, x.shape, x.dtype)
    gu = torch.empty((M, 2 * I), dtype=x.dtype, device=x.device)
    halves = (gu[:, :I], gu[:, I:])
    xq, sx = (pre.q, pre.scale) if pre is not None else quantize_act(x2)
    fp8_matmul_grouped(xq, sx, (gate_proj, up_proj), out_dtype=x.dtype, out=halves)
    hq, sh = silu_mul_quant(halves[0], halves[1])
    y = fp8_matmul(hq, sh, down_proj, out_dtype=x.dtype, residual=res2)
    return y.reshape(*lead, down_proj.shape[0])


def gated_output_projection(o: torch.Tensor, gate: torch.Tensor, o_proj: FP8Weight) -> torch.Tensor:
    """`linear(o * torch.sigmoid(gate), o_proj)` (braid/model/attention.py:215-216) in 2 launches."""
    *lead, K = o.shape
    oq, so = sigmoid_gate_quant(o, gate)
    res2 = _claim_residual(o_proj, lead, o_proj.shape[0], o.dtype)
    return fp8_matmul(oq.reshape(-1, K), so, o_proj, out_dtype=o.dtype,
                      residual=res2).reshape(*lead, o_proj.shape[0])
