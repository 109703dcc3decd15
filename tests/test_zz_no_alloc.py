"""The quantizer entry point that takes no scratch buffer (`bq_quantize_act_static`).

It is meant for hosts that cannot allocate device memory where they call the library (a
pre-carved GPU arena, a locked allocator, a no-allocation loop, a minimal FFI shim), so the test
drives it the way such a host would: straight through the C ABI with raw pointers.  The test
itself may allocate its inputs and outputs; the entry point may not allocate anything.  Results
must equal the ordinary entry point's bit for bit — same kernels, only the home of the 16 barrier
bytes differs — on two calls in a row, because the second call inherits whatever the first left in
the shared array.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, x):
    """(codes, scale) from the ordinary entry point and from the static one, for the same input."""
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[x.dtype]
    stream = torch.cuda.current_stream().cuda_stream
    out = []
    ws = torch.zeros(16, dtype=torch.uint8, device=x.device)
    for static in (False, True):
        q = torch.full((x.numel(),), 0xAA, dtype=torch.uint8, device=x.device)
        s = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
        if static:
            rc = lib.bq_quantize_act_static(x.data_ptr(), code, x.numel(), q.data_ptr(),
                                            s.data_ptr(), stream)
        else:
            rc = lib.bq_quantize_act(x.data_ptr(), code, x.numel(), q.data_ptr(), s.data_ptr(),
                                     ws.data_ptr(), 16, stream)
        assert rc == 0, f"static={static}: status {rc}"
        out.append((q, s))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_static_scratch_matches_the_ordinary_entry_point_twice_in_a_row(lib, dtype):
    g = torch.Generator().manual_seed(123)
    # two different inputs back to back: one single-CTA size, one that needs the grid barrier
    shapes = [(8, 4096), (128, 12288)]
    for round_ in range(2):
        for shape in shapes:
            x = (torch.randn(*shape, generator=g) * (2.0 + round_)).to(dtype).cuda()
            (q_ref, s_ref), (q_new, s_new) = _call_pair(lib, x)
            assert torch.equal(s_new, s_ref), f"{dtype} {shape} round {round_}: scale differs"
            assert torch.equal(q_new, q_ref), f"{dtype} {shape} round {round_}: codes differ"
            assert s_new.item() > 0


def test_static_scratch_rejects_what_it_cannot_take(lib):
    from braid_b200 import _lib
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(64, dtype=torch.uint8, device="cuda")
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    too_many = (1 << 28) + 8
    assert lib.bq_quantize_act_static(x.data_ptr(), 1, too_many, q.data_ptr(), s.data_ptr(),
                                      None) == _lib.BQ_ERR_TOO_LARGE
    assert "capacity" in _lib.status_string(_lib.BQ_ERR_TOO_LARGE)
    assert lib.bq_quantize_act_static(None, 1, 64, q.data_ptr(), s.data_ptr(), None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_quantize_act_static(x.data_ptr(), 5, 64, q.data_ptr(), s.data_ptr(), None) == _lib.BQ_ERR_BAD_ARG
    assert lib.bq_quantize_act_static(x.data_ptr() + 2, 1, 32, q.data_ptr(), s.data_ptr(),
                                      None) == _lib.BQ_ERR_UNSUPPORTED
    torch.cuda.synchronize()
    assert int(q.max().item()) == 0, "a rejected call must not launch anything"
