"""qe_w4_gemv_static: the W4 GEMV variant that allocates nothing.

Hosts that cannot reach the CUDA allocator at call time (a plugin called back from another
runtime, code between graph capture and replay, an embedder bound to a pool it does not own) use
this entry point; its partial-sum scratch is a fixed array inside the library. The test calls it
through the C ABI and requires bit-identical output to the regular entry point (same kernel, same
launch plan, so the tolerance is zero), on two calls in a row that reuse the shared scratch with
different inputs, and checks that an oversized shape is refused. Collected last on purpose.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(rows, K, seed, gate_up=False):
    from qengine_b200 import synth
    g = torch.Generator(device="cuda").manual_seed(seed)
    return synth.random_w4(rows, K, g, "cuda", 0.02, gate_up=gate_up)


@pytest.mark.parametrize("rows,K,kw,gate_up", [
    (5120, 6144, dict(), False),                 # large matrix: warp-private rings, partial tiles via scratch
    (64, 8192, dict(mode=0, ksplit=16), False),  # split-K grid: every tile goes through the scratch
    (1024, 5120, dict(mode=2, min_units=1), False),
    (2048, 5120, dict(), True),                  # fused SwiGLU epilogue
])
def test_static_scratch_matches_regular_entry_point(rows, K, kw, gate_up):
    from qengine_b200 import _w4
    p = _mk(rows, K, 3, gate_up)
    before = torch.cuda.memory_allocated()
    for call in range(2):  # second call finds the first call's leftovers in the shared scratch
        x = torch.randn(5, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(10 + call)).to(torch.bfloat16)
        want = torch.empty(5, p.M, dtype=torch.bfloat16, device="cuda")
        got = torch.zeros_like(want)
        (_w4.gemv_swiglu if gate_up else _w4.gemv)(x, p.qw, p.scales, want, p.M, **kw)
        inside = torch.cuda.memory_allocated()
        _w4.gemv_static(x, p.qw, p.scales, got, p.M, swiglu=gate_up, **kw)
        assert torch.cuda.memory_allocated() == inside, "the static entry point must not allocate"
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"
        del x, want, got
    assert torch.cuda.memory_allocated() <= before + (1 << 22)


def test_static_scratch_refuses_oversized_shapes():
    from qengine_b200 import _w4
    p = _mk(16 * ((1 << 14) + 8), 128, 5)  # more 16-row tiles than the fixed counter array holds
    x = torch.randn(1, 128, device="cuda").to(torch.bfloat16)
    out = torch.empty(1, p.M, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="more scratch"):
        _w4.gemv_static(x, p.qw, p.scales, out, p.M)
    _w4.gemv(x, p.qw, p.scales, out, p.M)  # the regular entry point serves it
    torch.cuda.synchronize()
