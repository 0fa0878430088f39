"""W4A16 GEMM for up to 64 rows (qe_w4_gemm through `_w4.gemm`) against fp32 x @ dequantised(W)^T,
with the GEMV's per-element bound (tests/test_gemv_w4.py:1-18 of the reference):
    |out - ref| <= 2^-8 |ref| + K 2^-24 S,   S = |x| @ |W~|^T
plus what a prefill pass relies on: bitwise repeatability, a row's result independent of the
number of rows, and agreement with the 8-row GEMV to within fp32 reordering (one bf16 ulp).
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
H, I = 5120, 17408
# the matrices of a 27B decoder block (rows x K) and the tile counts that exercise each split:
# 1030 tiles -> 2 warps per tile, 320 -> 2 (slabs of 2 groups) or 4, 2176 -> one tile per warp
SHAPES = {"gdn.in_proj": (16480, H), "attn.in_proj": (14336, H), "out_proj": (H, 6144), "down": (H, I),
          "mtp.fc": (H, 2 * H)}


@pytest.fixture(scope="module")
def api():
    from qengine_b200 import _w4
    from qengine_b200.quant import dequantize_w4, gemm, gemv, quantize_w4, quantize_w4_gate_up
    torch.backends.cuda.matmul.allow_tf32 = False
    return dict(w4=_w4, deq=dequantize_w4, gemm=gemm, gemv=gemv, q=quantize_w4, qgu=quantize_w4_gate_up)


def rand_w(M, K, scale=0.02, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(M, K, generator=g, device=DEV) * scale).to(torch.bfloat16)


def rand_x(N, K, seed=1):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(N, K, generator=g, device=DEV).to(torch.bfloat16)


def check(out, x, Wd, what, exact_min=0.9):
    ref = x.float() @ Wd.T
    bnd = 2.0 ** -8 * ref.abs() + x.shape[1] * 2.0 ** -24 * (x.float().abs() @ Wd.abs().T)
    err = (out.float() - ref).abs()
    bad = err > bnd
    assert not bad.any(), f"{what}: {int(bad.sum())} elements over bound, worst {err.max().item():.3e}"
    exact = (out.float() == ref.to(torch.bfloat16).float()).float().mean().item()
    assert exact >= exact_min, f"{what}: only {exact:.3f} of outputs equal bf16(reference)"


def bits(t):
    return t.view(torch.int16).clone()


@pytest.fixture(params=[0, 1], ids=["tcgen05", "mma_sync"])
def variant(request):
    return request.param


@pytest.mark.parametrize("name", list(SHAPES))
def test_27b_shapes(api, name, variant):
    M, K = SHAPES[name]
    gemm = lambda x, p: api["gemm"](x, p, variant=variant)
    p = api["q"](rand_w(M, K, seed=5))
    Wd = api["deq"](p)
    x = rand_x(64, K, seed=6)
    full = gemm(x, p)
    check(full, x, Wd, f"{name} N=64")
    assert torch.equal(bits(gemm(x, p)), bits(full)), "not repeatable"
    for N in (1, 8, 9, 31, 32, 33, 40, 63):
        out = gemm(x[:N].contiguous(), p)
        check(out, x[:N], Wd, f"{name} N={N}")
    # a row does not depend on how many rows there are (mma.sync: within one slab geometry,
    # N <= 32 or N > 32)
    assert torch.equal(bits(gemm(x[:40].contiguous(), p)), bits(full[:40]))
    assert torch.equal(bits(gemm(x[:7].contiguous(), p)), bits(gemm(x[:32].contiguous(), p)[:7]))
    if variant == 0:
        assert torch.equal(bits(gemm(x[:7].contiguous(), p)), bits(full[:7]))
    # the 8-row GEMV adds the same exact per-unit sums in another order: at most one bf16 ulp apart
    g = api["gemv"](x[:8].contiguous(), p).float()
    d = (full[:8].float() - g).abs()
    assert (d <= 2.0 ** -7 * g.abs() + 1e-6).all()
    assert (full[:8].float() == g).float().mean().item() > 0.97


def test_gate_up_swiglu(api, variant):
    g, u = rand_w(I, H, seed=11), rand_w(I, H, seed=12)
    p = api["qgu"](g, u)
    Wg, Wu = api["deq"](p)
    x = rand_x(64, H, seed=13)
    gemm = lambda x, p: api["gemm"](x, p, variant=variant)
    out = gemm(x, p)
    a, b = x.float() @ Wg.T, x.float() @ Wu.T
    ref = torch.nn.functional.silu(a) * b
    torch.testing.assert_close(out.float(), ref, rtol=2.0 ** -7, atol=2e-3)
    # the same epilogue as the GEMV on the same sums: nearly always the same bits
    v = api["gemv"](x[:8].contiguous(), p)
    assert (out[:8] == v).float().mean().item() > 0.97
    assert torch.equal(bits(gemm(x[:20].contiguous(), p)), bits(gemm(x[:32].contiguous(), p)[:20]))


@pytest.mark.parametrize("M,K", [(16, 256), (1, 256), (100, 512), (2368 * 16, 256), (2368 * 16 + 40, 256),
                                 (5000 * 16, 256), (148 * 16, 768), (149 * 16, 1024), (777, 1280),
                                 (148 * 128, 256), (148 * 128 + 16, 256), (300 * 128 - 40, 512),
                                 (1000, 2048), (200, 3072), (5000, 1024)])
def test_tile_counts_and_rounds(api, M, K, variant):
    """One tile, fewer tiles than SMs, exactly 16 per SM, more than 16 per SM (several rounds of the
    mma.sync kernel); one super-tile of 128 rows per SM, one more, a ragged last super-tile; few
    super-tiles, so that K is split into 2, 3 and 3 parts, the last super-tile ragged."""
    p = api["q"](rand_w(M, K, seed=21))
    Wd = api["deq"](p)
    x = rand_x(64, K, seed=22)
    for N in (3, 32, 64):
        check(api["gemm"](x[:N].contiguous(), p, variant=variant), x[:N], Wd, f"{M}x{K} N={N}")


@pytest.mark.parametrize("M,K", [(64, 128), (200, 384), (1000, 640)])
def test_odd_group_counts(api, M, K):
    """The tensor-memory kernel walks K one group at a time: any number of groups."""
    p = api["q"](rand_w(M, K, seed=23))
    Wd = api["deq"](p)
    x = rand_x(64, K, seed=24)
    for N in (1, 17, 64):
        check(api["gemm"](x[:N].contiguous(), p), x[:N], Wd, f"{M}x{K} N={N}")


def test_fp32_sums_and_strided_rows(api, variant):
    p = api["q"](rand_w(H, 6144, seed=31))
    Wd = api["deq"](p)
    big = rand_x(64, 6144 + 64, seed=32)
    x = big[:, 8:6144 + 8]  # rows 16-byte aligned, not contiguous
    out32 = torch.empty(48, H, dtype=torch.float32, device=DEV)
    api["w4"].gemm(x[:48], p.qw, p.scales, out32, H, variant=variant)
    ref = x[:48].float() @ Wd.T
    assert ((out32 - ref).abs() <= 6144 * 2.0 ** -24 * (x[:48].float().abs() @ Wd.abs().T) + 1e-6).all()
    wide = torch.zeros(48, H + 24, dtype=torch.bfloat16, device=DEV)
    api["w4"].gemm(x[:48], p.qw, p.scales, wide[:, :H], H, variant=variant)
    assert torch.equal(wide[:, :H].float(), out32.to(torch.bfloat16).float())
    assert not wide[:, H:].any()


def test_unsupported_arguments_are_refused(api):
    p = api["q"](rand_w(64, 384, seed=41))  # three groups: no slab size of the mma.sync kernel divides K
    with pytest.raises(RuntimeError):
        api["gemm"](rand_x(16, 384), p, variant=1)
    p = api["q"](rand_w(64, 512, seed=42))
    with pytest.raises(RuntimeError):
        api["gemm"](rand_x(65, 512), p)
    with pytest.raises(RuntimeError):
        api["gemm"](rand_x(16, 520)[:, 4:516], p)  # rows not 16-byte aligned
    with pytest.raises(RuntimeError):
        api["gemm"](rand_x(16, 500), api["q"](rand_w(64, 500, seed=43)))  # K != Kp
    assert api["w4"].ring_error() == 0
