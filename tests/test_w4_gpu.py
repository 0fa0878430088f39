"""W4A16 GEMV (qe_w4_gemv through `_w4`) against fp32 x @ dequantised(W)^T.

Per-element tolerance, with S = |x| @ |W~|^T in fp32 (the reference's own bound,
tests/test_gemv_w4.py:1-18 of the reference):
    |out - ref| <= 2^-8 |ref| + K 2^-24 S
(one bf16 rounding of the output plus reordering of K exact fp32 products), and at least 90 % of
the outputs must be bit-identical to bf16(fp32 reference). On top of the value checks: bitwise
repeatability, and row r of an N-row call bit-identical to the 1-row call, in every launch
configuration the boundary accepts.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
H, I, V = 5120, 17408, 248320
SHAPES_27B = {
    "gdn.in_proj_qkv": (10240, H), "gdn.in_proj_z": (6144, H), "gdn.in_proj_a/b": (48, H),
    "gdn.in_proj_fused": (16480, H), "gdn.out_proj": (H, 6144), "attn.q_proj": (12288, H),
    "attn.k/v_proj": (1024, H), "attn.in_proj_fused": (14336, H), "attn.o_proj": (H, 6144),
    "mlp.gate/up_proj": (I, H), "mlp.down_proj": (H, I), "lm_head": (V, H), "mtp.fc": (H, 2 * H),
}
# per-rank shapes of the 27B model under tensor parallelism (rows x K): t = 2, 4, 8
SHAPES_TP = {
    "t2.gdn_in": (8240, H), "t2.attn_in": (7168, H), "t2.out": (H, 3072), "t2.down": (H, 8704),
    "t4.gdn_in": (4120, H), "t4.attn_in": (3584, H), "t4.out": (H, 1536), "t4.down": (H, 4352),
    "t8.gdn_in": (2060, H), "t8.attn_in": (2048, H), "t8.out": (H, 768), "t8.down": (H, 2176),
    "t8.lm_head": (31040, H), "t8.gate_up_rows": (4352, H),
}
ODD_SHAPES = [(1, 1), (1, 128), (7, 127), (16, 129), (127, 1000), (1000, 4097), (33, 32768), (4097, 7),
              (17, 255), (100, 136)]
# every launch option the boundary accepts (the reference's names); all map onto one kernel family
CFGS = [dict(), dict(warps=4), dict(warps=16), dict(unroll=1), dict(unroll=4), dict(warps=16, unroll=1),
        dict(mode=0), dict(mode=0, ksplit=2), dict(mode=0, ksplit=7), dict(mode=2), dict(mode=2, min_units=1),
        dict(mode=2, warps=4, unroll=1), dict(variant=1), dict(pdl=False), dict(mode=3),
        dict(mode=3, blocks_per_sm=1, min_units=1), dict(mode=4), dict(mode=4, unroll=2, min_units=1),
        dict(mode=4, unroll=1, blocks_per_sm=1), dict(min_units=6), dict(min_units=64), dict(warps=8, min_units=2)]


@pytest.fixture(scope="module")
def api():
    from qengine_b200 import _w4
    from qengine_b200.quant import dequantize_w4, gemv, quantize_w4, quantize_w4_gate_up
    torch.backends.cuda.matmul.allow_tf32 = False
    return dict(w4=_w4, deq=dequantize_w4, gemv=gemv, q=quantize_w4, qgu=quantize_w4_gate_up)


def rand_w(M, K, scale=0.02, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(M, K, generator=g, device=DEV) * scale).to(torch.bfloat16)


def rand_x(N, K, seed=1):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(N, K, generator=g, device=DEV).to(torch.bfloat16)


def bound(x, Wd, ref):
    return 2.0 ** -8 * ref.abs() + x.shape[1] * 2.0 ** -24 * (x.float().abs() @ Wd.abs().T)


def check(out, ref, bnd, what):
    o = out.float()
    assert torch.equal(torch.isnan(o), torch.isnan(ref)), f"{what}: NaN pattern differs"
    inf = torch.isinf(ref)
    assert torch.equal(torch.isinf(o), inf), f"{what}: inf pattern differs"
    assert torch.equal(o[inf], ref[inf]), f"{what}: inf sign differs"
    fin = ~(torch.isnan(ref) | inf)
    err = (o - ref).abs()[fin]
    bad = err > bnd[fin]
    assert not bad.any(), f"{what}: {int(bad.sum())} elements over bound, worst {err.max().item():.3e}"
    if fin.sum() >= 8:
        exact = (o[fin] == ref[fin].to(torch.bfloat16).float()).float().mean().item()
        assert exact >= 0.9, f"{what}: only {exact:.3f} of outputs equal bf16(reference)"


def bits(t):
    return t.view(torch.int16).clone()


def test_product_dequantiser_matches_oracle_dequantiser(api):
    from util import dequant_oracle
    p = api["q"](rand_w(100, 300, seed=2))
    assert torch.equal(api["deq"](p).cpu(), dequant_oracle(p))
    pg = api["qgu"](rand_w(21, 200, seed=3), rand_w(21, 200, seed=4))
    g, u = api["deq"](pg)
    og, ou = dequant_oracle(pg)
    assert torch.equal(g.cpu(), og) and torch.equal(u.cpu(), ou)


@pytest.mark.parametrize("name", list(SHAPES_27B))
def test_27b_shapes_all_row_counts(api, name):
    M, K = SHAPES_27B[name]
    p = api["q"](rand_w(M, K, seed=5))
    Wd = api["deq"](p)
    x = rand_x(8, K, seed=6)
    ref = x.float() @ Wd.T
    bnd = bound(x, Wd, ref)
    for N in range(1, 9):
        check(api["gemv"](x[:N].contiguous(), p), ref[:N], bnd[:N], f"{name} N={N}")


@pytest.mark.parametrize("name", list(SHAPES_TP))
def test_tensor_parallel_shard_shapes(api, name):
    """The matrices a rank of a 2 / 4 / 8-way tensor-parallel engine multiplies with, at the
    engine's own launch options (default, and min_units = 6)."""
    M, K = SHAPES_TP[name]
    p = api["q"](rand_w(M, K, seed=60))
    Wd = api["deq"](p)
    x = rand_x(8, K, seed=61)
    ref = x.float() @ Wd.T
    bnd = bound(x, Wd, ref)
    for kw in (dict(), dict(min_units=6)):
        one = bits(api["gemv"](x[:1].contiguous(), p, **kw))
        for N in (1, 5, 8):
            out = api["gemv"](x[:N].contiguous(), p, **kw)
            check(out, ref[:N], bnd[:N], f"{name} N={N} {kw}")
            assert torch.equal(bits(out[:1]), one), f"{name} N={N} {kw}: row 0 depends on N"


@pytest.mark.parametrize("M,K", ODD_SHAPES)
def test_odd_shapes(api, M, K):
    p = api["q"](rand_w(M, K, seed=7))
    Wd = api["deq"](p)
    x = rand_x(8, K, seed=8)
    for N in range(1, 9):
        ref = x[:N].float() @ Wd.T
        check(api["gemv"](x[:N].contiguous(), p), ref, bound(x[:N], Wd, ref), f"{M}x{K} N={N}")


@pytest.mark.parametrize("mode,ksplit,min_units", [(0, 1, 4), (0, 2, 4), (0, 3, 4), (0, 7, 4), (0, 40, 4),
                                                  (2, 0, 1), (2, 0, 4), (-1, 0, 4), (3, 0, 1), (3, 0, 4), (4, 0, 1), (4, 0, 4)])
@pytest.mark.parametrize("warps,unroll", [(4, 1), (8, 2), (8, 4), (16, 1)])
def test_launch_configs(api, mode, ksplit, min_units, warps, unroll):
    p = api["q"](rand_w(1000, 5120, seed=9))
    Wd = api["deq"](p)
    x = rand_x(5, 5120, seed=10)
    ref = x.float() @ Wd.T
    for variant in range(4):
        for pdl in (False, True):
            out = api["gemv"](x, p, ksplit=ksplit, warps=warps, unroll=unroll, variant=variant, pdl=pdl,
                              mode=mode, min_units=min_units)
            check(out, ref, bound(x, Wd, ref), f"mode={mode} ks={ksplit} w={warps} u={unroll} v={variant}")


@pytest.mark.parametrize("kw", [dict(mode=0, ksplit=16), dict(mode=2, min_units=1)])
def test_partial_sum_scratch_left_clean(api, kw):
    """The arrival counters must be zero again after every call: repeated calls agree."""
    p = api["q"](rand_w(64, 8192, seed=11))
    Wd = api["deq"](p)
    x = rand_x(3, 8192, seed=12)
    ref = x.float() @ Wd.T
    for _ in range(20):
        check(api["gemv"](x, p, **kw), ref, bound(x, Wd, ref), f"repeat {kw}")


def test_cuda_graph_replay(api):
    p = api["q"](rand_w(1024, 5120, seed=13))
    Wd = api["deq"](p)
    x = rand_x(2, 5120, seed=14)
    out = torch.empty(2, 1024, dtype=torch.bfloat16, device=DEV)
    for kw in (dict(mode=0, ksplit=8), dict(mode=2, min_units=1), dict()):
        api["gemv"](x, p, out, **kw)  # sizes the scratch outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        api["gemv"](x, p, out, mode=0, ksplit=8)
        api["gemv"](x, p, out, mode=2, min_units=1)
        api["gemv"](x, p, out)
    for seed in range(3):
        x.copy_(rand_x(2, 5120, seed=100 + seed))
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        ref = x.float() @ Wd.T
        check(out, ref, bound(x, Wd, ref), f"graph replay {seed}")


@pytest.mark.parametrize("Iw,K", [(I, H), (37, 200), (8, 128), (1000, 4097)])
def test_swiglu_epilogue(api, Iw, K):
    p = api["qgu"](rand_w(Iw, K, seed=15), rand_w(Iw, K, seed=16))
    gd, ud = api["deq"](p)
    x = rand_x(8, K, seed=17)
    for N in range(1, 9):
        xs = x[:N].contiguous()
        g, u = xs.float() @ gd.T, xs.float() @ ud.T
        ref = torch.nn.functional.silu(g) * u
        kb = K * 2.0 ** -24
        eg, eu = kb * (xs.float().abs() @ gd.abs().T), kb * (xs.float().abs() @ ud.abs().T)
        bnd = 2.0 ** -8 * ref.abs() + 1.1 * u.abs() * eg + torch.nn.functional.silu(g).abs() * eu + 1e-30
        out = api["gemv"](xs, p)
        assert out.shape == (N, Iw)
        check(out, ref, bnd, f"swiglu {Iw}x{K} N={N}")


def test_nan_inf_rows(api):
    p = api["q"](rand_w(300, 1000, seed=18))
    Wd = api["deq"](p)
    x = rand_x(4, 1000, seed=19)
    x[1, 17] = float("nan")
    x[2, 900] = float("inf")
    x[3, 5], x[3, 6] = float("-inf"), float("inf")
    ref = x.float() @ Wd.T
    out = api["gemv"](x, p)
    check(out, ref, bound(x, Wd, ref).nan_to_num(posinf=0.0), "nan/inf")
    assert torch.isnan(out[1]).all() and not torch.isnan(out[0]).any()


@pytest.mark.parametrize("mag", [1e-30, 1e-4, 1e4, 1e30])
def test_extreme_magnitudes(api, mag):
    p = api["q"](rand_w(256, 2048, seed=20))
    Wd = api["deq"](p)
    x = (rand_x(3, 2048, seed=21).float() * mag).to(torch.bfloat16)
    ref = x.float() @ Wd.T
    check(api["gemv"](x, p), ref, bound(x, Wd, ref), f"mag {mag}")


def test_weight_extremes(api):
    W = rand_w(64, 1024, seed=22).float()
    W[0] *= 1e3
    W[1] *= 1e-3
    W[2, :128] = 0
    W[3, 5] = 50.0
    p = api["q"](W.to(torch.bfloat16))
    Wd = api["deq"](p)
    x = rand_x(2, 1024, seed=23)
    ref = x.float() @ Wd.T
    check(api["gemv"](x, p), ref, bound(x, Wd, ref), "weight extremes")


@pytest.mark.parametrize("pad,offset", [(64, 0), (3, 0), (0, 1), (8, 3)])
def test_strided_and_misaligned_views(api, pad, offset):
    M, K = 500, 1024
    p = api["q"](rand_w(M, K, seed=24))
    Wd = api["deq"](p)
    big = rand_x(4, K + pad + offset, seed=25)
    x = big[:, offset:offset + K]
    obig = torch.full((4, M + 40), 7.0, dtype=torch.bfloat16, device=DEV)
    out = obig[:, 8:8 + M]
    api["gemv"](x, p, out)
    ref = x.float() @ Wd.T
    check(out, ref, bound(x, Wd, ref), f"strided pad={pad} off={offset}")
    assert (obig[:, :8] == 7).all() and (obig[:, 8 + M:] == 7).all(), "wrote outside the out view"


def test_rejects_bad_inputs(api):
    p = api["q"](rand_w(32, 256))
    w4 = api["w4"]
    o1 = torch.empty(1, 32, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        w4.gemv(rand_x(1, 256).half(), p.qw, p.scales, o1, 32)
    with pytest.raises(RuntimeError):
        w4.gemv(rand_x(9, 256), p.qw, p.scales, torch.empty(9, 32, dtype=torch.bfloat16, device=DEV), 32)
    with pytest.raises(RuntimeError):
        w4.gemv(rand_x(1, 384), p.qw, p.scales, o1, 32)
    with pytest.raises(RuntimeError):
        w4.gemv(rand_x(1, 256), p.qw, p.scales, o1, 32, warps=3)


@pytest.mark.parametrize("M,K", [(5120, 17408), (1024, 5120), (1000, 4097), (16480, 5120)])
def test_bitwise_repeatable(api, M, K):
    p = api["q"](rand_w(M, K, seed=30))
    x = rand_x(8, K, seed=31)
    out = torch.empty(8, M, dtype=torch.bfloat16, device=DEV)
    for kw in CFGS:
        api["gemv"](x, p, out, **kw)
        first = bits(out)
        for _ in range(30):
            out.fill_(0)
            api["gemv"](x, p, out, **kw)
            assert torch.equal(bits(out), first), f"{M}x{K} {kw}: run differs bitwise"


@pytest.mark.parametrize("M,K", [(5120, 17408), (1024, 5120), (127, 1000), (16480, 5120)])
def test_row_independent_of_row_count(api, M, K):
    p = api["q"](rand_w(M, K, seed=32))
    x = rand_x(8, K, seed=33)
    for kw in CFGS:
        single = [bits(api["gemv"](x[r:r + 1].contiguous(), p, **kw)) for r in range(8)]
        for N in range(2, 9):
            out = api["gemv"](x[:N].contiguous(), p, **kw)
            for r in range(N):
                assert torch.equal(bits(out[r:r + 1]), single[r]), f"{M}x{K} {kw} N={N} row {r}"


def test_swiglu_bitwise_and_row_independent(api):
    p = api["qgu"](rand_w(I, H, seed=34), rand_w(I, H, seed=35))
    x = rand_x(8, H, seed=36)
    for kw in CFGS:
        full = bits(api["gemv"](x, p, **kw))
        for _ in range(5):
            assert torch.equal(bits(api["gemv"](x, p, **kw)), full), f"swiglu {kw} repeat"
        for r in range(8):
            assert torch.equal(bits(api["gemv"](x[r:r + 1].contiguous(), p, **kw)), full[r:r + 1]), \
                f"swiglu {kw} row {r}"


@pytest.mark.parametrize("name", list(SHAPES_27B))
def test_ring_mode_all_row_counts(api, name):
    """Both ring geometries on every 27B shape; the bounded waits of the rings must never expire."""
    M, K = SHAPES_27B[name]
    p = api["q"](rand_w(M, K, seed=50))
    Wd = api["deq"](p)
    x = rand_x(8, K, seed=51)
    ref = x.float() @ Wd.T
    bnd = bound(x, Wd, ref)
    for N in (1, 2, 5, 8):
        for mode in (3, 4):
            check(api["gemv"](x[:N].contiguous(), p, mode=mode), ref[:N], bnd[:N], f"ring mode {mode} {name} N={N}")
    assert api["w4"].ring_error() == 0


def test_linearity_at_full_size(api):
    """Size-independent property on the full lm_head shape: the kernel is linear in x up to the
    output rounding: gemv(2 x) == 2 gemv(x) bit for bit (scaling by 2 is exact in bf16/fp32)."""
    p = api["q"](rand_w(V, H, seed=40))
    x = rand_x(2, H, seed=41)
    a = api["gemv"](x, p).float()
    b = api["gemv"]((x.float() * 2).to(torch.bfloat16), p).float()
    assert torch.equal(a * 2, b)


# ---------------------------------------------------------------------------------------------
# Fused prologue: residual add + RMSNorm1p (+ embedding gather) inside the GEMV launch
# ---------------------------------------------------------------------------------------------
def _norm_ref(h, delta, w, eps):
    """bf16(h + delta) and the normed rows as the torch path computes them (fp32, one rounding)."""
    hs = (h.float() + delta.float()).to(torch.bfloat16) if delta is not None else h
    v = hs.float()
    xn = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(torch.bfloat16)
    return hs, xn


@pytest.mark.parametrize("M,K,gate_up", [(16480, H, False), (I, H, True), (4096, 512, False), (1536, 512, True),
                                         (V // 8, H, False)])
def test_fused_norm_prologue(api, M, K, gate_up):
    from util import bf16_ulp_close
    w4 = api["w4"]
    p = api["qgu"](rand_w(M, K, seed=70), rand_w(M, K, seed=71)) if gate_up else api["q"](rand_w(M, K, seed=70))
    g = torch.Generator(device=DEV).manual_seed(72)
    h = torch.randn(8, K, generator=g, device=DEV).to(torch.bfloat16)
    d = (torch.randn(8, K, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    nw = (torch.randn(K, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    for delta in (d, None):
        hs_ref, xn_ref = _norm_ref(h, delta, nw, 1e-6)
        single = None
        for N in (1, 2, 5, 7, 8):
            out = torch.empty(N, M, dtype=torch.bfloat16, device=DEV)
            h_out = torch.full((N, K), 3.0, dtype=torch.bfloat16, device=DEV)
            xn = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
            kw = dict(unroll=2) if N == 8 else {}
            w4.gemv_fused(h[:N], None if delta is None else delta[:N], nw, 1e-6, p.qw, p.scales, out, M,
                          h_out=h_out, xn_out=xn, swiglu=gate_up, **kw)
            assert torch.equal(bits(h_out), bits(hs_ref[:N])), "residual stream rows"
            ok, err = bf16_ulp_close(xn, xn_ref[:N], ulps=1)
            assert ok, f"normed rows differ by more than 1 ulp ({err})"
            # the product itself: exactly the unfused kernel on the kernel's own normed rows
            want = api["gemv"](xn, p, **kw)
            assert torch.equal(bits(out), bits(want)), f"N={N}: fused product differs from gemv(xn)"
            if single is None:
                single = bits(out[:1])
            assert torch.equal(bits(out[:1]), single), f"N={N}: row 0 depends on N"
    assert w4.ring_error() == 0


def test_norm_rows_equals_the_fused_prologue(api):
    """`norm_rows` + `gemv` must give the bits of `gemv_fused` (the engine mixes the two: fused for
    one-row passes, separate launches for verify passes, and the outputs have to agree)."""
    w4 = api["w4"]
    K, M = H, 2048
    p = api["q"](rand_w(M, K, seed=73))
    g = torch.Generator(device=DEV).manual_seed(74)
    h = torch.randn(8, K, generator=g, device=DEV).to(torch.bfloat16)
    d = (torch.randn(8, K, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    nw = (torch.randn(K, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    for kw in (dict(), dict(warps=16), dict(warps=8)):
        for N in (1, 5, 8):
            for delta in (d[:N], None):
                out_f = torch.empty(N, M, dtype=torch.bfloat16, device=DEV)
                ho_f = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
                xn_f = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
                w4.gemv_fused(h[:N], delta, nw, 1e-6, p.qw, p.scales, out_f, M, h_out=ho_f, xn_out=xn_f, **kw)
                hh = h[:N].clone()
                xn = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
                w4.norm_rows(hh, delta, nw, 1e-6, xn, h_out=hh if delta is not None else None, **kw)  # in place
                assert torch.equal(bits(xn), bits(xn_f)), f"{kw} N={N}: normed rows differ"
                if delta is not None:
                    assert torch.equal(bits(hh), bits(ho_f)), "residual rows differ"
                assert torch.equal(bits(api["gemv"](xn, p, **kw)), bits(out_f))


def test_fused_prologue_gathers_embedding_rows(api):
    w4 = api["w4"]
    Vt, K, M = 1000, 512, 1552
    p = api["q"](rand_w(M, K, seed=80))
    g = torch.Generator(device=DEV).manual_seed(81)
    table = torch.randn(Vt, K, generator=g, device=DEV).to(torch.bfloat16)
    nw = (torch.randn(K, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    tok = torch.tensor([5, 999, -1, 1000, 0, 17, 3, 3, 42], dtype=torch.int32, device=DEV)  # two out of range
    for N in (1, 4, 8):
        rows = table[tok[:N].clamp(0, Vt - 1).long()].clone()
        rows[(tok[:N] < 0) | (tok[:N] >= Vt)] = 0
        _, xn_ref = _norm_ref(rows, None, nw, 1e-6)
        out = torch.empty(N, M, dtype=torch.bfloat16, device=DEV)
        h_out = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
        xn = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
        w4.gemv_fused(table, None, nw, 1e-6, p.qw, p.scales, out, M, tok=tok, h_out=h_out, xn_out=xn)
        assert torch.equal(bits(h_out), bits(rows))
        from util import bf16_ulp_close
        assert bf16_ulp_close(xn, xn_ref, ulps=1)[0]
        assert torch.equal(bits(out), bits(api["gemv"](xn, p)))


def test_fused_prologue_rejects_what_it_cannot_serve(api):
    w4 = api["w4"]
    q = api["q"](rand_w(64, 1024, seed=83))
    h = rand_x(1, 1024)
    with pytest.raises(RuntimeError):  # h_out aliases h_in
        w4.gemv_fused(h, h.clone(), rand_x(1, 1024)[0], 1e-6, q.qw, q.scales,
                      torch.empty(1, 64, dtype=torch.bfloat16, device=DEV), 64, h_out=h)
    big = api["q"](rand_w(64, H, seed=82))
    with pytest.raises(RuntimeError):  # eight rows of 5120 do not fit beside the largest ring geometry
        w4.gemv_fused(rand_x(8, H), None, rand_x(1, H)[0], 1e-6, big.qw, big.scales,
                      torch.empty(8, 64, dtype=torch.bfloat16, device=DEV), 64, unroll=4)
    with pytest.raises(RuntimeError):  # width of h must be the padded K of the matrix
        w4.gemv_fused(rand_x(1, 512), None, rand_x(1, 512)[0], 1e-6, q.qw, q.scales,
                      torch.empty(1, 64, dtype=torch.bfloat16, device=DEV), 64)


def _block_tensors(api, Hh, Ii, Vd, seed):
    """out-projection, gate/up, down and the next in_proj of a decoder block of width Hh."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda M, K, s: api["q"](rand_w(M, K, seed=s))
    W = dict(out=mk(Hh, Vd, seed + 1), gu=api["qgu"](rand_w(Ii, Hh, seed=seed + 2), rand_w(Ii, Hh, seed=seed + 3)),
             down=mk(Hh, Ii, seed + 4), inp=mk(3 * Hh + 32, Hh, seed + 5))
    W["n1"] = (torch.randn(Hh, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    W["n2"] = (torch.randn(Hh, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    return W


def _run_block(api, W, mix, h, n, chained, **kw):
    """The four GEMVs between two mixers, either as one chain or one launch each."""
    w4 = api["w4"]
    Hh, Ii = W["down"].M, W["gu"].M
    z = lambda *sh: torch.zeros(*sh, dtype=torch.bfloat16, device=DEV)
    mo, h2, h3, act, proj, xn = z(n, Hh), z(n, Hh), z(n, Hh), z(n, Ii), z(n, W["inp"].M), z(n, Hh)
    jobs = [
        w4.job(mix[:n], W["out"].qw, W["out"].scales, mo, Hh),
        w4.job_fused(h[:n], mo, W["n1"], 1e-6, W["gu"].qw, W["gu"].scales, act, Ii, h_out=h2, swiglu=True),
        w4.job(act, W["down"].qw, W["down"].scales, mo, Hh),
        w4.job_fused(h2, mo, W["n2"], 1e-6, W["inp"].qw, W["inp"].scales, proj, W["inp"].M, h_out=h3, xn_out=xn),
    ]
    if chained:
        w4.gemv_chain(jobs, **kw)
    else:
        for j in jobs:
            w4.gemv_chain([j], **kw)
    torch.cuda.synchronize()
    return [bits(t) for t in (mo, h2, h3, act, proj, xn)]


@pytest.mark.parametrize("Hh,Ii,Vd", [(512, 1536, 512), (H, I, 6144)])
def test_chain_equals_separate_launches(api, Hh, Ii, Vd):
    W = _block_tensors(api, Hh, Ii, Vd, seed=90)
    mix, h = rand_x(8, Vd, seed=95), rand_x(8, Hh, seed=96)
    for n, kw in ((1, {}), (5, {}), (8, dict(unroll=1)), (3, dict(warps=16)), (2, dict(min_units=64))):
        want = _run_block(api, W, mix, h, n, chained=False, **kw)
        for rep in range(3):  # the grid barrier's generation counter carries over from launch to launch
            got = _run_block(api, W, mix, h, n, chained=True, **kw)
            for a, b, name in zip(got, want, ("mo", "h2", "h3", "act", "proj", "xn")):
                assert torch.equal(a, b), f"n={n} {kw} rep {rep}: {name} differs between chain and separate launches"
    assert api["w4"].ring_error() == 0


def test_chain_in_a_cuda_graph(api):
    w4 = api["w4"]
    W = _block_tensors(api, 512, 1536, 512, seed=97)
    mix, h = rand_x(4, 512, seed=98), rand_x(4, 512, seed=99)
    want = _run_block(api, W, mix, h, 4, chained=True)  # eager run: also sizes scratch and barrier words
    z = lambda *sh: torch.zeros(*sh, dtype=torch.bfloat16, device=DEV)
    mo, h2, h3, act, proj, xn = z(4, 512), z(4, 512), z(4, 512), z(4, 1536), z(4, W["inp"].M), z(4, 512)
    jobs = [
        w4.job(mix, W["out"].qw, W["out"].scales, mo, 512),
        w4.job_fused(h, mo, W["n1"], 1e-6, W["gu"].qw, W["gu"].scales, act, 1536, h_out=h2, swiglu=True),
        w4.job(act, W["down"].qw, W["down"].scales, mo, 512),
        w4.job_fused(h2, mo, W["n2"], 1e-6, W["inp"].qw, W["inp"].scales, proj, W["inp"].M, h_out=h3, xn_out=xn),
    ]
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        w4.gemv_chain(jobs)
        w4.gemv_chain(jobs[:2])
    for _ in range(5):
        for t in (mo, h2, h3, act, proj, xn):
            t.zero_()
        g.replay()
        torch.cuda.synchronize()
        # the trailing 2-job chain rewrites mo / act / h2 with the same values
        for a, b in zip([bits(t) for t in (h2, h3, act, proj, xn)], want[1:]):
            assert torch.equal(a, b)


@pytest.mark.parametrize("M,K,gate_up", [(16480, H, False), (I, H, True), (4096, 512, False), (V // 8, H, False)])
def test_fp16_activation_flavour(api, M, K, gate_up):
    """GEMVs behind an RMSNorm may take their input as fp16 (qe_w4_params::x_f16, qe_w4_norm::f16):
    the codes are then unpacked to fp16 with one shift per word. Normalised rows are numbers fp16
    holds exactly, so the fp16 flavour must give the bits of the bf16 flavour; the fused launch and
    norm_rows(xn16_out) + a GEMV on the fp16 rows must agree bit for bit for every row count."""
    w4 = api["w4"]
    p = api["qgu"](rand_w(M, K, seed=80), rand_w(M, K, seed=81)) if gate_up else api["q"](rand_w(M, K, seed=80))
    g = torch.Generator(device=DEV).manual_seed(82)
    h = torch.randn(8, K, generator=g, device=DEV).to(torch.bfloat16)
    d = (torch.randn(8, K, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    nw = (torch.randn(K, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    single = None
    for N in (1, 2, 5, 8):
        kw = dict(unroll=2) if N == 8 else {}
        o_bf = torch.empty(N, M, dtype=torch.bfloat16, device=DEV)
        o_h = torch.empty_like(o_bf)
        xn_b = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
        xn_h = torch.empty_like(xn_b)
        w4.gemv_fused(h[:N], d[:N], nw, 1e-6, p.qw, p.scales, o_bf, M, xn_out=xn_b, swiglu=gate_up, **kw)
        w4.gemv_fused(h[:N], d[:N], nw, 1e-6, p.qw, p.scales, o_h, M, xn_out=xn_h, swiglu=gate_up, f16=True, **kw)
        assert torch.equal(bits(xn_b), bits(xn_h)), "the bf16 copy of the normed rows must not change"
        # every normalised value here is far above 2^-17 in magnitude or zero: fp16 holds it exactly
        assert torch.equal(bits(o_bf), bits(o_h)), f"N={N}: fp16 flavour differs from the bf16 flavour"
        # the stand-alone norm + a GEMV on its fp16 rows
        xn2 = torch.empty(N, K, dtype=torch.bfloat16, device=DEV)
        x16 = torch.empty(N, K, dtype=torch.float16, device=DEV)
        w4.norm_rows(h[:N], d[:N], nw, 1e-6, xn2, xn16_out=x16, **kw)
        assert torch.equal(bits(xn2), bits(xn_b)) and torch.equal(x16.float(), xn_b.float())
        o_r = torch.empty_like(o_bf)
        w4.gemv_chain([w4.job(x16, p.qw, p.scales, o_r, M, swiglu=gate_up, allow_f16_x=True)], **kw)
        assert torch.equal(bits(o_r), bits(o_h)), f"N={N}: norm_rows + fp16 GEMV differs from the fused launch"
        if single is None:
            single = bits(o_h[:1])
        assert torch.equal(bits(o_h[:1]), single), f"N={N}: row 0 depends on N"
    # other block sizes and rings: each must agree with its own bf16 flavour
    for kw in (dict(warps=8), dict(variant=2), dict(variant=1), dict(unroll=1), dict(min_units=6), dict(pdl=False)):
        o_bf = torch.empty(3, M, dtype=torch.bfloat16, device=DEV)
        o_h = torch.empty_like(o_bf)
        w4.gemv_fused(h[:3], d[:3], nw, 1e-6, p.qw, p.scales, o_bf, M, swiglu=gate_up, **kw)
        w4.gemv_fused(h[:3], d[:3], nw, 1e-6, p.qw, p.scales, o_h, M, swiglu=gate_up, f16=True, **kw)
        assert torch.equal(bits(o_bf), bits(o_h)), f"{kw}: fp16 flavour differs from the bf16 flavour"
    assert w4.ring_error() == 0


def test_fp16_activations_are_not_part_of_the_reference_surface(api):
    w4 = api["w4"]
    p = api["q"](rand_w(32, 256, seed=83))
    x16 = torch.randn(1, 256, device=DEV).half()
    out = torch.empty(1, 32, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        w4.gemv(x16, p.qw, p.scales, out, 32)          # the reference rejects fp16 x; so does this mirror
    with pytest.raises(RuntimeError):                   # rows that are not 16-byte aligned
        w4.job(torch.randn(1, 264, device=DEV).half()[:, 4:260], p.qw, p.scales, out, 32, allow_f16_x=True)
    p2 = api["q"](rand_w(32, 200, seed=84))              # K != Kp
    with pytest.raises(RuntimeError):
        w4.job(torch.randn(1, 200, device=DEV).half(), p2.qw, p2.scales, out, 32, allow_f16_x=True)
