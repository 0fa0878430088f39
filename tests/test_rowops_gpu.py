"""Row ops and device bookkeeping through the C ABI (`_C`) against the CPU oracle.

Tolerances (bf16 has an 8-bit significand): embedding, swiglu, argmax, fused residual add and all
integer bookkeeping are exact; rmsnorm1p is within 1 bf16 ulp (only the order of the fp32 sum of
squares differs); the bf16 GEMV obeys |y - y_exact| <= 2^-8 |y_exact| + K 2^-23 sum|w x|.
"""
from __future__ import annotations

import random

import pytest
import torch

from oracle import model as OM
from oracle import spec as OS
from util import bf16_ulp_close

pytestmark = pytest.mark.gpu
dev = "cuda"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def C():
    from qengine_b200 import _C
    return _C


@pytest.mark.parametrize("V,H", [(7, 8), (1000, 1024), (248320, 1024), (33, 5120), (50, 7)])
def test_embed(C, V, H):
    tab = torch.randn(V, H, device=dev).to(BF)
    tokens = torch.tensor([3 % V, V - 1, 0, V + 5, -1], dtype=torch.int32, device=dev)
    out = torch.full((5, H), 3.0, dtype=BF, device=dev)
    C.embed(tab, tokens, out)
    for i in range(3):
        assert torch.equal(out[i], tab[tokens[i]])
    assert torch.equal(out[3:], torch.zeros_like(out[3:]))  # out of range: zeros, no fault


@pytest.mark.parametrize("rows,H", [(1, 1024), (1, 5120), (1, 1000), (8, 256), (3, 7), (1, 127), (4, 4097),
                                    (5, 512), (2, 10240)])
@pytest.mark.parametrize("scale", [1.0, 1e-3, 300.0])
def test_rmsnorm1p(C, rows, H, scale):
    x = (torch.randn(rows, H, device=dev) * scale).to(BF)
    w = (torch.randn(H, device=dev) * 0.3).to(BF)
    out = torch.empty_like(x)
    C.rmsnorm1p(x, None, w, out, 1e-6)
    ok, err = bf16_ulp_close(out.cpu(), OM.rmsnorm1p(x.cpu(), w.cpu(), 1e-6))
    assert ok, err


def test_rmsnorm1p_fused_residual_nan_and_rows(C):
    H = 1024
    h = torch.randn(4, H, device=dev).to(BF)
    d = torch.randn(4, H, device=dev).to(BF)
    d[2, 5] = float("nan")
    d[3, 0] = float("inf")
    w = torch.randn(H, device=dev).to(BF)
    h_ref = (h + d).cpu()
    h1 = h.clone()
    out = torch.empty_like(h)
    C.rmsnorm1p(h1, d, w, out, 1e-6)
    assert torch.equal(h1.cpu().nan_to_num(9.0), h_ref.nan_to_num(9.0))  # residual add exact, in place
    ok, err = bf16_ulp_close(out.cpu(), OM.rmsnorm1p(h_ref, w.cpu(), 1e-6))
    assert ok, err
    assert torch.isnan(out[2]).all() and not torch.isnan(out[:2]).any()
    # row r of a 4-row call == 1-row call, bit for bit; strided views
    for r in range(2):
        hr, o1 = h[r:r + 1].clone(), torch.empty(1, H, dtype=BF, device=dev)
        C.rmsnorm1p(hr, d[r:r + 1], w, o1, 1e-6)
        assert torch.equal(o1[0], out[r])
    wide = torch.randn(3, H + 24, device=dev).to(BF)
    ow = torch.zeros(3, H + 8, dtype=BF, device=dev)
    C.rmsnorm1p(wide[:, 8:8 + H], None, w, ow[:, :H], 1e-6)
    ok, err = bf16_ulp_close(ow[:, :H].cpu(), OM.rmsnorm1p(wide[:, 8:8 + H].cpu(), w.cpu(), 1e-6))
    assert ok and (ow[:, H:] == 0).all()


@pytest.mark.parametrize("N,K", [(1, 8), (7, 64), (127, 1000), (1000, 1024), (4097, 1024), (1024, 3584),
                                 (5120, 17408), (33, 24)])
def test_gemv_bf16(C, N, K):
    W = torch.randn(N, K, device=dev).to(BF)
    x = torch.randn(K, device=dev).to(BF)
    out = torch.empty(N, dtype=BF, device=dev)
    C.gemv_bf16(W, x, out)
    exact = W.double() @ x.double()
    bnd = 2.0 ** -8 * exact.abs() + K * 2.0 ** -23 * (W.double().abs() @ x.double().abs()) + 1e-30
    assert ((out.double() - exact).abs() <= bnd).all()


@pytest.mark.parametrize("nr", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("N,K", [(7, 64), (1000, 1024), (1024, 3584), (33, 24)])
def test_gemv_bf16_rows_bit_exact(C, nr, N, K):
    W = torch.randn(N, K, device=dev).to(BF)
    xb = torch.randn(nr, K + 16, device=dev).to(BF)
    x = xb[:, :K]
    ob = torch.empty(nr, N + 8, dtype=BF, device=dev)
    out = ob[:, :N]
    C.gemv_bf16(W, x, out)
    one = torch.empty(N, dtype=BF, device=dev)
    for r in range(nr):
        C.gemv_bf16(W, x[r].contiguous(), one)
        assert torch.equal(out[r], one), r
    xn = x.clone()
    xn[0, 3] = float("nan")
    C.gemv_bf16(W, xn, out)
    assert torch.isnan(out[0]).all() and (nr == 1 or not torch.isnan(out[1]).any())


@pytest.mark.parametrize("I", [1, 7, 127, 3584, 17408, 4097])
def test_swiglu(C, I):
    gu = (torch.randn(2 * I, device=dev) * 4).to(BF)
    if I > 1:
        gu[0] = float("-inf")
    out = torch.empty(I, dtype=BF, device=dev)
    C.swiglu(gu, out)
    g = gu.cpu()
    ref = torch.nn.functional.silu(g[:I]) * g[I:]  # bf16 silu rounds, bf16 product rounds
    ok, err = bf16_ulp_close(out.cpu(), ref)
    assert ok, err
    out3 = torch.empty(3, I, dtype=BF, device=dev)
    C.swiglu(gu.repeat(3, 1), out3)
    assert torch.equal(out3.view(torch.int16), out.expand(3, I).contiguous().view(torch.int16))


def _argmax(C, x, nb=256):
    out = torch.empty(1, dtype=torch.int32, device=dev)
    C.argmax(x, torch.empty(nb, device=dev), torch.empty(nb, dtype=torch.int32, device=dev), out)
    return int(out)


def test_argmax_rows_and_idmap(C):
    x = torch.randn(5, 248320, device=dev).to(BF)
    out = torch.empty(5, dtype=torch.int32, device=dev)
    C.argmax(x, torch.empty(5 * 256, device=dev), torch.empty(5 * 256, dtype=torch.int32, device=dev), out)
    assert out.tolist() == x.float().argmax(-1).tolist()
    # pruned vocabulary through the id map, on a strided view of a wider logits buffer
    ids = (torch.arange(49152, dtype=torch.int32, device=dev) * 3 + 1)
    view = x[:3, :49152]
    C.argmax(view, torch.empty(3 * 256, device=dev), torch.empty(3 * 256, dtype=torch.int32, device=dev), out, ids)
    assert out[:3].tolist() == [int(ids[i]) for i in view.float().argmax(-1)]


@pytest.mark.parametrize("n", [1, 7, 127, 1000, 4097, 32768, 248320])
def test_argmax_torch_semantics(C, n):
    x = torch.randn(n, device=dev).to(BF)
    assert _argmax(C, x) == int(x.float().argmax())
    x[:] = 1.0
    assert _argmax(C, x) == 0
    if n > 3:
        x = torch.randn(n, device=dev).to(BF)
        x[n // 2] = 50.0
        x[n - 1] = 50.0
        assert _argmax(C, x) == n // 2
        x[n - 2] = float("nan")
        assert _argmax(C, x) == n - 2
        x = torch.full((n,), float("-inf"), device=dev).to(BF)
        assert _argmax(C, x) == 0
    # misaligned start (odd offset into a larger buffer)
    big = torch.randn(n + 3, device=dev).to(BF)
    assert _argmax(C, big[1:1 + n]) == int(big[1:1 + n].float().argmax())


# ---------------------------------------------------------------------------- bookkeeping, bit-exact
def _gpu_i32(v):
    return torch.tensor(v, dtype=torch.int32, device=dev)


def test_accept_commit_select_match_oracle_bit_for_bit(C):
    rng = random.Random(3)
    for trial in range(300):
        n = rng.randint(1, 8)
        k = n - 1
        max_len = rng.choice([40, 64])
        pos = rng.randint(0, max_len - 1)
        mode = rng.randint(0, 1)
        am = [rng.randint(0, 5) for _ in range(8)]
        in_tok = [rng.randint(0, 5) for _ in range(9)]
        if mode == 1:
            good = rng.randint(0, k)  # make a matching prefix of random length likely
            for i in range(good):
                in_tok[i + 1] = am[i]
        else:
            in_tok[n] = rng.choice([-1, 3])
        ctl = [pos, rng.randint(0, 8), mode, 0, rng.randint(0, 9), rng.randint(0, 9)] + [0] * 10 + \
              [rng.randint(0, 4) for _ in range(16)]
        drafts = [rng.randint(0, 99) for _ in range(8)]
        # oracle
        o_ctl, o_in, o_next, o_log = list(ctl), list(in_tok), [0] * 8, [0] * max_len
        OS.accept(o_in, am, n, o_ctl, o_next, o_log)
        o_mpos = [OS.mtp_position(o_ctl, off) for off in (-1, 0, 2)]
        OS.commit(o_ctl, o_in, am, drafts, k)
        # device
        g_ctl, g_in, g_am = _gpu_i32(ctl), _gpu_i32(in_tok), _gpu_i32(am)
        g_next, g_log, g_dr = _gpu_i32([0] * 8), _gpu_i32([0] * max_len), _gpu_i32(drafts)
        C.accept(g_in, g_am, n, g_ctl, g_next, g_log)
        mp, g_mpos = _gpu_i32([0]), []
        for off in (-1, 0, 2):
            C.mtp_select(g_ctl, mp, off)
            g_mpos.append(int(mp))
        C.commit(g_ctl, g_in, g_am, g_dr, k)
        assert g_ctl.tolist() == o_ctl, trial
        assert g_in.tolist() == o_in and g_log.tolist() == o_log and g_mpos == o_mpos, trial
        assert g_next.tolist()[:n] == o_next[:n], trial


def test_mtp_select_copies_row_m(C):
    ctl = _gpu_i32([17, 0, 1, 2] + [0] * 28)
    src = torch.randn(5, 5120 + 16, device=dev).to(BF)[:, :5120]
    dst = torch.zeros(5120, dtype=BF, device=dev)
    mtp_am, d0, mp = _gpu_i32([4, 5, 6, 7, 8]), _gpu_i32([0]), _gpu_i32([0])
    C.mtp_select(ctl, mp, 0, src, dst, mtp_am, d0)
    assert torch.equal(dst, src[2]) and int(d0) == 6 and int(mp) == 17 + 2 + 1


def test_force_drafts_hook(C):
    truth = _gpu_i32(list(range(100, 200)))
    ctl = _gpu_i32([10, 0, 1, 0] + [0] * 28)
    in_tok = _gpu_i32([1] * 9)
    C.force_drafts(in_tok, ctl, truth, 2, 4, 4096)
    assert in_tok.tolist()[:5] == [1, 111, 112, 114, 115]
    ctl[2] = 0  # prefill mode: untouched
    in_tok.fill_(1)
    C.force_drafts(in_tok, ctl, truth, 2, 4, 4096)
    assert in_tok.tolist() == [1] * 9
