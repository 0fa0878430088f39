"""Gated DeltaNet step and gated GQA attention through the C ABI (`_C`) against the CPU oracle.

Chains of bf16 roundings (conv -> silu, o -> norm -> weight -> gate) can each flip by one ulp when
fp32 sums are reordered, so outputs are compared to 2^-6 relative (2 ulp) plus a small absolute
term, and the fraction of elements off by more than 1 ulp is bounded (the reference's own
tolerances, tests/test_kernels.py:1-13 of the reference). Rollback and row independence are
checked bit for bit.
"""
from __future__ import annotations

import pytest
import torch

from oracle import model as OM
from util import bf16_ulp_close

pytestmark = pytest.mark.gpu
dev = "cuda"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def C():
    from qengine_b200 import _C
    return _C


# ------------------------------------------------------------------------------------ DeltaNet
def gdn_cfg(hk, hv, d):
    return OM.Config(hidden=0, layers=1, inter=0, vocab=0, eps=1e-6, layer_types=["linear_attention"], hq=1,
                     hkv=1, head_dim=256, rope_theta=1e7, rotary_dim=64, hk=hk, hv=hv, dk=d, dv=d)


def gdn_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"conv_w": (torch.randn(cfg.conv_dim, 1, 4, generator=g) * 0.5).to(BF),
            "A_log": (torch.rand(cfg.hv, generator=g) * 5.7 - 3).to(BF),
            "dt_bias": torch.randn(cfg.hv, generator=g).to(BF),
            "norm_w": (1 + 0.2 * torch.randn(cfg.dv, generator=g)).to(BF)}


def gdn_rows(cfg, n, g):
    Cd, hv = cfg.conv_dim, cfg.hv
    w = Cd + cfg.value_dim + 2 * hv
    buf = torch.empty(n, w + 24, dtype=BF)
    buf[:, :Cd] = (torch.randn(n, Cd, generator=g) * 2).to(BF)
    buf[:, Cd:Cd + cfg.value_dim] = torch.randn(n, cfg.value_dim, generator=g).to(BF)
    buf[:, Cd + cfg.value_dim:Cd + cfg.value_dim + hv] = (torch.randn(n, hv, generator=g) * 2).to(BF)
    buf[:, Cd + cfg.value_dim + hv:w] = (torch.randn(n, hv, generator=g) * 3).to(BF)
    buf[:, w:] = 0
    return buf


class GdnLayer:
    """One DeltaNet layer driven through _C.gdn_step_n with its own (pos, pending)."""

    def __init__(self, C, cfg, W):
        self.C, self.cfg = C, cfg
        self.W = {k: v.to(dev) for k, v in W.items()}
        hv, d = cfg.hv, cfg.dk
        self.ring = torch.zeros(16, cfg.conv_dim, dtype=BF, device=dev)
        self.S = torch.zeros(hv, d, d, device=dev)
        self.st = [torch.zeros(8, hv, d, device=dev), torch.zeros(8, hv, d, device=dev),
                   torch.zeros(8, hv, 2, device=dev)]
        self.ctl = torch.zeros(8, dtype=torch.int32, device=dev)

    def run(self, rows_wide, keep):
        cfg = self.cfg
        rows = rows_wide.to(dev)[:, :cfg.conv_dim + cfg.value_dim + 2 * cfg.hv]  # strided view
        n = rows.shape[0]
        c0, c1 = cfg.conv_dim, cfg.conv_dim + cfg.value_dim
        out = torch.empty(n, cfg.value_dim, dtype=BF, device=dev)
        self.C.gdn_step_n(rows[:, :c0], rows[:, c0:c1], rows[:, c1:c1 + cfg.hv], rows[:, c1 + cfg.hv:],
                          self.ring, self.W["conv_w"], self.W["A_log"], self.W["dt_bias"], self.W["norm_w"],
                          self.S, *self.st, self.ctl, out, cfg.hk, 1e-6, q=4)
        self.ctl[0] += keep
        self.ctl[1] = keep
        return out


def oracle_rows(cfg, W, rows_wide, conv, S):
    out = []
    for r in rows_wide:
        qkv, z, b, a = OM.split_gdn_proj(r, cfg)
        out.append(OM.deltanet_core(qkv, z, b, a, W, conv, S, cfg))
    return torch.stack(out)


@pytest.mark.parametrize("hk,hv,d", [(16, 16, 128), (16, 48, 128), (2, 2, 128), (1, 3, 128), (4, 8, 64), (2, 2, 64)])
def test_gdn_speculative_pattern_vs_oracle(C, hk, hv, d):
    """Passes of n rows, keep some: every row (kept or not) against the oracle run from the
    committed state, and the committed state itself."""
    cfg, W = gdn_cfg(hk, hv, d), gdn_weights(gdn_cfg(hk, hv, d))
    layer = GdnLayer(C, cfg, W)
    conv_ref = torch.zeros(cfg.conv_dim, 3, dtype=BF)
    S_ref = torch.zeros(hv, d, d)
    g = torch.Generator().manual_seed(1)
    for it, n in enumerate([1, 4, 8, 3, 1, 1, 5, 8, 2, 4]):
        rows = gdn_rows(cfg, n, g)
        if it == 4:
            rows[0, cfg.conv_dim + cfg.value_dim + hv] = 30.0  # softplus threshold branch
        keep = int(torch.randint(1, n + 1, (1,), generator=g))
        S_before = S_ref.clone()
        out = layer.run(rows, keep).cpu()
        torch.testing.assert_close(layer.S.cpu(), S_before, rtol=1e-3, atol=1e-4)
        ref = oracle_rows(cfg, W, rows, conv_ref.clone(), S_ref.clone()).float()
        diff = (out.float() - ref).abs()
        assert (diff <= 2.0 ** -6 * ref.abs() + 1e-3).all(), (it, diff.max().item())
        assert (diff > 2.0 ** -7 * ref.abs() + 1e-6).float().mean().item() < 0.01
        oracle_rows(cfg, W, rows[:keep], conv_ref, S_ref)  # advance the committed oracle state


@pytest.mark.parametrize("hk,hv,d", [(16, 48, 128), (2, 2, 128), (4, 8, 64)])
def test_gdn_rollback_bit_exact(C, hk, hv, d):
    """Kept rows of n-row passes (rejected rows thrown away) == plain 1-row decoding of the same
    tokens, bit for bit, outputs and committed state."""
    cfg, W = gdn_cfg(hk, hv, d), gdn_weights(gdn_cfg(hk, hv, d), seed=3)
    spec, plain = GdnLayer(C, cfg, W), GdnLayer(C, cfg, W)
    g = torch.Generator().manual_seed(7)
    for it, n in enumerate([8, 1, 3, 8, 8, 2, 5, 1, 7, 4, 8]):
        rows = gdn_rows(cfg, n, g)
        keep = int(torch.randint(1, n + 1, (1,), generator=g))
        out = spec.run(rows, keep)
        for t in range(keep):
            o1 = plain.run(rows[t:t + 1], 1)
            assert torch.equal(out[t], o1[0]), (it, t)
    last = gdn_rows(cfg, 1, g)
    assert torch.equal(spec.run(last, 1), plain.run(last, 1))
    # (the conv rings may differ in slots of rejected positions: those are rewritten before use)
    assert torch.equal(spec.S, plain.S)


def test_gdn_nan_stays_in_its_head(C):
    cfg, W = gdn_cfg(2, 2, 128), gdn_weights(gdn_cfg(2, 2, 128))
    layer = GdnLayer(C, cfg, W)
    rows = gdn_rows(cfg, 1, torch.Generator().manual_seed(2))
    rows[0, 2 * 256 + 128 + 5] = float("nan")  # a v channel of head 1
    out = layer.run(rows, 1)
    assert torch.isnan(out[0, 128:]).all() and not torch.isnan(out[0, :128]).any()


# ------------------------------------------------------------------------------------ attention
def attn_cfg(hq, hkv, hd, rd):
    return OM.Config(hidden=0, layers=1, inter=0, vocab=0, eps=1e-6, layer_types=["full_attention"], hq=hq,
                     hkv=hkv, head_dim=hd, rope_theta=1e7, rotary_dim=rd, hk=1, hv=1, dk=128, dv=128)


@pytest.mark.parametrize("hq,hkv,hd,rd,steps,start,n,NS", [
    (8, 2, 256, 64, 20, 0, 1, 16), (24, 4, 256, 64, 6, 0, 1, 16), (8, 2, 256, 64, 3, 4094, 1, 16),
    (1, 1, 256, 64, 5, 125, 1, 16), (8, 2, 256, 64, 24, 0, 8, 16), (24, 4, 256, 64, 12, 100, 3, 16),
    (8, 2, 64, 16, 20, 0, 5, 16), (4, 2, 128, 32, 9, 33, 3, 16),
    # long slices: the shared-memory ring of the grouped-query kernel wraps many times (groups of 6, 3)
    (12, 2, 256, 64, 4, 5000, 2, 16), (3, 1, 256, 64, 3, 2100, 3, 16), (16, 2, 128, 32, 2, 700, 1, 16),
    # a number of splits that is a multiple of 6 selects the tensor-core kernel (head dim 256)
    (24, 4, 256, 64, 6, 0, 1, 12), (8, 2, 256, 64, 24, 0, 8, 6), (12, 2, 256, 64, 4, 5000, 2, 12),
    (3, 1, 256, 64, 3, 2100, 3, 24), (1, 1, 256, 64, 5, 125, 1, 6), (16, 2, 256, 64, 3, 1000, 3, 18)])
def test_attention_vs_oracle_and_row_independence(C, hq, hkv, hd, rd, steps, start, n, NS):
    g = torch.Generator().manual_seed(1)
    cfg = attn_cfg(hq, hkv, hd, rd)
    max_len = start + steps
    L = {"q_norm": (0.3 * torch.randn(hd, generator=g)).to(BF), "k_norm": (0.3 * torch.randn(hd, generator=g)).to(BF)}
    kc_ref = torch.zeros(hkv, max_len, hd, dtype=BF)
    vc_ref = torch.zeros_like(kc_ref)
    kc_ref[:, :start] = torch.randn(hkv, start, hd, generator=g).to(BF)
    vc_ref[:, :start] = torch.randn(hkv, start, hd, generator=g).to(BF)
    kc, vc = kc_ref.to(dev), vc_ref.to(dev)
    inv = OM.inv_freq(cfg).to(dev)
    qn, kn = L["q_norm"].to(dev), L["k_norm"].to(dev)
    pos_t = torch.zeros(1, dtype=torch.int32, device=dev)
    po = torch.empty(8, hq, NS, hd, device=dev)
    pml = torch.empty(8, hq, NS, 2, device=dev)
    qw, kw = hq * 2 * hd, hkv * hd
    for p0 in range(start, start + steps, n):
        nn = min(n, start + steps - p0)
        proj = torch.empty(nn, qw + 2 * kw + 8, dtype=BF)
        proj[:, :qw] = (torch.randn(nn, qw, generator=g) * 3).to(BF)
        proj[:, qw:qw + kw] = (torch.randn(nn, kw, generator=g) * 3).to(BF)
        proj[:, qw + kw:qw + 2 * kw] = torch.randn(nn, kw, generator=g).to(BF)
        proj[:, qw + 2 * kw:] = 0
        qrs, gates = [], []
        for t in range(nn):
            q, gate, kk, vv = OM.attention_qkv(proj[t, :qw], proj[t, qw:qw + kw], proj[t, qw + kw:qw + 2 * kw],
                                               L, p0 + t, cfg)
            kc_ref[:, p0 + t], vc_ref[:, p0 + t] = kk, vv
            qrs.append(q.reshape(-1))
            gates.append(gate)
        refs = [OM.attention_core(qrs[t].view(hq, hd), gates[t], kc_ref, vc_ref, p0 + t + 1, cfg) for t in range(nn)]
        pg = proj.to(dev)
        qg, k, v = pg[:, :qw], pg[:, qw:qw + kw], pg[:, qw + kw:qw + 2 * kw]
        pos_t.fill_(p0)
        q_out = torch.empty(nn, hq * hd, dtype=BF, device=dev)
        C.attn_prep(qg, k, v, qn, kn, inv, pos_t, q_out, kc, vc, 1e-6)
        ok, err = bf16_ulp_close(q_out.cpu(), torch.stack(qrs))
        assert ok, ("q", p0, err)
        ok, err = bf16_ulp_close(kc[:, p0:p0 + nn].cpu(), kc_ref[:, p0:p0 + nn])
        assert ok, ("k", p0, err)
        assert torch.equal(vc[:, p0:p0 + nn].cpu(), vc_ref[:, p0:p0 + nn])
        # decode on the oracle's cache and queries, so q/k rounding flips do not enter the check
        kcr, vcr = kc_ref.to(dev), vc_ref.to(dev)
        qr = torch.stack(qrs).to(dev).contiguous()
        out = torch.empty(nn, hq * hd, dtype=BF, device=dev)
        C.attn_decode(qr, kcr, vcr, pos_t, qg, po, pml, out)
        for t in range(nn):
            ref = refs[t].float()
            diff = (out[t].cpu().float() - ref).abs()
            assert (diff <= 2.0 ** -6 * ref.abs() + 2e-3).all(), (p0 + t, diff.max().item())
            o1 = torch.empty(1, hq * hd, dtype=BF, device=dev)
            C.attn_decode(qr[t:t + 1], kcr, vcr, pos_t + t, qg[t:t + 1], po, pml, o1)
            assert torch.equal(o1[0], out[t]), "row differs from the 1-row pass"
    assert C.attn_error() == 0


def _decode_against_oracle(C, hq, hkv, NS, n, start, max_len, seed, stale=1.0):
    """attn_decode on a random cache of head dim 256 against the oracle's attention, plus the
    1-row passes of every row. Cache rows past the prefixes hold `stale`-scaled random numbers
    (rejected drafts leave such rows behind). Returns worst error / bound."""
    g = torch.Generator().manual_seed(seed)
    hd = 256
    cfg = attn_cfg(hq, hkv, hd, 64)
    kc = torch.randn(hkv, max_len, hd, generator=g).to(BF)
    vc = torch.randn(hkv, max_len, hd, generator=g).to(BF)
    kc[:, start + n:] *= stale
    vc[:, start + n:] *= stale
    q = torch.randn(n, hq, hd, generator=g).to(BF)
    gate = (torch.randn(n, hq, hd, generator=g) * 2).to(BF)
    qg = torch.cat([q, gate], dim=-1).reshape(n, hq * 2 * hd)  # per head [q | gate]
    refs = [OM.attention_core(q[t], gate[t].reshape(-1), kc, vc, min(start + t + 1, max_len), cfg) for t in range(n)]
    kcd, vcd, qd, qgd = kc.to(dev), vc.to(dev), q.reshape(n, hq * hd).to(dev).contiguous(), qg.to(dev)
    pos_t = torch.tensor([start], dtype=torch.int32, device=dev)
    po = torch.empty(8, hq, NS, hd, device=dev)
    pml = torch.empty(8, hq, NS, 2, device=dev)
    out = torch.empty(n, hq * hd, dtype=BF, device=dev)
    C.attn_decode(qd, kcd, vcd, pos_t, qgd, po, pml, out)
    worst = 0.0
    for t in range(n):
        ref = refs[t].float()
        diff = (out[t].cpu().float() - ref).abs()
        worst = max(worst, float((diff / (2.0 ** -6 * ref.abs() + 2e-3)).max()))
        o1 = torch.empty(1, hq * hd, dtype=BF, device=dev)
        C.attn_decode(qd[t:t + 1], kcd, vcd, pos_t + t, qgd[t:t + 1], po, pml, o1)
        assert torch.equal(o1[0], out[t]), f"row {t} differs from the 1-row pass"
    # and a second n-row pass gives the same bits (no state left behind in the scratch)
    out2 = torch.empty_like(out)
    C.attn_decode(qd, kcd, vcd, pos_t, qgd, po, pml, out2)
    assert torch.equal(out, out2)
    assert C.attn_error() == 0
    return worst


def test_attention_at_the_long_context_operating_point(C):
    """The split kernel as the engine runs it on a 32K-position cache of the 27B shape: 24 query /
    4 KV heads of dim 256, 5 rows (verify), 222 splits, against the oracle's attention over the
    same cache; rows bit-identical to 1-row passes."""
    worst = _decode_against_oracle(C, 24, 4, 222, 5, 32003, 32003 + 5 + 3, seed=5)
    print(f"\n32K positions, 222 splits: worst error / bound = {worst:.3f}")
    assert worst <= 1.0


@pytest.mark.parametrize("hq,hkv,NS,n,start,slack", [
    # the rows of a pass share one K/V stream cut into splits of 16 * ceil(len / (16 NS)) positions;
    # these passes have rows on both sides of a multiple of 16 NS, where that length changes:
    (24, 4, 6, 5, 93, 40),      # lengths 94..98 around 96
    (8, 2, 6, 2, 95, 1),        # the two rows of one tile on different sides (96 | 97)
    (12, 2, 12, 8, 190, 0),     # 191..198 around 192, the pass ends with the cache
    (4, 1, 6, 3, 286, 7),       # 287..289 around 288 = 3 * 96
    (24, 4, 222, 5, 3550, 16),  # the engine's 222 splits around 3552
    # every row count (1..8 rows = 1..4 warps per stream) well inside one split length
    (24, 4, 12, 1, 700, 9), (24, 4, 12, 2, 700, 9), (24, 4, 12, 3, 700, 9), (24, 4, 12, 4, 700, 9),
    (24, 4, 12, 5, 700, 9), (24, 4, 12, 6, 700, 9), (24, 4, 12, 7, 700, 9), (24, 4, 12, 8, 700, 9),
    # eight query heads per KV head: 3..8 rows need three or four tiles (four warps per stream)
    (16, 2, 12, 8, 700, 9), (16, 2, 12, 7, 96 * 2 - 3, 5), (8, 1, 6, 5, 300, 2), (16, 2, 222, 6, 9000, 11),
    # rows on both sides of 4,096 positions, where the probabilities stop being carried as two bf16
    (24, 4, 12, 5, 4093, 8), (8, 2, 24, 2, 4095, 3),
    # rows that run past the end of the cache see the whole cache
    (8, 2, 6, 4, 61, -2)])
def test_attention_rows_share_one_stream(C, hq, hkv, NS, n, start, slack):
    worst = _decode_against_oracle(C, hq, hkv, NS, n, start, start + n + slack, seed=start + n, stale=50.0)
    assert worst <= 1.0, worst


def test_attention_never_writes_past_the_cache(C):
    hq, hkv, hd = 8, 2, 256
    cfg = attn_cfg(hq, hkv, hd, 64)
    max_len = 8
    guard = torch.zeros(hkv * max_len * hd + 4096, dtype=BF, device=dev)
    kc = guard[:hkv * max_len * hd].view(hkv, max_len, hd)
    vc = torch.zeros(hkv, max_len, hd, dtype=BF, device=dev)
    proj = torch.randn(4, hq * 2 * hd + 2 * hkv * hd, device=dev).to(BF)
    qw, kw = hq * 2 * hd, hkv * hd
    pos = torch.tensor([6], dtype=torch.int32, device=dev)  # rows at 6, 7, 8, 9: two fall outside
    z = torch.zeros(hd, dtype=BF, device=dev)
    q_out = torch.empty(4, hq * hd, dtype=BF, device=dev)
    C.attn_prep(proj[:, :qw], proj[:, qw:qw + kw], proj[:, qw + kw:], z, z, OM.inv_freq(cfg).to(dev), pos, q_out,
                kc, vc, 1e-6)
    torch.cuda.synchronize()
    assert (guard[hkv * max_len * hd:] == 0).all()
    assert (kc[:, 6:8] != 0).any() and (kc[:, :6] == 0).all()
