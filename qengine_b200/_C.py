"""Python op surface `_C`: same names, argument order, defaults and error behaviour as the
reference module `qengine._C` (csrc/bindings.cpp:189-212), bound to the C ABI of
libqengine_b200.so through ctypes.

Every op writes into caller-provided tensors, launches on the current CUDA stream, never
allocates and never synchronises, so it can be captured in a CUDA graph
(csrc/bindings.cpp:1-4). Row-batched ops take 2-D views [n, width] with unit inner stride and
any row stride; a 1-D tensor counts as one row. Validation failures raise RuntimeError, as
TORCH_CHECK does in the reference. Head sizes are taken from tensor shapes (the reference fixes
DeltaNet d = 128 and attention head_dim = 256; here d in {64, 128}, head_dim in {64, 128, 256}).
"""
from __future__ import annotations

import torch

from ._lib import check, lib

BF, I32, F32 = torch.bfloat16, torch.int32, torch.float32


def _req(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(t, dt, name):
    _req(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be a CUDA tensor")
    _req(t.dtype == dt, f"{name} has wrong dtype {t.dtype}")
    _req(t.is_contiguous(), f"{name} must be contiguous")


def _rows(t, dt, name):
    """(rows, width, row stride) of a row view (csrc/bindings.cpp:21-27)."""
    _req(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dt, f"{name}: wrong device/dtype")
    if t.dim() == 1:
        _req(t.stride(0) == 1, f"{name} not contiguous")
        return 1, t.size(0), t.size(0)
    _req(t.dim() == 2 and t.stride(1) == 1, f"{name} must be [n, w] with unit inner stride")
    return t.size(0), t.size(1), t.stride(0)


def _chk16(t, ld, name):
    _req(t.data_ptr() % 16 == 0 and ld % 8 == 0, f"{name} must be 16-byte aligned rows")


def embed(table, tok, out):
    """out[r] = table[tok[r]] for r < rows(out); out-of-range ids give zero rows."""
    _chk(table, BF, "table")
    _req(tok.is_cuda and tok.dtype == I32, "tok must be int32 CUDA")
    n, w, ld = _rows(out, BF, "out")
    _req(w == table.size(1) and tok.numel() >= n, "embed: shape mismatch")
    check(lib.qe_embed(table.data_ptr(), tok.data_ptr(), out.data_ptr(), n, w, table.size(0), ld,
                       _stream()), "embed")


def rmsnorm1p(x, delta, w, out, eps):
    """x: [rows, H]; delta optional (fused residual add, x updated in place)."""
    _chk(w, BF, "w")
    xn, xw, xld = _rows(x, BF, "x")
    on, ow, old = _rows(out, BF, "out")
    _req(xw == w.numel() and ow == xw and on == xn, "rmsnorm1p: shape mismatch")
    dptr, ldd = None, 0
    if delta is not None:
        dn, dw, ldd = _rows(delta, BF, "delta")
        _req(dn == xn and dw == xw, "rmsnorm1p: delta shape mismatch")
        dptr = delta.data_ptr()
    check(lib.qe_rmsnorm1p(x.data_ptr(), dptr, w.data_ptr(), out.data_ptr(), xn, xw, xld, ldd, old,
                           float(eps), _stream()), "rmsnorm1p")


def gemv_bf16(W, x, out):
    """out[n, N] = x[n, K] @ W[N, K]^T, n = 1..8."""
    _chk(W, BF, "W")
    xn, xw, xld = _rows(x, BF, "x")
    on, ow, old = _rows(out, BF, "out")
    _req(W.dim() == 2 and xw == W.size(1) and ow == W.size(0) and xn == on, "gemv_bf16: shape mismatch")
    _req(1 <= xn <= 8, "1..8 rows")
    _req(W.size(1) % 8 == 0, "K must be a multiple of 8")
    _chk16(W, W.size(1), "W")
    _chk16(x, xld, "x")
    check(lib.qe_gemv_bf16(W.data_ptr(), x.data_ptr(), out.data_ptr(), xn, W.size(0), W.size(1), xld,
                           old, _stream()), "gemv_bf16")


def swiglu(gu, out):
    gn, gw, gld = _rows(gu, BF, "gu")
    on, ow, old = _rows(out, BF, "out")
    _req(gw == 2 * ow and gn == on, "swiglu: shape mismatch")
    check(lib.qe_swiglu(gu.data_ptr(), out.data_ptr(), on, ow, gld, old, _stream()), "swiglu")


def argmax(x, ws_v, ws_i, out, idmap=None):
    """out[r] = argmax(x[r]); ws_v/ws_i: workspaces with rows*nb entries, nb = ws numel // rows."""
    xn, xw, xld = _rows(x, BF, "x")
    _chk(ws_v, F32, "ws_v"); _chk(ws_i, I32, "ws_i"); _chk(out, I32, "out")
    nb = ws_v.numel() // xn
    _req(ws_v.numel() == ws_i.numel() and nb >= 1 and out.numel() >= xn, "argmax: workspace/out too small")
    mp = None
    if idmap is not None:
        _chk(idmap, I32, "idmap")
        _req(idmap.numel() == xw, "idmap size")
        mp = idmap.data_ptr()
    check(lib.qe_argmax(x.data_ptr(), xn, xw, xld, ws_v.data_ptr(), ws_i.data_ptr(), nb,
                        out.data_ptr(), mp, _stream()), "argmax", kernels=2)


def rmsnorm1p_parts(x, parts, w, out, eps):
    """Tensor-parallel residual + norm (not in the reference): parts fp32 [nparts, rows, H] are the
    all-gathered partial sums of a K-split GEMV; x += bf16(sum of parts, ascending), out = norm(x)."""
    _chk(w, BF, "w"); _chk(parts, F32, "parts")
    xn, xw, xld = _rows(x, BF, "x")
    on, ow, old = _rows(out, BF, "out")
    _req(parts.dim() == 3 and parts.size(1) == xn and parts.size(2) == xw, "parts must be [nparts, rows, H]")
    _req(xw == w.numel() and ow == xw and on == xn, "rmsnorm1p_parts: shape mismatch")
    check(lib.qe_rmsnorm1p_parts(x.data_ptr(), parts.data_ptr(), parts.size(0), w.data_ptr(), out.data_ptr(),
                                 xn, xw, xld, old, float(eps), _stream()), "rmsnorm1p_parts")


def argmax_v(x, ws_v, ws_i, out, out_v, base=0, idmap=None):
    """argmax that also stores the winning value and adds `base` to the index (vocabulary shard)."""
    xn, xw, xld = _rows(x, BF, "x")
    _chk(ws_v, F32, "ws_v"); _chk(ws_i, I32, "ws_i"); _chk(out, I32, "out"); _chk(out_v, F32, "out_v")
    nb = ws_v.numel() // xn
    _req(ws_v.numel() == ws_i.numel() and nb >= 1 and out.numel() >= xn and out_v.numel() >= xn, "argmax_v sizes")
    check(lib.qe_argmax_v(x.data_ptr(), xn, xw, xld, ws_v.data_ptr(), ws_i.data_ptr(), nb, out.data_ptr(),
                          out_v.data_ptr(), idmap.data_ptr() if idmap is not None else None, int(base),
                          _stream()), "argmax_v", kernels=2)


def argmax_merge(vals, idx, out):
    """Best of nparts candidates per row: vals fp32 / idx int32 [nparts, rows] -> out int32 [rows]."""
    _chk(vals, F32, "vals"); _chk(idx, I32, "idx"); _chk(out, I32, "out")
    _req(vals.dim() == 2 and vals.shape == idx.shape and out.numel() >= vals.size(1), "argmax_merge sizes")
    check(lib.qe_argmax_merge(vals.data_ptr(), idx.data_ptr(), vals.size(0), vals.size(1), out.data_ptr(),
                              _stream()), "argmax_merge")


def attn_error():
    """Sticky error word of the attention kernel's bounded ring waits (0 = none); synchronises."""
    return int(lib.qe_attn_error())


def accept(in_tok, am, n, ctl, next_tok, log):
    for t in (in_tok, am, ctl, next_tok, log):
        _chk(t, I32, "int buffer")
    n = int(n)
    _req(in_tok.numel() > n and am.numel() >= n and next_tok.numel() >= n and ctl.numel() >= 24,
         "accept: buffers too small")
    check(lib.qe_accept(in_tok.data_ptr(), am.data_ptr(), n, ctl.data_ptr(), next_tok.data_ptr(),
                        log.data_ptr(), log.numel(), _stream()), "accept")


def commit(ctl, in_tok, am, drafts, k):
    for t in (ctl, in_tok, am, drafts):
        _chk(t, I32, "int buffer")
    k = int(k)
    _req(in_tok.numel() > k and drafts.numel() >= k, "commit: buffers too small")
    check(lib.qe_commit(ctl.data_ptr(), in_tok.data_ptr(), am.data_ptr(), drafts.data_ptr(), k,
                        _stream()), "commit")


def accept_commit(in_tok, am, n, ctl, next_tok, log, drafts, k):
    """`accept` then `commit` in one launch (passes without draft rows; not in the reference)."""
    for t in (in_tok, am, ctl, next_tok, log, drafts):
        _chk(t, I32, "int buffer")
    n, k = int(n), int(k)
    _req(in_tok.numel() > max(n, k) and am.numel() >= n and next_tok.numel() >= n and ctl.numel() >= 24 and
         drafts.numel() >= k, "accept_commit: buffers too small")
    check(lib.qe_accept_commit(in_tok.data_ptr(), am.data_ptr(), n, ctl.data_ptr(), next_tok.data_ptr(),
                               log.data_ptr(), log.numel(), drafts.data_ptr(), k, _stream()), "accept_commit")


def chain_draft(mtp_am, draft_out, src, dst):
    """draft_out[0] = mtp_am[0]; dst = src (one hidden row): the hand-over between two chained
    single-row draft passes (not in the reference, which uses two tensor copies)."""
    _chk(mtp_am, I32, "mtp_am"); _chk(draft_out, I32, "draft_out")
    _req(src.dtype == BF and dst.dtype == BF and src.is_cuda and dst.is_cuda and src.is_contiguous() and
         dst.is_contiguous() and src.numel() == dst.numel() and draft_out.numel() >= 1, "chain_draft: row shapes")
    check(lib.qe_chain_draft(mtp_am.data_ptr(), draft_out.data_ptr(), src.data_ptr(), dst.data_ptr(),
                             src.numel(), _stream()), "chain_draft")


def mtp_select(ctl, mpos, off, src=None, dst=None, mtp_am=None, draft0=None):
    """mpos = off < 0 ? pos : pos + m + 1 + off; optional: dst = src[m], draft0 = mtp_am[m]."""
    _chk(ctl, I32, "ctl"); _chk(mpos, I32, "mpos")
    sp = dp = None
    lds = H = 0
    if src is not None:
        _, H, lds = _rows(src, BF, "src")
        _chk(dst, BF, "dst")
        _req(dst.numel() == H, "dst size")
        sp, dp = src.data_ptr(), dst.data_ptr()
    check(lib.qe_mtp_select(ctl.data_ptr(), mpos.data_ptr(), int(off), sp, lds, dp, H,
                            mtp_am.data_ptr() if mtp_am is not None else None,
                            draft0.data_ptr() if draft0 is not None else None, _stream()), "mtp_select")


def force_drafts(in_tok, ctl, truth, a, k, vocab):
    """Measurement hook (not in the reference): make exactly `a` of the k drafts acceptable."""
    for t in (in_tok, ctl, truth):
        _chk(t, I32, "int buffer")
    _req(in_tok.numel() > int(k), "force_drafts: in_tok too small")
    check(lib.qe_force_drafts(in_tok.data_ptr(), ctl.data_ptr(), truth.data_ptr(), truth.numel(), int(a),
                              int(k), int(vocab), _stream()), "force_drafts")


def gdn_step_n(qkv, z, b, a, ring, conv_w, A_log, dt_bias, norm_w, S, st_k, st_v, st_g, ctl, out,
               Hk, eps, q=2):
    """Gated DeltaNet n-row step with lazy rollback; qkv/z/b/a are row views of one projection
    buffer. `q` is accepted for compatibility and ignored."""
    qn, qw, qld = _rows(qkv, BF, "qkv")
    zn, zw, zld = _rows(z, BF, "z")
    bn, bw, bld = _rows(b, BF, "b")
    an, aw, ald = _rows(a, BF, "a")
    on, ow, old = _rows(out, BF, "out")
    _req(qld == zld == bld == ald, "qkv/z/b/a must share a row stride")
    for t, nm in ((ring, "ring"), (conv_w, "conv_w"), (A_log, "A_log"), (dt_bias, "dt_bias"), (norm_w, "norm_w")):
        _chk(t, BF, nm)
    for t, nm in ((S, "S"), (st_k, "st_k"), (st_v, "st_v"), (st_g, "st_g")):
        _chk(t, F32, nm)
    _chk(ctl, I32, "ctl")
    n, Hv, Hk = qn, S.size(0), int(Hk)
    _req(1 <= n <= 8 and zn == n and bn == n and an == n and on == n, "1..8 rows, equal row counts")
    _req(S.dim() == 3 and S.size(1) == S.size(2) and S.size(1) in (64, 128), "dk = dv in {64, 128}")
    D = S.size(1)
    _req(Hk >= 1 and Hv % Hk == 0, "Hv must be a multiple of Hk")
    Cc = 2 * Hk * D + Hv * D
    _req(qw == Cc and ring.numel() == 16 * Cc and conv_w.numel() == 4 * Cc, "conv channel count")
    _req(zw == Hv * D and ow == Hv * D and bw == Hv and aw == Hv, "z/out/b/a widths")
    _req(A_log.numel() == Hv and dt_bias.numel() == Hv and norm_w.numel() == D, "per-head parameter sizes")
    _req(st_k.numel() == 8 * Hv * D and st_v.numel() == 8 * Hv * D and st_g.numel() == 8 * Hv * 2,
         "staging buffers must hold 8 rows")
    _req(ctl.numel() >= 2, "ctl too small")
    check(lib.qe_gdn_step_n(qkv.data_ptr(), z.data_ptr(), b.data_ptr(), a.data_ptr(), qld,
                            ring.data_ptr(), conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
                            norm_w.data_ptr(), S.data_ptr(), st_k.data_ptr(), st_v.data_ptr(),
                            st_g.data_ptr(), ctl.data_ptr(), out.data_ptr(), old, n, Hk, Hv, D,
                            float(eps), int(q), _stream()), "gdn_step_n")


def attn_prep(qg, k, v, qnw, knw, inv_freq, pos, q_out, kc, vc, eps):
    """pos: int32 tensor whose element 0 is the position of row 0."""
    gn, gw, gld = _rows(qg, BF, "qg")
    kn, kw, kld = _rows(k, BF, "k")
    vn, vw, vld = _rows(v, BF, "v")
    on, ow, old = _rows(q_out, BF, "q_out")
    _req(gld == kld == vld, "qg/k/v must share a row stride")
    for t, nm in ((qnw, "qnw"), (knw, "knw"), (kc, "kc"), (vc, "vc")):
        _chk(t, BF, nm)
    _chk(inv_freq, F32, "inv_freq")
    _req(pos.is_cuda and pos.dtype == I32, "pos must be int32 CUDA")
    _req(kc.dim() == 3 and kc.size(2) in (64, 128, 256), "head_dim in {64, 128, 256}")
    hd = kc.size(2)
    n, Hkv, max_len, Hq = gn, kc.size(0), kc.size(1), ow // hd
    _req(1 <= n <= 8 and kn == n and vn == n and on == n and old == ow, "row counts / contiguous q_out")
    _req(gw == Hq * 2 * hd and kw == Hkv * hd and vw == Hkv * hd, "projection widths")
    _req(vc.shape == kc.shape and qnw.numel() == hd and knw.numel() == hd, "cache / norm shapes")
    rd = inv_freq.numel() * 2
    _req(rd <= hd, "rotary dim")
    check(lib.qe_attn_prep(qg.data_ptr(), k.data_ptr(), v.data_ptr(), gld, qnw.data_ptr(),
                           knw.data_ptr(), inv_freq.data_ptr(), pos.data_ptr(), q_out.data_ptr(),
                           kc.data_ptr(), vc.data_ptr(), n, Hq, Hkv, hd, max_len, rd, float(eps),
                           _stream()), "attn_prep")


def attn_decode(q, kc, vc, pos, qg, part_o, part_ml, out):
    """q: [n, Hq*hd] contiguous; part_o: fp32 [>=n, Hq, NS, hd]; part_ml [>=n, Hq, NS, 2];
    out: [n, Hq*hd] (gated by sigmoid of the gate half of the qg rows)."""
    qn, qw, qld = _rows(q, BF, "q")
    gn, gw, gld = _rows(qg, BF, "qg")
    on, ow, old = _rows(out, BF, "out")
    _chk(kc, BF, "kc"); _chk(vc, BF, "vc"); _chk(part_o, F32, "part_o"); _chk(part_ml, F32, "part_ml")
    _req(pos.is_cuda and pos.dtype == I32, "pos must be int32 CUDA")
    _req(kc.dim() == 3 and kc.size(2) in (64, 128, 256), "head_dim in {64, 128, 256}")
    hd = kc.size(2)
    _chk16(q, qld, "q"); _chk16(kc, hd, "kc"); _chk16(vc, hd, "vc")
    n, Hq, Hkv, max_len = qn, qw // hd, kc.size(0), kc.size(1)
    _req(qld == qw and gn == n and on == n and Hq % Hkv == 0, "row counts / contiguous q")
    _req(part_o.dim() == 4 and part_o.size(0) >= n and part_o.size(1) == Hq and part_o.size(3) == hd,
         "part_o shape")
    NS = part_o.size(2)
    _req(part_ml.numel() == part_o.size(0) * Hq * NS * 2 and ow == Hq * hd and gw == Hq * 2 * hd,
         "part_ml / out / qg shapes")
    check(lib.qe_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), qg.data_ptr(),
                             gld, part_o.data_ptr(), part_ml.data_ptr(), out.data_ptr(), old, n, Hq,
                             Hkv, hd, max_len, NS, float(hd) ** -0.5, _stream()), "attn_decode", kernels=2)


def l2_persist_limit(nbytes):
    check(lib.qe_l2_persist_limit(int(nbytes)), "l2_persist_limit")


def stream_window(base, nbytes, hit):
    """Access-policy window on the current stream (bytes = 0 clears)."""
    check(lib.qe_stream_access_window(int(base), int(nbytes), float(hit), _stream()), "stream_window")


def set_gdn_phases(on):
    lib.qe_set_gdn_phases(int(bool(on)))


def set_gdn_early(on):
    lib.qe_set_gdn_early(int(bool(on)))


def set_pdl_launch(on):
    lib.qe_set_pdl_launch(int(bool(on)))


def set_pdl_trigger(on):
    lib.qe_set_pdl_trigger(int(bool(on)))
