"""Batch-1 decode engine for B200: plain greedy decoding and MTP speculative decoding, each pass
variant captured once as a CUDA graph, all bookkeeping on the device.

The public names mirror the reference engine (python/qengine/engine.py:189-687) so that its
callers can switch: `Engine` with `generate`, `generate_spec`, `prefill`, `graph`,
`sequence_logits`, `mtp_rows_logits`, `reset`, `pin_mtp_l2`, and the linear backends `W4Linear` /
`BF16Linear`. The model arrives as a weights dict in the fused layout (qengine_b200.synth or
qengine_b200.cache) rather than as a checkpoint directory.

What is different from the reference is the graph itself. The reference launches one kernel per
operator (487 per token at the 27B shape); here the residual stream is an object (`_Residual`)
that remembers which sub-layer output is still to be added, and the add + RMSNorm is executed
inside the next W4 GEMV launch (qe_w4_gemv_ex): every block of the GEMV recomputes the ten
kilobytes of normalised input in its shared memory while its weight rings are already filling.
The embedding gather rides on the first GEMV the same way, the final norm on the lm_head GEMV,
accept + commit are one kernel in plain decoding. A 27B-shape token is 4 GEMV launches per layer
plus the mixer.

A pass runs n = 1..8 rows (tokens at positions pos .. pos + n - 1):
  decode   n = 1
  verify   n = k + 1 rows [last token, draft 1 .. draft k]; the longest prefix of drafts that
           equals the model's own greedy choice is kept, plus the model's next token
  prefill  up to 8 prompt tokens per pass
One graph replay is one decode step or one whole speculative cycle (verify, MTP rows, k - 1
chained drafts, commit); the host reads the position once per batch of cycles.

Rollback costs nothing: K/V rows of rejected drafts are simply overwritten, DeltaNet rows are
staged as per-position checkpoints of which the next pass replays only the kept ones
(csrc/deltanet.cu). Every kernel computes row r of an n-row pass exactly as a 1-row pass would,
which makes speculative output token-identical to plain greedy output.
"""
from __future__ import annotations

import gc
import os
from contextlib import contextmanager

import torch

from . import _C, _w4
from ._lib import launches, lib
from .quant import W4Packed
from .synth import Config

BF16, I32, F32 = torch.bfloat16, torch.int32, torch.float32
NMAX = 8  # rows per pass


# ----------------------------------------------------------------------------------------------
# Linear backends
# ----------------------------------------------------------------------------------------------
class BF16Linear:
    """Unquantised GEMV backend (weights read once for all rows, fp32 accumulate)."""
    name = "bf16"

    def prepare(self, w):
        return w.contiguous()

    def __call__(self, x, w, out):
        _C.gemv_bf16(w, x, out)


class W4Linear:
    """Adapter over the W4A16 GEMV (`_w4`); like its namesake in the reference
    (python/qengine/engine.py:74-115) it is the only place that touches that API. Keyword
    arguments given at construction are forwarded to every launch."""
    name = "w4"
    cache_tag = "w4-rtn-g128-v1"  # names the prepared-weights directory (qengine_b200.cache)

    def __init__(self, **launch_kw):
        self.kw = dict(launch_kw)

    def prepare(self, w):
        from .quant import quantize_w4
        return quantize_w4(w)

    def prepare_from_grid(self, Wq, rows_per_step: int = 2048):
        """Pack a matrix that is already on the W4 grid (a GPTQ lm_head) without quantising it
        again; returns (packed, stats). See qengine_b200.cache.pack_from_grid."""
        from .cache import pack_from_grid
        return pack_from_grid(Wq, rows_per_step)

    def prepare_gate_up(self, wg, wu):
        from .quant import quantize_w4_gate_up
        return quantize_w4_gate_up(wg, wu)

    @staticmethod
    def dequantize(p):
        from .quant import dequantize_w4
        return dequantize_w4(p)

    def __call__(self, x, p, out, **kw):
        _w4.gemv(x, p.qw, p.scales, out, p.M, **{**self.kw, **kw})

    def gate_up(self, x, p, out):
        _w4.gemv_swiglu(x, p.qw, p.scales, out, p.M, **self.kw)

    def partial(self, x, p, out32):
        """fp32 partial sums of a matrix whose K dimension is split over tensor-parallel ranks."""
        _w4.gemv_partial(x, p.qw, p.scales, out32, p.M, **self.kw)

    def after_norm(self, h, delta, w, eps, p, out, **kw):
        """out = p(RMSNorm1p(h + delta)) in one launch (see `_w4.gemv_fused`)."""
        _w4.gemv_fused(h, delta, w, eps, p.qw, p.scales, out, p.M, swiglu=p.gate_up, **{**self.kw, **kw})

    # The same four operations as job descriptions, for `launch` below: the engine queues the
    # GEMVs that follow one another without another kernel in between and runs them as one chain.
    @staticmethod
    def job(x, p, out):
        return _w4.job(x, p.qw, p.scales, out, p.M, swiglu=p.gate_up, allow_f16_x=True)

    @staticmethod
    def job_partial(x, p, out32):
        return _w4.job(x, p.qw, p.scales, out32, p.M, allow_f32_out=True)

    @staticmethod
    def job_after_norm(h, delta, w, eps, p, out, **kw):
        return _w4.job_fused(h, delta, w, eps, p.qw, p.scales, out, p.M, swiglu=p.gate_up, **kw)

    def launch(self, jobs, **kw):
        _w4.gemv_chain(jobs, **{**self.kw, **kw})

    def norm_rows(self, h, delta, w, eps, xn_out, **kw):
        """The prologue of `after_norm` as its own launch, one block per row, same bits."""
        _w4.norm_rows(h, delta, w, eps, xn_out, **{**self.kw, **kw})


class _AfterFlush:
    """`_C` seen through the engine: any kernel other than a W4 GEMV first launches the GEMVs that
    are still queued, so the stream order is the program order."""

    def __init__(self, ops, flush):
        self._ops, self._flush = ops, flush

    def __getattr__(self, name):
        fn = getattr(self._ops, name)

        def call(*a, **kw):
            self._flush()
            return fn(*a, **kw)
        return call


# ----------------------------------------------------------------------------------------------
# The residual stream of one pass
# ----------------------------------------------------------------------------------------------
class _Residual:
    """Rows h[:n] of a residual stream plus whatever has been produced but not yet added to it.

    `owed` is the output of the last K-split matrix (attention / DeltaNet out-projection, MLP
    down-projection, MTP fc): one bf16 buffer on a single GPU, fp32 partial rows per rank under
    tensor parallelism. It is added by the next norm, which is where the three execution modes
    differ:
      fused   the add + norm run inside the next GEMV (`W4Linear.after_norm`); the updated stream
              is written to the spare buffer by one block, so the two buffers swap roles;
      plain   `_C.rmsnorm1p` with its residual argument, then the GEMV;
      tp      the ranks' partial rows are exchanged and summed inside the norm kernel
              (`TPGroup.exchange_norm`, or all-gather + `_C.rmsnorm1p_parts`).
    """

    def __init__(self, eng, n, rows, spare, xn):
        self.e, self.n = eng, n
        self.h, self.spare, self.xn = rows[:n], spare[:n], xn[:n]
        self.owed = False
        self.tok = None  # set: the rows are embedding rows that have not been gathered yet

    def start_from_tokens(self, tok, ordered):
        """Rows = embedding rows of `tok`. Returns True when the plain-stream-order launch that
        opens a pass (Engine._ordered_first_launch) is still to come."""
        e = self.e
        self.owed = False
        if e.fuse and isinstance(e.layers[0]["in_proj"], W4Packed) and isinstance(e.linear, W4Linear):
            self.tok = tok  # gathered by the prologue of the first GEMV
            return ordered
        if ordered:
            with e._ordered_first_launch():
                e.K.embed(e.embed, tok, self.h)
        else:
            e.K.embed(e.embed, tok, self.h)
        return False

    def start_from_rows(self):
        self.owed, self.tok = False, None

    def owe(self, x, p, lin):
        """A matrix split along K on the ranks: its result is added by the next norm."""
        e, n = self.e, self.n
        w4 = isinstance(lin, W4Linear) and isinstance(p, W4Packed)
        if e.tp is None:
            if w4:
                e._gemv(lin.job(x, p, e.mo[:n]))
            else:
                e._flush()
                lin(x, p, e.mo[:n])
        else:
            if w4:
                e._gemv(lin.job_partial(x, p, e.part32[:n]))
            else:
                e._flush()
                lin.partial(x, p, e.part32[:n])
            if e.tp.transport == "nccl":
                e._flush()
                e.tp.all_gather(e.parts[n], e.part32[:n])
        self.owed = True

    def zero_then_owe(self, x, p, lin):
        """Tensor parallel only: the stream starts as the sum of the ranks' partial rows."""
        self.e._flush()
        self.h.zero_()
        self.owe(x, p, lin)

    def _norm(self, w, out, out16=None):
        """out = norm(h + owed). Returns True when out16 was filled too (only the exchange kernel of
        the tensor-parallel path writes the fp16 copy)."""
        e, n = self.e, self.n
        K = e.K  # kernels other than the W4 GEMV: the queue of GEMVs is flushed first
        if not self.owed:
            K.rmsnorm1p(self.h, None, w, out, e.cfg.eps)
        elif e.tp is None:
            K.rmsnorm1p(self.h, e.mo[:n], w, out, e.cfg.eps)
        elif e.tp.transport == "nccl":
            K.rmsnorm1p_parts(self.h, e.parts[n], w, out, e.cfg.eps)
        else:
            e._flush()
            e.tp.exchange_norm(self.h, e.part32[:n], w, out, e.cfg.eps, out16=out16)
            self.owed = False
            return out16 is not None
        self.owed = False
        return False

    def through(self, w, p, out, lin, keep_normed=None, ordered=False):
        """out = p(norm(h + owed)); keep_normed optionally receives the normed rows. ordered: this
        is the launch that opens a pass (no programmatic overlap with the previous pass)."""
        e, n = self.e, self.n
        w4 = isinstance(p, W4Packed) and isinstance(lin, W4Linear)
        if e.fuse and w4 and n > e.FUSE_MAX_ROWS:
            # Several rows: every block of the GEMV would repeat the norm of all rows; one block per
            # row in front of a plain GEMV is faster, and (same arithmetic) gives the same bits.
            xn = keep_normed if keep_normed is not None else self.xn
            e._flush()
            kw = {"pdl": False} if ordered else {}
            if e.f16:  # the rows also as fp16: input of the GEMV's fp16 flavour, like the fused launch
                kw["xn16_out"] = e.xn16[:n]
            if self.tok is not None:
                lin.norm_rows(e.embed, None, w, e.cfg.eps, xn, tok=self.tok, h_out=self.h, **kw)
                self.tok = None
            else:
                lin.norm_rows(self.h, e.mo[:n] if self.owed else None, w, e.cfg.eps, xn,
                              h_out=self.h if self.owed else None, **kw)
            self.owed = False
            e._gemv(lin.job(e.xn16[:n] if e.f16 else xn, p, out))
            return
        if e.fuse and w4:
            if self.tok is not None:
                j = lin.job_after_norm(e.embed, None, w, e.cfg.eps, p, out, tok=self.tok, h_out=self.h,
                                       xn_out=keep_normed, f16=e.f16)
                self.tok = None
            elif self.owed:
                j = lin.job_after_norm(self.h, e.mo[:n], w, e.cfg.eps, p, out, h_out=self.spare, xn_out=keep_normed,
                                       f16=e.f16)
                self.h, self.spare = self.spare, self.h
            else:
                j = lin.job_after_norm(self.h, None, w, e.cfg.eps, p, out, xn_out=keep_normed, f16=e.f16)
            self.owed = False
            e._gemv(j, ordered=ordered)
            return
        xn = keep_normed if keep_normed is not None else self.xn
        as16 = self._norm(w, xn, e.xn16[:n] if (w4 and e.tp_f16) else None)
        if w4:
            e._gemv(lin.job(e.xn16[:n] if as16 else xn, p, out))
        else:
            e._flush()
            lin(xn, p, out)


# ----------------------------------------------------------------------------------------------
class Engine:
    GDN_Q = 4
    FUSE_MAX_ROWS = 1  # passes of more rows run the norm as its own launch (see _Residual.through)
    POS, PENDING, MODE, M, CYCLES, ACCEPTED = range(6)

    def __init__(self, cfg: Config, weights: dict, max_len: int = 4096, linear=None, device="cuda",
                 mtp: bool = True, attn_splits: int | None = None, draft_vocab: int | None = None, tp=None,
                 fuse: bool | None = None, chain: bool | None = None, wide_prefill: bool = False):
        """weights: dict in the fused layout (qengine_b200.synth.build_model), already on `device`.
        tp: a qengine_b200.tp.TPGroup for tensor parallelism; `cfg` then still describes the whole
        model and `weights` is this rank's shard (qengine_b200.tp.shard_model).
        attn_splits: flash-decoding splits per head (fixed, so graphs stay static); default 16, more
        for caches beyond 8192 positions. draft_vocab: drafts score only the first `draft_vocab`
        token ids (pruned draft head through the argmax id map); verify keeps the full head.
        fuse: run residual add + RMSNorm inside the following W4 GEMV launch (default: on for a
        single GPU; under tensor parallelism the norm is fused with the exchange instead).
        chain: launch runs of consecutive W4 GEMVs as one cooperative kernel with grid barriers
        (default off, QE_CHAIN=1 turns it on: measured slower than one launch per GEMV under
        programmatic dependent launch, whose hand-over costs about 1 us against 2.5 us for the
        barrier).
        wide_prefill: feed prompts in passes of up to 64 rows through the tensor-memory GEMM
        (`_w4.gemm`, every matrix read once per pass) instead of 8 rows through the GEMV; see
        `prefill`. Off by default: the reference prefills 8 rows at a time, and only that way is a
        chunked prefill bit-identical to feeding the prompt token by token."""
        self.tp, self.vocab_full, self.vocab_base = tp, cfg.vocab, 0
        if tp is not None:
            from .tp import local_config
            tp.open(cfg.hidden)
            cfg = local_config(cfg, tp.size)
            self.vocab_base = tp.rank * cfg.vocab
        self.cfg, self.max_len, self.dev = cfg, max_len, torch.device(device)
        self.linear = linear or W4Linear()
        self.fuse = (tp is None) if fuse is None else (bool(fuse) and tp is None)
        self.chain = (os.environ.get("QE_CHAIN", "0") == "1") if chain is None else bool(chain)
        self.embed, self.final_norm = weights["embed"], weights["final_norm"]
        self.lm_head = weights["lm_head"]
        self.lm_lin = self.linear if isinstance(self.lm_head, W4Packed) else BF16Linear()
        self.layers = [dict(L) for L in weights["layers"]]
        self.has_mtp = bool(mtp and weights.get("mtp"))
        self.mtp = dict(weights["mtp"]) if self.has_mtp else None
        fits = os.environ.get("QE_F16", "1") == "1" and self._norms_fit_fp16()
        self.f16 = self.fuse and fits
        # tensor parallel over own exchange kernels: the exchange + norm writes the fp16 rows
        self.tp_f16 = fits and tp is not None and tp.transport == "peer"
        # caches beyond 8K positions: a multiple of 6 selects the tensor-core split kernel, sized
        # to one CTA per SM and row
        self.ATTN_SPLITS = attn_splits or (16 if max_len <= 8192 else 6 * -(-max(1, int(lib.qe_sm_count())) // cfg.hkv))
        self.draft_head = self.draft_ids = None
        if draft_vocab and self.has_mtp:
            self._make_draft_head(draft_vocab)
        self._make_buffers()
        self.graphs, self.graph_kernels = {}, {}
        self._q, self._q_ordered = [], False  # W4 GEMVs waiting to be launched as one chain
        self.K = _AfterFlush(_C, self._flush)
        self.start_pos = 0      # positions [0, start_pos) hold a pre-filled context (set_context)
        self.force_a = -1       # forced acceptance length of verify passes (< 0: off)
        self.truth = torch.zeros(1, dtype=I32, device=self.dev)
        self.l2_win = None      # (base, bytes) of the persisting window around the draft phase
        self.wide_prefill = bool(wide_prefill)
        self.wb = None          # buffers of the wide prefill passes (allocated on first use)

    @classmethod
    def from_cache(cls, path, cache_dir, device="cuda", linear=None, **kw):
        """Engine over a checkpoint directory whose prepared weights were cached (by this package
        or by the reference, python/qengine/engine.py:215-236): `path` supplies config.json, the
        weights come from `<cache_dir>/<path name>-<linear.cache_tag>/`."""
        from pathlib import Path
        from . import cache
        linear = linear or W4Linear()
        cfg = cache.config_from_dir(path)
        d = cache.cache_path(cache_dir, Path(path).name, linear.cache_tag)
        weights = cache.load_cache(d, cfg, device=device, mtp=kw.get("mtp", True))
        return cls(cfg, weights, linear=linear, device=device, **kw)

    def _norms_fit_fp16(self) -> bool:
        """GEMVs behind an RMSNorm can take their input as fp16 (cheaper unpack, same bits, see
        qe_w4_params::x_f16) when every normalised value fits: |x_i| <= sqrt(H) * |1 + w_i|."""
        ws = [self.final_norm] + [L[k] for L in self.layers for k in ("in_norm", "post_norm")]
        if self.mtp:
            ws += [self.mtp[k] for k in ("in_norm", "post_norm", "norm")]
        top = max(float((1.0 + w.float()).abs().max()) for w in ws)
        return top * float(self.cfg.hidden) ** 0.5 < 60000.0

    # -- construction -------------------------------------------------------------------------
    def _make_draft_head(self, nv: int):
        """The first nv rows of the packed lm_head serve as the draft head (ids 0 .. nv - 1): tiles
        of 16 rows are independent in the packed format, so this is a slice, not a requantisation.
        Under tensor parallelism every rank keeps the first nv / t rows of its vocabulary slice."""
        if self.tp is not None:
            nv //= self.tp.size
        if nv % 16 or not isinstance(self.lm_head, W4Packed):
            raise ValueError("draft_vocab must be a multiple of 16 (per rank) on a W4 lm_head")
        p = self.lm_head
        self.draft_head = W4Packed(p.qw[:nv // 16].contiguous(), p.scales[:nv // 16].contiguous(), nv, p.K)
        self.draft_ids = torch.arange(nv, dtype=I32, device=self.dev)

    def _make_buffers(self):
        c, dev, N = self.cfg, self.dev, NMAX
        H = c.hidden

        def buf(*shape, dt=BF16):
            return torch.zeros(*shape, dtype=dt, device=dev)

        # control words: ctl[0] pos, [1] pending DeltaNet rows, [2] mode, [3] m, [4] cycles,
        # [5] accepted drafts, [16 + m] histogram (include/qengine_b200.h)
        self.ctl, self.in_tok, self.mpos = buf(32, dt=I32), buf(N + 1, dt=I32), buf(1, dt=I32)
        self.am, self.next_tok, self.drafts, self.mtp_am = (buf(N, dt=I32) for _ in range(4))
        self.log = buf(self.max_len, dt=I32)
        # activations of a pass; the residual stream has two homes (see _Residual)
        self.h, self.h2, self.xn, self.mo, self.hid = (buf(N, H) for _ in range(5))
        self.xn16 = buf(N, H, dt=torch.float16)  # normalised rows as fp16 (passes of several rows)
        width = max(c.gdn_proj_rows, c.attn_proj_rows)
        self.proj = buf(N, -(-width // 8) * 8)
        self.mix = buf(N, max(c.value_dim, c.hq * c.head_dim))
        self.act = buf(N, c.inter)
        self.gu = None  # [N, 2 I], only for an unfused gate/up pair (allocated on first use)
        self.logits = buf(N, c.vocab)
        self.am_v, self.am_i = buf(N * 256, dt=F32), buf(N * 256, dt=I32)
        self.q = buf(N, c.hq * c.head_dim)
        self.part_o = buf(N, c.hq, self.ATTN_SPLITS, c.head_dim, dt=F32)
        self.part_ml = buf(N, c.hq, self.ATTN_SPLITS, 2, dt=F32)
        rd = c.rotary_dim  # fp32 on the CPU like the reference (python/qengine/engine.py:403-404)
        self.inv_freq = (1.0 / (c.rope_theta ** (torch.arange(0, rd, 2, dtype=F32) / rd))).to(dev)
        for L in self.layers + ([self.mtp] if self.has_mtp else []):
            if L["type"] == "linear_attention":
                L["ring"] = buf(16, c.conv_dim)
                L["S"] = buf(c.hv, c.dk, c.dv, dt=F32)
                L["st_k"], L["st_v"] = buf(N, c.hv, c.dk, dt=F32), buf(N, c.hv, c.dv, dt=F32)
                L["st_g"] = buf(N, c.hv, 2, dt=F32)
            else:
                L["kc"], L["vc"] = (buf(c.hkv, self.max_len, c.head_dim) for _ in range(2))
        if self.has_mtp:
            self.cat = buf(N, 2 * H)
            self.mh, self.mh2, self.mout, self.chain_h = buf(N, H), buf(N, H), buf(N, H), buf(1, H)
        if self.tp is not None:
            t = self.tp.size
            self.part32 = buf(N, H, dt=F32)
            self.parts = {n: buf(t, n, H, dt=F32) for n in range(1, N + 1)}
            self.cand_v, self.cand_i = buf(N, dt=F32), buf(N, dt=I32)
            self.all_v = {n: buf(t, n, dt=F32) for n in range(1, N + 1)}
            self.all_i = {n: buf(t, n, dt=I32) for n in range(1, N + 1)}

    def pin_mtp_l2(self, on: bool, names=("fc", "in_proj", "out"), limit: int | None = None):
        """Keep the named MTP matrices resident in L2 across the draft passes of a cycle (the
        reference's experiment, python/qengine/engine.py:360-381, sized for B200: fc + in_proj +
        o_proj of the 27B draft layer are 81 MB of its ~126 MB L2). The matrices are re-homed into
        one contiguous buffer so that a single access-policy window covers them; the draft phase
        of every graph captured afterwards runs under that window. Call before the first
        `generate_spec`; existing graphs are dropped."""
        if not self.has_mtp:
            return
        if on and getattr(self, "_l2_buf", None) is None:
            mats = [self.mtp[n] for n in names]
            chunks = [t for m in mats for t in (m.qw, m.scales)]
            sizes = [-(-t.numel() * t.element_size() // 256) * 256 for t in chunks]
            arena = torch.empty(sum(sizes), dtype=torch.uint8, device=self.dev)
            views, at = [], 0
            for t, sz in zip(chunks, sizes):
                v = arena[at:at + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
                v.copy_(t)
                views.append(v)
                at += sz
            for i, n in enumerate(names):
                old = self.mtp[n]
                self.mtp[n] = W4Packed(views[2 * i], views[2 * i + 1], old.M, old.K, old.gate_up)
            self._l2_buf = arena
        if on:
            nbytes = self._l2_buf.numel()
            _C.l2_persist_limit(int(limit if limit is not None else nbytes))
            self.l2_win = (self._l2_buf.data_ptr(), nbytes)
        else:
            self.l2_win = None
            _C.l2_persist_limit(0)
        self.graphs.clear()
        self.graph_kernels.clear()

    def reset(self):
        """Start an empty sequence: DeltaNet state, conv history and control words are cleared;
        K/V caches are not (rows at or beyond `pos` are never read)."""
        for L in self.layers:
            if "S" in L:
                L["ring"].zero_()
                L["S"].zero_()
        self.ctl.zero_()
        if self.start_pos:
            self.ctl[self.POS].fill_(self.start_pos)

    @torch.no_grad()
    def set_context(self, length: int, seed: int = 99):
        """Measurement harness for long caches: behave as if `length` positions had already been
        decoded. K and V rows [0, length) of every attention layer (and the draft layer) get seeded
        N(0, 1) values; sequences then start at position `length` with an empty DeltaNet state."""
        if not 0 <= length < self.max_len - 2 * NMAX:
            raise ValueError("context does not fit max_len")
        g = torch.Generator(device=self.dev).manual_seed(seed)
        for L in self.layers + ([self.mtp] if self.has_mtp else []):
            for name in ("kc", "vc"):
                if name in L:
                    for head in L[name]:
                        head[:length].copy_(torch.randn(length, head.shape[1], generator=g, device=self.dev))
        self.start_pos = int(length)
        self.reset()

    # -- the pass, as the kernels it launches ----------------------------------------------------
    def _gemv(self, job, ordered=False):
        """Queue one W4 GEMV. GEMVs that follow one another with no other kernel in between (out
        projection -> gate/up -> down -> next block's in_proj, once the norms ride in the GEMV
        prologues) are launched together as one chain: see `_w4.gemv_chain`."""
        if not self.chain:
            self.linear.launch([job], **({"pdl": False} if ordered else {}))
            return
        self._q.append(job)
        self._q_ordered = self._q_ordered or ordered
        if len(self._q) == 4:
            self._flush()

    def _flush(self):
        if self._q:
            self.linear.launch(self._q, **({"pdl": False} if self._q_ordered else {}))
            self._q, self._q_ordered = [], False

    @contextmanager
    def _ordered_first_launch(self):
        """Programmatic dependent launch lets a kernel's prologue run before its predecessor has
        finished. Across two passes that is not wanted: the first kernel of a pass is launched in
        plain stream order, so everything the previous pass wrote (position, pending rows,
        DeltaNet state and checkpoints) is complete before any early section of this pass runs."""
        _C.set_pdl_launch(False)
        try:
            yield
        finally:
            _C.set_pdl_launch(True)

    def _mixer(self, L, n, pos):
        """Token mixing on the projected rows in self.proj; result in self.mix."""
        c = self.cfg
        if L["type"] == "linear_attention":
            pr = self.proj[:n, :c.gdn_proj_rows]
            a0, a1 = c.conv_dim, c.conv_dim + c.value_dim
            out = self.mix[:n, :c.value_dim]
            self.K.gdn_step_n(pr[:, :a0], pr[:, a0:a1], pr[:, a1:a1 + c.hv], pr[:, a1 + c.hv:], L["ring"],
                          L["conv_w"], L["A_log"], L["dt_bias"], L["norm_w"], L["S"], L["st_k"], L["st_v"],
                          L["st_g"], self.ctl, out, c.hk, c.eps, q=self.GDN_Q)
            return out
        pr = self.proj[:n, :c.attn_proj_rows]
        nq = c.hq * 2 * c.head_dim
        nk = nq + c.hkv * c.head_dim
        qg, q = pr[:, :nq], self.q[:n]
        self.K.attn_prep(qg, pr[:, nq:nk], pr[:, nk:], L["q_norm"], L["k_norm"], self.inv_freq, pos, q,
                     L["kc"], L["vc"], c.eps)
        out = self.mix[:n, :c.hq * c.head_dim]
        self.K.attn_decode(q, L["kc"], L["vc"], pos, qg, self.part_o, self.part_ml, out)
        return out

    def _block(self, L, R: _Residual, pos, ordered=False):
        """One decoder block on the residual stream R: norm -> in_proj -> mixer -> out_proj, then
        norm -> gate/up + SwiGLU -> down. Both sub-layer outputs stay owed to the stream."""
        n, lin = R.n, self.linear
        width = self.cfg.gdn_proj_rows if L["type"] == "linear_attention" else self.cfg.attn_proj_rows
        R.through(L["in_norm"], L["in_proj"], self.proj[:n, :width], lin, ordered=ordered)
        mixed = self._mixer(L, n, pos)
        gu = L["gate_up"]
        R.owe(mixed, L["out"], lin)
        if isinstance(gu, W4Packed) and gu.gate_up:
            R.through(L["post_norm"], gu, self.act[:n], lin)
        else:  # unfused gate / up pair: plain GEMV into [gate | up], SwiGLU as its own kernel
            if self.gu is None:
                self.gu = torch.zeros(NMAX, 2 * self.cfg.inter, dtype=BF16, device=self.dev)
            R.through(L["post_norm"], gu, self.gu[:n], lin)
            self.K.swiglu(self.gu[:n], self.act[:n])
        R.owe(self.act[:n], L["down"], lin)

    def _greedy(self, logits, n, out, idmap=None):
        """Greedy token per row, lowest id on ties; vocabulary shards exchange (value, id)."""
        ws_v, ws_i = self.am_v[:n * 256], self.am_i[:n * 256]
        if self.tp is None:
            self.K.argmax(logits, ws_v, ws_i, out, idmap)
            return
        self.K.argmax_v(logits, ws_v, ws_i, self.cand_i, self.cand_v, self.vocab_base, idmap)
        if self.tp.transport == "nccl":
            self.tp.all_gather(self.all_v[n], self.cand_v[:n])
            self.tp.all_gather(self.all_i[n], self.cand_i[:n])
            self.K.argmax_merge(self.all_v[n], self.all_i[n], out)
        else:
            self.tp.exchange_argmax(self.cand_v, self.cand_i, n, out)

    def _trunk(self, n, force, then_commit_k=None):
        """The main model on the n rows of in_tok: logits, greedy tokens, acceptance (and, for a
        pass without draft rows, the commit in the same kernel)."""
        R = _Residual(self, n, self.h, self.h2, self.xn)
        ordered = True
        if force:
            with self._ordered_first_launch():
                self.K.force_drafts(self.in_tok, self.ctl, self.truth, self.force_a, n - 1, self.vocab_full)
            ordered = False
        ordered = R.start_from_tokens(self.in_tok, ordered)
        for L in self.layers:
            self._block(L, R, self.ctl, ordered=ordered)
            ordered = False
        R.through(self.final_norm, self.lm_head, self.logits[:n], self.lm_lin, keep_normed=self.hid[:n])
        self._greedy(self.logits[:n], n, self.am)
        if then_commit_k is None:
            self.K.accept(self.in_tok, self.am, n, self.ctl, self.next_tok, self.log)
        else:
            self.K.accept_commit(self.in_tok, self.am, n, self.ctl, self.next_tok, self.log, self.drafts, then_commit_k)

    def _draft_rows(self, n, hid, tok):
        """MTP rows: hid [n, H] (main model, after its final norm) and the tokens that follow
        them, at positions mpos + r. Leaves the draft layer's normed output in self.mout[:n] and
        the drafted tokens in self.mtp_am[:n] (reference python/qengine/engine.py:479-496)."""
        M, c, H = self.mtp, self.cfg, self.cfg.hidden
        cat = self.cat[:n]
        R = _Residual(self, n, self.mh, self.mh2, self.xn)
        self.K.embed(self.embed, tok, R.h)
        self.K.rmsnorm1p(R.h, None, M["pre_e"], cat[:, :H], c.eps)
        self.K.rmsnorm1p(hid, None, M["pre_h"], cat[:, H:], c.eps)
        R.start_from_rows()
        if self.tp is None:
            if isinstance(M["fc"], W4Packed) and isinstance(self.linear, W4Linear):
                self._gemv(self.linear.job(cat, M["fc"], R.h))
            else:
                self._flush()
                self.linear(cat, M["fc"], R.h)
        else:  # fc is split along K: this rank multiplies its slice of [e | h]
            w = 2 * H // self.tp.size
            R.zero_then_owe(cat[:, self.tp.rank * w:(self.tp.rank + 1) * w], M["fc"], self.linear)
        self._block(M, R, self.mpos)
        if self.draft_head is not None:
            lg = self.logits[:n, :self.draft_ids.numel()]
            R.through(M["norm"], self.draft_head, lg, self.lm_lin, keep_normed=self.mout[:n])
            self._greedy(lg, n, self.mtp_am, self.draft_ids)
        else:
            R.through(M["norm"], self.lm_head, self.logits[:n], self.lm_lin, keep_normed=self.mout[:n])
            self._greedy(self.logits[:n], n, self.mtp_am)

    def _pass(self, n, mtp_rows, k, force=False):
        """Everything one graph replay does: the trunk on n rows; with mtp_rows the draft layer on
        the same n rows (which fills its K/V cache and yields draft 1 from the last kept row) and
        k - 1 chained single-row drafts; commit."""
        if not mtp_rows:
            self._trunk(n, force, then_commit_k=k)
            self._flush()
            return
        self._trunk(n, force)
        stream = torch.cuda.current_stream().cuda_stream
        if self.l2_win:
            self._flush()
            lib.qe_stream_access_window(self.l2_win[0], self.l2_win[1], 1.0, stream)
        self.K.mtp_select(self.ctl, self.mpos, -1)
        self._draft_rows(n, self.hid[:n], self.next_tok)
        if k > 0:
            self.K.mtp_select(self.ctl, self.mpos, 0, self.mout[:n], self.chain_h, self.mtp_am, self.drafts[:1])
        for j in range(1, k):
            if j > 1:
                self.K.mtp_select(self.ctl, self.mpos, j - 1)
            self._draft_rows(1, self.chain_h, self.drafts[j - 1:j])
            self.K.chain_draft(self.mtp_am, self.drafts[j:j + 1], self.mout[:1], self.chain_h)
        if self.l2_win:
            self._flush()
            lib.qe_stream_access_window(0, 0, 0.0, stream)
        self.K.commit(self.ctl, self.in_tok, self.am, self.drafts, k)
        self._flush()

    # -- graphs ----------------------------------------------------------------------------------
    def graph(self, n, mtp_rows=False, k=0, force=False):
        """The CUDA graph of one pass variant, captured on first use. The body first runs once
        eagerly (this sizes the W4 scratch, which may not grow during capture) on a side stream;
        both runs advance the sequence state, so callers reset() afterwards."""
        key = (n, mtp_rows, k, force)
        if not (1 <= n <= NMAX) or (mtp_rows and not self.has_mtp):
            raise ValueError(f"no such pass: {key}")
        if key in self.graphs:
            return self.graphs[key]
        _C.set_gdn_early(True)  # safe inside a pass: see _ordered_first_launch
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._pass(n, mtp_rows, k, force)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            count0 = launches[0]
            # Python's cyclic collector must not run inside the capture: an engine that was dropped
            # earlier (engines hold reference cycles) would have its graphs destroyed there, which
            # CUDA refuses while a stream is capturing and which invalidates this capture.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                # a process group's watchdog thread makes CUDA calls of its own during capture
                with torch.cuda.graph(g, capture_error_mode="global" if self.tp is None else "thread_local"):
                    self._pass(n, mtp_rows, k, force)
            finally:
                if gc_was_on:
                    gc.enable()
            torch.cuda.synchronize()
        finally:
            _C.set_gdn_early(False)
        self.graphs[key] = g
        self.graph_kernels[key] = launches[0] - count0
        return g

    def _need(self, keys):
        fresh = [key for key in keys if key not in self.graphs]
        for key in fresh:
            self.graph(*key)
        if fresh:
            self.reset()

    @staticmethod
    def _split(seq, size):
        return [seq[i:i + size] for i in range(0, len(seq), size)]

    def _prefill_keys(self, P, mtp, k, chunk=NMAX, skip=0):
        """Graph keys a prompt of P tokens needs: full chunks, and the last one carrying k. The
        first `skip` tokens go through wide passes."""
        sizes = [len(c) for c in self._split(range(P - skip), chunk)]
        return {(s, mtp, 0, False) for s in sizes[:-1]} | {(sizes[-1], mtp, k, False)}

    def _feed(self, tokens, follow):
        """Host -> device: the rows of the next pass and the token after them (-1: none)."""
        row = torch.full((NMAX + 1,), -1, dtype=I32)
        row[:len(tokens)] = torch.tensor(list(tokens), dtype=I32)
        row[len(tokens)] = follow
        self.in_tok.copy_(row)

    def _check_device_errors(self):
        """Bounded waits in the kernels report through sticky error words instead of hanging. Read
        them where the host synchronises anyway; a set word means the tokens are not to be trusted."""
        bad = []
        if _w4.ring_error():
            bad.append("W4 weight ring: a bulk copy did not complete")
            _w4.clear_error()
            _w4.reset_workspaces()
        if _C.attn_error():
            bad.append("attention K/V ring: a bulk copy did not complete")
        if self.tp is not None:
            err = self.tp.error()
            if err:
                bad.append(f"tensor-parallel exchange: rank {err['late_rank']} was late ({err['kind']}, row {err['row']})")
        if bad:
            raise RuntimeError("decode aborted: " + "; ".join(bad))

    # -- wide prefill passes ------------------------------------------------------------------------
    WIDE, WIDE_MIN = 64, 32  # rows per wide pass; shorter prompts are not worth a second set of graphs

    def wide_ok(self) -> bool:
        """Wide passes exist for a single GPU with every decoder matrix in the W4 wire format."""
        if self.tp is not None or not isinstance(self.linear, W4Linear):
            return False
        blocks = self.layers + ([self.mtp] if self.has_mtp else [])
        names = ("in_proj", "out", "gate_up", "down")
        mats = [L[n] for L in blocks for n in names] + ([self.mtp["fc"]] if self.has_mtp else [])
        return all(isinstance(p, W4Packed) and p.K % 128 == 0 for p in mats) and all(L["gate_up"].gate_up for L in blocks)

    def _wide_split(self, P: int, wide) -> int:
        """How many leading tokens of a prompt of P go through wide passes: the largest multiple of
        8 below P (the rest, 1..8 tokens, runs as an ordinary pass, which emits the first token)."""
        wide = self.wide_prefill if wide is None else wide
        head = ((P - 1) // NMAX) * NMAX
        return head if wide and head >= self.WIDE_MIN and self.wide_ok() else 0

    def _make_wide_buffers(self):
        c, dev, W, H = self.cfg, self.dev, self.WIDE, self.cfg.hidden

        def buf(*shape, dt=BF16):
            return torch.zeros(*shape, dtype=dt, device=dev)

        class _B:
            pass
        B = _B()
        B.tok = buf(W + 1, dt=I32)
        B.ctl = buf(W // NMAX, 32, dt=I32)  # control words of the 8-row sub-passes
        B.off = (torch.arange(W // NMAX, dtype=I32, device=dev) * NMAX).contiguous()
        B.h, B.xn, B.mo, B.hid = (buf(W, H) for _ in range(4))
        B.proj = buf(W, -(-max(c.gdn_proj_rows, c.attn_proj_rows) // 8) * 8)
        B.mix = buf(W, max(c.value_dim, c.hq * c.head_dim))
        B.act = buf(W, c.inter)
        B.q = buf(W, c.hq * c.head_dim)
        if self.has_mtp:
            B.cat, B.mh = buf(W, 2 * H), buf(W, H)
        self.wb = B

    def _wide_mixer(self, L, n, kv_only=False):
        """Token mixing of a wide pass: the mixers take 8 rows, so the rows go through them in
        sub-passes of 8, each with its own control words (position, and the 8 DeltaNet rows the
        sub-pass before it staged). kv_only: just write K and V (a draft layer during prefill:
        nothing else of it is kept)."""
        c, B = self.cfg, self.wb
        for j in range(n // NMAX):
            rows = slice(j * NMAX, (j + 1) * NMAX)
            ctl = B.ctl[j]
            if L["type"] == "linear_attention":
                pr = B.proj[rows, :c.gdn_proj_rows]
                a0, a1 = c.conv_dim, c.conv_dim + c.value_dim
                _C.gdn_step_n(pr[:, :a0], pr[:, a0:a1], pr[:, a1:a1 + c.hv], pr[:, a1 + c.hv:], L["ring"],
                              L["conv_w"], L["A_log"], L["dt_bias"], L["norm_w"], L["S"], L["st_k"], L["st_v"],
                              L["st_g"], ctl, B.mix[rows, :c.value_dim], c.hk, c.eps, q=self.GDN_Q)
            else:
                pr = B.proj[rows, :c.attn_proj_rows]
                nq = c.hq * 2 * c.head_dim
                nk = nq + c.hkv * c.head_dim
                _C.attn_prep(pr[:, :nq], pr[:, nq:nk], pr[:, nk:], L["q_norm"], L["k_norm"], self.inv_freq, ctl,
                             B.q[rows], L["kc"], L["vc"], c.eps)
                if not kv_only:
                    _C.attn_decode(B.q[rows], L["kc"], L["vc"], ctl, pr[:, :nq], self.part_o, self.part_ml,
                                   B.mix[rows, :c.hq * c.head_dim])
        width = c.value_dim if L["type"] == "linear_attention" else c.hq * c.head_dim
        return B.mix[:n, :width]

    def _wide_pass(self, n, mtp):
        """One prefill pass over n rows (a multiple of 8, at most WIDE) of wb.tok: what n / 8
        ordinary prefill passes do to the K/V caches, the DeltaNet state and the position, with
        every matrix streamed once (`_w4.gemm`). No logits: the pass that follows emits them.
        Follows python/qengine/engine.py:434-477 (layer, main) and :479-496 (draft layer) of the
        reference with 8-row sub-passes for the mixers."""
        c, B, lin, eps = self.cfg, self.wb, self.linear, self.cfg.eps
        nb = n // NMAX
        self._flush()
        # control words of the sub-passes: positions 8 apart; every sub-pass but the first finds the
        # 8 DeltaNet rows of the one before it pending
        B.ctl[:nb].copy_(self.ctl.expand(nb, -1))
        B.ctl[:nb, self.POS].add_(B.off[:nb])
        if nb > 1:
            B.ctl[1:nb, self.PENDING].fill_(NMAX)
        h, xn, mo = B.h[:n], B.xn[:n], B.mo[:n]

        def mm(x, p, out):
            _w4.gemm(x, p.qw, p.scales, out, p.M, swiglu=p.gate_up)

        def block(L, stream, delta, table_tok=None):
            width = c.gdn_proj_rows if L["type"] == "linear_attention" else c.attn_proj_rows
            if table_tok is not None:  # rows = embedding rows of the tokens
                lin.norm_rows(self.embed, None, L["in_norm"], eps, xn, tok=table_tok, h_out=stream)
            else:
                lin.norm_rows(stream, delta, L["in_norm"], eps, xn, h_out=stream if delta is not None else None)
            mm(xn, L["in_proj"], B.proj[:n, :width])

        first = True
        for L in self.layers:
            block(L, h, None if first else mo, table_tok=B.tok if first else None)
            first = False
            mixed = self._wide_mixer(L, n)
            mm(mixed, L["out"], mo)
            lin.norm_rows(h, mo, L["post_norm"], eps, xn, h_out=h)
            mm(xn, L["gate_up"], B.act[:n])
            mm(B.act[:n], L["down"], mo)
        if mtp:
            # draft layer on the same rows (reference :479-496): input fc([norm(embed(next token)) |
            # norm(final-normed trunk row)]); during prefill only its K/V rows (or DeltaNet state) stay
            M, H = self.mtp, c.hidden
            lin.norm_rows(h, mo, self.final_norm, eps, B.hid[:n], h_out=h)
            cat = B.cat[:n]
            lin.norm_rows(self.embed, None, M["pre_e"], eps, cat[:, :H], tok=B.tok[1:])
            lin.norm_rows(B.hid[:n], None, M["pre_h"], eps, cat[:, H:])
            mm(cat, M["fc"], B.mh[:n])
            block(M, B.mh[:n], None)
            self._wide_mixer(M, n, kv_only=M["type"] != "linear_attention")
        # commit: the position moves on by n; the last sub-pass left 8 DeltaNet rows pending
        self.ctl[self.POS].add_(n)
        self.ctl[self.PENDING].fill_(NMAX)

    def wide_graph(self, n, mtp=False):
        """The CUDA graph of a wide prefill pass over n rows, captured on first use (like `graph`)."""
        key = ("wide", n, bool(mtp))
        if n % NMAX or not NMAX <= n <= self.WIDE or (mtp and not self.has_mtp) or not self.wide_ok():
            raise ValueError(f"no such pass: {key}")
        if key in self.graphs:
            return self.graphs[key]
        if self.wb is None:
            self._make_wide_buffers()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._wide_pass(n, mtp)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        count0 = launches[0]
        gc.collect()  # see graph()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, capture_error_mode="global"):
                self._wide_pass(n, mtp)
        finally:
            if gc_was_on:
                gc.enable()
        torch.cuda.synchronize()
        self.graphs[key] = g
        self.graph_kernels[key] = launches[0] - count0
        return g

    def _wide_blocks(self, head):
        return [min(self.WIDE, head - at) for at in range(0, head, self.WIDE)]

    def _need_wide(self, head, mtp):
        fresh = [n for n in set(self._wide_blocks(head)) if ("wide", n, bool(mtp)) not in self.graphs]
        for n in fresh:
            self.wide_graph(n, mtp)
        if fresh:
            self.reset()

    # -- public loops ---------------------------------------------------------------------------
    def prefill(self, prompt, mtp=False, k=0, chunk=NMAX, wide=None):
        """Feed the prompt `chunk` rows per pass. The last row's greedy token is the first
        generated token (log[len(prompt)]); with mtp / k the drafts of the first verify pass are
        ready afterwards. Leaves the engine in decode / verify mode. Expects reset() and captured
        graphs (`generate*` take care of both).
        wide (default: the engine's `wide_prefill`): all but the last 1..8 tokens go through passes
        of up to 64 rows (`_wide_pass`); the state they leave agrees with the 8-row passes to
        rounding (the GEMM adds a tile's groups in another order than the GEMV), not bit for bit."""
        prompt = list(prompt)
        head = self._wide_split(len(prompt), wide)
        self.ctl[self.MODE].fill_(0)
        at = 0
        for n in self._wide_blocks(head):
            row = torch.tensor(prompt[at:at + n + 1], dtype=I32)
            self.wb.tok[:n + 1].copy_(row)
            self.wide_graph(n, mtp).replay()
            at += n
        pieces = self._split(prompt[head:], chunk)
        for i, piece in enumerate(pieces):
            last = i == len(pieces) - 1
            self._feed(piece, -1 if last else pieces[i + 1][0])
            self.graph(len(piece), mtp, k if last else 0).replay()
        self.ctl[self.MODE].fill_(1)

    @torch.no_grad()
    def generate(self, prompt, n_new, timing=False, chunk=NMAX, wide=None):
        """Plain greedy decoding: prefill, then n_new - 1 single-row passes. Returns the n_new token
        ids; timing=True returns (tokens, prefill seconds, decode seconds)."""
        P = len(prompt)
        first = self.start_pos + P
        if first + n_new + 1 > self.max_len:
            raise ValueError("sequence does not fit max_len")
        step_key = (1, False, 0, False)
        head = self._wide_split(P, wide)
        self._need_wide(head, False)
        self._need(self._prefill_keys(P, False, 0, chunk, skip=head) | {step_key})
        self.reset()
        t = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        t[0].record()
        self.prefill(prompt, chunk=chunk, wide=wide)
        t[1].record()
        step = self.graphs[step_key]
        for _ in range(n_new - 1):
            step.replay()
        t[2].record()
        torch.cuda.synchronize()
        self._check_device_errors()
        out = self.log[first:first + n_new].tolist()
        return (out, t[0].elapsed_time(t[1]) / 1e3, t[1].elapsed_time(t[2]) / 1e3) if timing else out

    @torch.no_grad()
    def generate_spec(self, prompt, n_new, k, timing=False, chunk=NMAX, force_accept=None, truth=None, wide=None):
        """Greedy speculative decoding with k MTP drafts per cycle (verify over k + 1 rows). The
        output equals `generate` token for token. force_accept = a (0..k) together with truth =
        prompt + known greedy continuation overwrites the drafts before every verify so that
        exactly `a` are accepted (measurement harness). timing=True returns (tokens, prefill s,
        decode s, stats)."""
        if not self.has_mtp or not 1 <= k <= NMAX - 1:
            raise ValueError("speculative decoding needs the MTP layer and 1 <= k <= 7")
        P = len(prompt)
        first = self.start_pos + P
        if first + n_new + 2 * NMAX + 2 > self.max_len:
            raise ValueError("sequence does not fit max_len")
        forced = force_accept is not None
        if forced:
            if truth is None or not 0 <= force_accept <= k:
                raise ValueError("force_accept needs truth and 0 <= a <= k")
            self.truth = torch.tensor([0] * self.start_pos + list(truth), dtype=I32, device=self.dev)  # by position
            self.force_a = int(force_accept)
            self.graphs.pop((k + 1, True, k, True), None)  # the graph holds the old truth buffer
        cycle_key = (k + 1, True, k, forced)
        head = self._wide_split(P, wide)
        self._need_wide(head, True)
        self._need(self._prefill_keys(P, True, k, chunk, skip=head) | {cycle_key})
        self.reset()
        t = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        t[0].record()
        self.prefill(prompt, mtp=True, k=k, chunk=chunk, wide=wide)
        self.ctl[self.CYCLES:self.ACCEPTED + 1].zero_()
        self.ctl[16:].zero_()
        t[1].record()
        cycle = self.graphs[cycle_key]
        goal, pos = first + n_new - 1, first
        while pos < goal:
            # every cycle yields at least one token and at most k + 1: replay as many as cannot
            # overshoot, then look at the position (the only host sync of the loop)
            for _ in range(max(1, (goal - pos) // (k + 1))):
                cycle.replay()
            pos = int(self.ctl[self.POS].item())
        t[2].record()
        torch.cuda.synchronize()
        self._check_device_errors()
        out = self.log[first:first + n_new].tolist()
        if not timing:
            return out
        c = self.ctl.tolist()
        cycles, kept, hist = c[self.CYCLES], c[self.ACCEPTED], c[16:16 + k + 1]
        reach = [sum(hist[d:]) for d in range(k + 1)]  # cycles that kept at least d drafts
        stats = {"cycles": cycles, "accepted": kept, "accept_rate": kept / max(1, cycles * k),
                 "tokens_per_cycle": 1 + kept / max(1, cycles), "hist": hist,
                 "accept_by_depth": [reach[d] / max(1, reach[d - 1]) for d in range(1, k + 1)]}
        return out, t[0].elapsed_time(t[1]) / 1e3, t[1].elapsed_time(t[2]) / 1e3, stats

    @torch.no_grad()
    def sequence_logits(self, seq, keep="full", chunk=NMAX):
        """Teacher forcing: `seq` goes through prefill passes; returns the logits of every position
        [T, V] bf16 (keep='full') or their argmax [T] (keep='argmax')."""
        pieces = self._split(list(seq), chunk)
        self._need({(len(p), False, 0, False) for p in pieces})
        self.reset()
        full = keep == "full"
        out = torch.empty((len(seq), self.cfg.vocab) if full else (len(seq),), dtype=BF16 if full else I32,
                          device=self.dev)
        self.ctl[self.MODE].fill_(0)
        at = 0
        for i, piece in enumerate(pieces):
            self._feed(piece, pieces[i + 1][0] if i + 1 < len(pieces) else -1)
            self.graph(len(piece), False, 0).replay()
            out[at:at + len(piece)].copy_(self.logits[:len(piece)] if full else self.am[:len(piece)])
            at += len(piece)
        torch.cuda.synchronize()
        self._check_device_errors()
        return out

    @torch.no_grad()
    def mtp_rows_logits(self, seq):
        """Validation helper: teacher-forced single-row passes with the MTP rows on. Returns the
        main model's hidden rows after the final norm [T, H] and the MTP logits [T, V]; MTP row t
        sees the hidden row t and token seq[t + 1] (at the last position: the model's own choice)."""
        self._need({(1, True, 0, False)})
        self.reset()
        T = len(seq)
        hid = torch.empty(T, self.cfg.hidden, dtype=BF16, device=self.dev)
        lg = torch.empty(T, self.cfg.vocab, dtype=BF16, device=self.dev)
        self.ctl[self.MODE].fill_(0)
        for t in range(T):
            self._feed([seq[t]], seq[t + 1] if t + 1 < T else -1)
            self.graph(1, True, 0).replay()
            hid[t].copy_(self.hid[0])
            lg[t].copy_(self.logits[0])
        torch.cuda.synchronize()
        self._check_device_errors()
        return hid, lg
