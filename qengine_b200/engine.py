"""Batch-1 decode engine: plain greedy decoding and MTP speculative decoding, every pass captured
as one CUDA graph with all bookkeeping on the device.

Public surface mirrors the reference engine (python/qengine/engine.py:189-687): `Engine`,
`.generate`, `.generate_spec`, `.prefill`, `.graph`, `.sequence_logits`, `.mtp_rows_logits`,
`.reset`, and the linear backends `W4Linear` / `BF16Linear`. The model comes as a weights dict
in the fused layout (see qengine_b200.synth) instead of a checkpoint directory: weight loading,
quantisation caches and tokenizers are outside this library.

A pass runs n = 1..8 rows (tokens at positions pos .. pos + n - 1):
  plain decode  n = 1;
  verify        n = k + 1 rows [last token, draft 1..k]; the longest prefix of drafts equal to
                the model's own argmax is kept, plus the model's next token;
  prefill       up to 8 prompt tokens per pass.
One graph replay = one decode step or one whole speculative cycle (verify, MTP rows, k - 1
chained drafts, commit); the host only reads `pos` once per batch of cycles.

Rollback: KV rows of rejected drafts are overwritten later; DeltaNet rows are staged as
per-position checkpoints and only the kept ones are replayed by the next pass (deltanet.cu).
Every kernel computes row r of an n-row pass exactly as a 1-row pass would, so speculative output
is token-identical to plain greedy output.
"""
from __future__ import annotations

import torch

from . import _C
from ._lib import launches
from .quant import W4Packed
from .synth import Config

BF16, I32, F32 = torch.bfloat16, torch.int32, torch.float32


def _lib_sm_count() -> int:
    from ._lib import lib
    return max(1, int(lib.qe_sm_count()))
NMAX = 8  # rows per pass


class BF16Linear:
    """BF16 GEMV backend (weights read once for all rows, fp32 accumulate)."""
    name = "bf16"

    def prepare(self, w):
        return w.contiguous()

    def __call__(self, x, w, out):
        _C.gemv_bf16(w, x, out)


class W4Linear:
    """Adapter over the W4A16 GEMV (`_w4`), the only caller of that API
    (reference python/qengine/engine.py:74-115). Launch keyword arguments are passed through."""
    name = "w4"

    def __init__(self, ksplit_max=64, **kw):
        self.ksplit_max, self.kw = ksplit_max, dict(kw)
        # at least 6 units per warp: the 5120 x 6144 out_proj (320 tiles of 48 units) then runs on
        # 2,560 warps = 320 CTAs of exactly one tile each, so no tile crosses a CTA boundary and all
        # of them finish through shared memory: 3 % of the whole W4 time of a token (measured; 5 and
        # 7 are both slower, and forcing the same alignment on `down` or the lm_head costs more in
        # idle warp slots than it saves)
        self.kw.setdefault("min_units", 6)

    def prepare(self, w):
        from .quant import quantize_w4
        return quantize_w4(w)

    def prepare_gate_up(self, wg, wu):
        from .quant import quantize_w4_gate_up
        return quantize_w4_gate_up(wg, wu)

    def _ks(self, p, n):
        from . import _w4
        ks = _w4.auto_ksplit(p.qw.shape[0] * 16, p.qw.shape[1] * 64, n, self.kw.get("warps", 8) or 8)
        return min(ks, self.ksplit_max)

    def __call__(self, x, p, out):
        from . import _w4
        _w4.gemv(x, p.qw, p.scales, out, p.M, ksplit=self._ks(p, x.shape[0]), **self.kw)

    def gate_up(self, x, p, out):
        from . import _w4
        _w4.gemv_swiglu(x, p.qw, p.scales, out, p.M, ksplit=self._ks(p, x.shape[0]), **self.kw)

    def partial(self, x, p, out32):
        """Unrounded fp32 result: one rank's partial sums of a matrix split along K."""
        from . import _w4
        _w4.gemv_act16(x, p.qw, p.scales, out32, p.M, ksplit=self._ks(p, x.shape[0]), **self.kw)

    @staticmethod
    def dequantize(p):
        from .quant import dequantize_w4
        return dequantize_w4(p)


class Engine:
    GDN_Q = 4
    POS, PENDING, MODE, M, CYCLES, ACCEPTED = range(6)

    def __init__(self, cfg: Config, weights: dict, max_len: int = 4096, linear=None, device="cuda",
                 mtp: bool = True, attn_splits: int | None = None, draft_vocab: int | None = None, tp=None):
        """weights: dict from qengine_b200.synth.build_model (already on `device`).
        tp: a qengine_b200.tp.TPGroup for tensor parallelism; then `cfg` is still the whole model's
        configuration and `weights` is this rank's shard (qengine_b200.tp.shard_model).
        attn_splits: flash-decoding splits per head (fixed so the graphs are static); default 16,
        more for caches longer than 8192 positions. draft_vocab: MTP drafts score only the first `draft_vocab` token ids
        (pruned draft head through the argmax id map); verify keeps the full head."""
        self.tp, self.vocab_full, self.vocab_base = tp, cfg.vocab, 0
        if tp is not None:
            from .tp import local_config
            tp.open(cfg.hidden)
            cfg = local_config(cfg, tp.size)
            self.vocab_base = tp.rank * cfg.vocab
        self.cfg, self.max_len = cfg, max_len
        self.dev = torch.device(device)
        # the shards of a tensor-parallel rank are small enough that every warp should get work:
        # 4 units per warp there (measured: 2.17 vs 2.45 ms per token at 4 ranks), 6 on one GPU
        self.linear = linear or (W4Linear() if tp is None else W4Linear(min_units=4))
        self.lm_lin = self.linear
        self.embed, self.final_norm = weights["embed"], weights["final_norm"]
        self.lm_head = weights["lm_head"]
        self.layers = [dict(L) for L in weights["layers"]]
        self.has_mtp = bool(mtp and weights.get("mtp"))
        self.mtp = dict(weights["mtp"]) if self.has_mtp else None
        # long caches: a multiple of 6 selects the tensor-core split kernel (6 splits per CTA);
        # one CTA per SM and row, i.e. 6 * ceil(SMs / KV heads) splits
        self.ATTN_SPLITS = attn_splits or (16 if max_len <= 8192 else 6 * -(-_lib_sm_count() // cfg.hkv))
        self.draft_head = self.draft_ids = None
        if draft_vocab and self.has_mtp:
            self._build_draft_head(draft_vocab)
        self._alloc()
        self.graphs = {}
        self.graph_kernels = {}  # kernels of this library per captured graph
        self.start_pos = 0     # positions [0, start_pos) hold a pre-filled context (set_context)
        self.force_a = -1      # forced acceptance length for verify passes (< 0: off)
        self.truth = torch.zeros(1, dtype=I32, device=self.dev)
        _C.set_gdn_early(True)  # safe here: passes start with a fully ordered kernel (see _main)

    # ------------------------------------------------------------------------------------------
    def _build_draft_head(self, nv: int):
        """Pruned draft head: the first nv rows of the packed lm_head (ids 0..nv-1), no copy of
        the codes is re-quantised; nv must be a multiple of 16. Under tensor parallelism every rank
        keeps the first nv / t rows of its own vocabulary slice."""
        if self.tp is not None:
            nv //= self.tp.size
        assert nv % 16 == 0 and isinstance(self.lm_head, W4Packed)
        p = self.lm_head
        self.draft_head = W4Packed(p.qw[:nv // 16].contiguous(), p.scales[:nv // 16].contiguous(), nv, p.K)
        self.draft_ids = torch.arange(nv, dtype=I32, device=self.dev)

    def _alloc(self):
        cfg, dev, ml, N = self.cfg, self.dev, self.max_len, NMAX
        H, I, V = cfg.hidden, cfg.inter, cfg.vocab
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=dev)
        self.ctl = z(32, dt=I32)
        self.in_tok = z(N + 1, dt=I32)
        self.am, self.next_tok, self.drafts, self.mtp_am = (z(N, dt=I32) for _ in range(4))
        self.mpos = z(1, dt=I32)
        self.log = z(ml, dt=I32)
        self.h, self.xn, self.mo, self.hid = z(N, H), z(N, H), z(N, H), z(N, H)
        pw = max(cfg.gdn_proj_rows, cfg.attn_proj_rows)
        self.proj = z(N, (pw + 7) // 8 * 8)
        self.mix = z(N, max(cfg.value_dim, cfg.hq * cfg.head_dim))
        self.gu, self.act = z(N, 2 * I), z(N, I)
        self.logits = z(N, V)
        self.am_v, self.am_i = z(N * 256, dt=F32), z(N * 256, dt=I32)
        self.q = z(N, cfg.hq * cfg.head_dim)
        self.part_o = z(N, cfg.hq, self.ATTN_SPLITS, cfg.head_dim, dt=F32)
        self.part_ml = z(N, cfg.hq, self.ATTN_SPLITS, 2, dt=F32)
        rd = cfg.rotary_dim  # built on the CPU in fp32 like the reference, then moved
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, rd, 2, dtype=F32) / rd))).to(dev)
        for L in self.layers:
            if L["type"] == "linear_attention":
                L["ring"] = z(16, cfg.conv_dim)
                L["S"] = z(cfg.hv, cfg.dk, cfg.dv, dt=F32)
                L["st_k"], L["st_v"] = z(N, cfg.hv, cfg.dk, dt=F32), z(N, cfg.hv, cfg.dv, dt=F32)
                L["st_g"] = z(N, cfg.hv, 2, dt=F32)
            else:
                L["kc"], L["vc"] = z(cfg.hkv, ml, cfg.head_dim), z(cfg.hkv, ml, cfg.head_dim)
        if self.has_mtp:
            self.mtp["kc"], self.mtp["vc"] = z(cfg.hkv, ml, cfg.head_dim), z(cfg.hkv, ml, cfg.head_dim)
            self.cat = z(N, 2 * H)
            self.mh, self.mout, self.chain_h = z(N, H), z(N, H), z(1, H)
        if self.tp is not None:
            t = self.tp.size
            self.part32 = z(N, H, dt=F32)
            self.parts = {n: z(t, n, H, dt=F32) for n in range(1, N + 1)}
            self.cand_v, self.cand_i = z(N, dt=F32), z(N, dt=I32)
            self.all_v = {n: z(t, n, dt=F32) for n in range(1, N + 1)}
            self.all_i = {n: z(t, n, dt=I32) for n in range(1, N + 1)}

    def reset(self):
        """Empty sequence. KV caches need no clearing (only [0, pos] is ever read)."""
        for L in self.layers:
            if "ring" in L:
                L["ring"].zero_()
                L["S"].zero_()
        self.ctl.zero_()
        if self.start_pos:
            self.ctl[self.POS].fill_(self.start_pos)

    @torch.no_grad()
    def set_context(self, length: int, seed: int = 99):
        """Measurement harness for long caches: pretend `length` positions were already decoded.
        K and V rows [0, length) of every attention layer (and the draft head's) are filled with
        seeded N(0, 1) values; sequences then start at position `length` (DeltaNet state empty)."""
        assert 0 <= length < self.max_len - 2 * NMAX
        g = torch.Generator(device=self.dev).manual_seed(seed)
        for L in self.layers + ([self.mtp] if self.has_mtp else []):
            if "kc" in L:
                for c in (L["kc"], L["vc"]):
                    for h in range(c.shape[0]):
                        c[h, :length].copy_(torch.randn(length, c.shape[2], generator=g, device=self.dev))
        self.start_pos = int(length)
        self.reset()

    # ------------------------------------------------------------------------------------------
    # A matrix whose input is split over tensor-parallel ranks (out / o_proj, down, mtp.fc) leaves
    # its result "pending": single GPU -> bf16 in self.mo; tensor parallel -> every rank's fp32
    # partial rows gathered into self.parts[n]. The next norm adds the pending rows to the residual.
    def _ksplit(self, x, p, n, lin):
        if self.tp is None:
            lin(x, p, self.mo[:n])
        else:
            lin.partial(x, p, self.part32[:n])
            if self.tp.transport == "nccl":
                self.tp.all_gather(self.parts[n], self.part32[:n])

    def _norm(self, h, pending, w, out, eps, n):
        if not pending:
            _C.rmsnorm1p(h, None, w, out, eps)
        elif self.tp is None:
            _C.rmsnorm1p(h, self.mo[:n], w, out, eps)
        elif self.tp.transport == "nccl":
            _C.rmsnorm1p_parts(h, self.parts[n], w, out, eps)
        else:  # exchange of the partial rows fused into the norm, over peer memory
            self.tp.exchange_norm(h, self.part32[:n], w, out, eps)

    def _argmax(self, logits, n, out, idmap=None):
        """Greedy token per row (lowest id on ties); vocabulary shards exchange (value, id)."""
        ws_v, ws_i = self.am_v[:n * 256], self.am_i[:n * 256]
        if self.tp is None:
            _C.argmax(logits, ws_v, ws_i, out, idmap)
            return
        _C.argmax_v(logits, ws_v, ws_i, self.cand_i, self.cand_v, self.vocab_base, idmap)
        if self.tp.transport == "nccl":
            self.tp.all_gather(self.all_v[n], self.cand_v[:n])
            self.tp.all_gather(self.all_i[n], self.cand_i[:n])
            _C.argmax_merge(self.all_v[n], self.all_i[n], out)
        else:
            self.tp.exchange_argmax(self.cand_v, self.cand_i, n, out)

    def _layer(self, L, n, h, eps, first, pos, lin=None):
        """One decoder layer on rows h[:n]; the previous sub-layer's output in self.mo is added by
        this layer's first norm unless `first`."""
        cfg, lin = self.cfg, lin or self.linear
        xn = self.xn[:n]
        self._norm(h, not first, L["in_norm"], xn, eps, n)
        if L["type"] == "linear_attention":
            pr = self.proj[:n, :cfg.gdn_proj_rows]
            lin(xn, L["in_proj"], pr)
            c0, c1 = cfg.conv_dim, cfg.conv_dim + cfg.value_dim
            out = self.mix[:n, :cfg.value_dim]
            _C.gdn_step_n(pr[:, :c0], pr[:, c0:c1], pr[:, c1:c1 + cfg.hv], pr[:, c1 + cfg.hv:], L["ring"],
                          L["conv_w"], L["A_log"], L["dt_bias"], L["norm_w"], L["S"], L["st_k"],
                          L["st_v"], L["st_g"], self.ctl, out, cfg.hk, eps, q=self.GDN_Q)
        else:
            pr = self.proj[:n, :cfg.attn_proj_rows]
            lin(xn, L["in_proj"], pr)
            q0 = cfg.hq * 2 * cfg.head_dim
            k1 = q0 + cfg.hkv * cfg.head_dim
            qg, q = pr[:, :q0], self.q[:n]
            _C.attn_prep(qg, pr[:, q0:k1], pr[:, k1:], L["q_norm"], L["k_norm"], self.inv_freq, pos, q,
                         L["kc"], L["vc"], eps)
            out = self.mix[:n, :cfg.hq * cfg.head_dim]
            _C.attn_decode(q, L["kc"], L["vc"], pos, qg, self.part_o, self.part_ml, out)
        self._ksplit(out, L["out"], n, lin)
        self._norm(h, True, L["post_norm"], xn, eps, n)
        if L.get("fused_swiglu", False):
            lin.gate_up(xn, L["gate_up"], self.act[:n])
        else:
            lin(xn, L["gate_up"], self.gu[:n])
            _C.swiglu(self.gu[:n], self.act[:n])
        self._ksplit(self.act[:n], L["down"], n, lin)

    def _main(self, n, force=False):
        eps, k = self.cfg.eps, n - 1
        h = self.h[:n]
        # The first kernel of a pass is launched in plain stream order: it starts only after the
        # previous pass has fully finished, so everything that pass wrote (pos, pending, state,
        # checkpoints) is safe to read even from the early sections of this pass's kernels.
        _C.set_pdl_launch(False)
        if force:
            _C.force_drafts(self.in_tok, self.ctl, self.truth, self.force_a, k, self.vocab_full)
            _C.set_pdl_launch(True)
            _C.embed(self.embed, self.in_tok, h)
        else:
            _C.embed(self.embed, self.in_tok, h)
            _C.set_pdl_launch(True)
        for i, L in enumerate(self.layers):
            self._layer(L, n, h, eps, i == 0, self.ctl)
        self._norm(h, True, self.final_norm, self.hid[:n], eps, n)
        self.lm_lin(self.hid[:n], self.lm_head, self.logits[:n])
        self._argmax(self.logits[:n], n, self.am)
        _C.accept(self.in_tok, self.am, n, self.ctl, self.next_tok, self.log)

    def _mtp(self, n, hid, tok):
        """MTP rows: hid [n, H] (after the final norm), tok int32 next tokens, positions mpos + r.
        Output: self.mout[:n] (after mtp.norm) and self.mtp_am[:n] (draft tokens)."""
        M, eps, H = self.mtp, self.cfg.eps, self.cfg.hidden
        mh, cat = self.mh[:n], self.cat[:n]
        _C.embed(self.embed, tok, mh)
        _C.rmsnorm1p(mh, None, M["pre_e"], cat[:, :H], eps)
        _C.rmsnorm1p(hid, None, M["pre_h"], cat[:, H:], eps)
        if self.tp is None:
            self.linear(cat, M["fc"], mh)
        else:  # this rank's slice of [e | h]; the summed fc rows are added to a zeroed residual
            w = 2 * H // self.tp.size
            self._ksplit(cat[:, self.tp.rank * w:(self.tp.rank + 1) * w], M["fc"], n, self.linear)
            mh.zero_()
        self._layer(M, n, mh, eps, self.tp is None, self.mpos)
        self._norm(mh, True, M["norm"], self.mout[:n], eps, n)
        if self.draft_head is not None:
            lg = self.logits[:n, :self.draft_ids.numel()]
            self.lm_lin(self.mout[:n], self.draft_head, lg)
            self._argmax(lg, n, self.mtp_am, self.draft_ids)
        else:
            self.lm_lin(self.mout[:n], self.lm_head, self.logits[:n])
            self._argmax(self.logits[:n], n, self.mtp_am)

    def _pass(self, n, mtp_rows, k, force=False):
        """Graph body: main pass on n rows; optionally MTP over the n rows (fills the MTP cache and
        gives draft 1 from the last kept row) and k - 1 chained drafts; then commit."""
        self._main(n, force)
        if mtp_rows:
            _C.mtp_select(self.ctl, self.mpos, -1)
            self._mtp(n, self.hid[:n], self.next_tok)
            if k > 0:
                _C.mtp_select(self.ctl, self.mpos, 0, self.mout[:n], self.chain_h, self.mtp_am, self.drafts[:1])
            for j in range(1, k):
                if j > 1:
                    _C.mtp_select(self.ctl, self.mpos, j - 1)
                self._mtp(1, self.chain_h, self.drafts[j - 1:j])
                self.drafts[j:j + 1].copy_(self.mtp_am[:1])
                self.chain_h.copy_(self.mout[:1])
        _C.commit(self.ctl, self.in_tok, self.am, self.drafts, k)

    def graph(self, n, mtp_rows=False, k=0, force=False):
        """CUDA graph of one pass variant, captured on first use. Capturing runs the body once
        eagerly (which also sizes the W4 workspace) and changes the sequence state: call reset()."""
        key = (n, mtp_rows, k, force)
        assert 1 <= n <= NMAX and (not mtp_rows or self.has_mtp)
        if key not in self.graphs:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._pass(n, mtp_rows, k, force)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = launches[0]
            # with collectives in the graph, other threads of the process group must stay free to
            # make CUDA calls during capture
            mode = "global" if self.tp is None else "thread_local"
            with torch.cuda.graph(g, capture_error_mode=mode):
                self._pass(n, mtp_rows, k, force)
            torch.cuda.synchronize()
            self.graphs[key] = g
            self.graph_kernels[key] = launches[0] - before
        return self.graphs[key]

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _chunks(seq, size):
        return [seq[i:i + size] for i in range(0, len(seq), size)]

    def _prefill_keys(self, P, mtp, k, chunk=NMAX):
        sizes = [len(c) for c in self._chunks(list(range(P)), chunk)]
        keys = {(s, mtp, 0, False) for s in sizes[:-1]}
        keys.add((sizes[-1], mtp, k, False))
        return keys

    def _ensure(self, keys):
        new = [k for k in keys if k not in self.graphs]
        for key in new:
            self.graph(*key)
        if new:
            self.reset()

    def prefill(self, prompt, mtp=False, k=0, chunk=NMAX):
        """Feed the prompt in passes of `chunk` rows. The last row's argmax is the first generated
        token (log[len(prompt)]); with mtp/k the drafts for the first verify are ready. Leaves the
        engine in decode/verify mode. Assumes reset() and existing graphs."""
        chunks = self._chunks(prompt, chunk)
        self.ctl[self.MODE].fill_(0)
        buf = torch.full((NMAX + 1,), -1, dtype=I32)
        for ci, c in enumerate(chunks):
            last = ci == len(chunks) - 1
            buf.fill_(-1)
            buf[:len(c)] = torch.tensor(c, dtype=I32)
            if not last:
                buf[len(c)] = chunks[ci + 1][0]
            self.in_tok.copy_(buf)
            self.graph(len(c), mtp, k if last else 0).replay()
        self.ctl[self.MODE].fill_(1)

    @torch.no_grad()
    def generate(self, prompt, n_new, timing=False, chunk=NMAX):
        """Plain greedy: prefill, then n_new - 1 one-row passes. Returns n_new token ids
        (timing=True adds prefill_s, decode_s)."""
        P, P0 = len(prompt), self.start_pos + len(prompt)
        assert P0 + n_new + 1 <= self.max_len
        self._ensure(self._prefill_keys(P, False, 0, chunk) | {(1, False, 0, False)})
        self.reset()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        self.prefill(prompt, chunk=chunk)
        e1.record()
        g = self.graphs[(1, False, 0, False)]
        for _ in range(n_new - 1):
            g.replay()
        e2.record()
        torch.cuda.synchronize()
        gen = self.log[P0:P0 + n_new].tolist()
        if timing:
            return gen, e0.elapsed_time(e1) / 1e3, e1.elapsed_time(e2) / 1e3
        return gen

    @torch.no_grad()
    def generate_spec(self, prompt, n_new, k, timing=False, chunk=NMAX, force_accept=None, truth=None):
        """Greedy speculative decoding with k MTP drafts per cycle (verify n = k + 1 rows). Output
        equals `generate` token for token. force_accept = a (0..k) with truth = prompt + known
        greedy continuation replaces the drafts before every verify so that exactly `a` are
        accepted (measurement harness). timing=True adds prefill_s, decode_s and a stats dict."""
        assert self.has_mtp and 1 <= k <= NMAX - 1
        P, P0 = len(prompt), self.start_pos + len(prompt)
        assert P0 + n_new + 2 * NMAX + 2 <= self.max_len
        force = force_accept is not None
        if force:
            assert truth is not None and 0 <= force_accept <= k
            # indexed by absolute position
            self.truth = torch.tensor([0] * self.start_pos + list(truth), dtype=I32, device=self.dev)
            self.force_a = int(force_accept)
            self.graphs.pop((k + 1, True, k, True), None)  # truth buffer address changed
        self._ensure(self._prefill_keys(P, True, k, chunk) | {(k + 1, True, k, force)})
        self.reset()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        self.prefill(prompt, mtp=True, k=k, chunk=chunk)
        self.ctl[self.CYCLES:self.ACCEPTED + 1].zero_()
        self.ctl[16:].zero_()
        e1.record()
        g = self.graphs[(k + 1, True, k, force)]
        target = P0 + n_new - 1
        pos = P0
        while pos < target:
            for _ in range(max(1, (target - pos) // (k + 1))):
                g.replay()
            pos = int(self.ctl[self.POS].item())  # the only host sync: once per batch of cycles
        e2.record()
        torch.cuda.synchronize()
        gen = self.log[P0:P0 + n_new].tolist()
        if not timing:
            return gen
        c = self.ctl.tolist()
        stats = {"cycles": c[self.CYCLES], "accepted": c[self.ACCEPTED],
                 "accept_rate": c[self.ACCEPTED] / max(1, c[self.CYCLES] * k),
                 "tokens_per_cycle": 1 + c[self.ACCEPTED] / max(1, c[self.CYCLES]),
                 "hist": c[16:16 + k + 1]}
        return gen, e0.elapsed_time(e1) / 1e3, e1.elapsed_time(e2) / 1e3, stats

    @torch.no_grad()
    def sequence_logits(self, seq, keep="full", chunk=NMAX):
        """Teacher forcing: feed `seq` in prefill passes; per-position logits [T, V] bf16
        (keep='full') or argmax ids [T] (keep='argmax')."""
        T = len(seq)
        chunks = self._chunks(seq, chunk)
        self._ensure({(len(c), False, 0, False) for c in chunks})
        self.reset()
        full = keep == "full"
        out = torch.empty((T, self.cfg.vocab) if full else (T,), dtype=BF16 if full else I32, device=self.dev)
        self.ctl[self.MODE].fill_(0)
        buf = torch.full((NMAX + 1,), -1, dtype=I32)
        for ci, c in enumerate(chunks):
            buf.fill_(-1)
            buf[:len(c)] = torch.tensor(c, dtype=I32)
            if ci + 1 < len(chunks):
                buf[len(c)] = chunks[ci + 1][0]
            self.in_tok.copy_(buf)
            self.graph(len(c), False, 0).replay()
            o = ci * chunk
            out[o:o + len(c)].copy_(self.logits[:len(c)] if full else self.am[:len(c)])
        torch.cuda.synchronize()
        return out

    @torch.no_grad()
    def mtp_rows_logits(self, seq):
        """Validation helper: teacher-forced one-row passes with MTP rows on; returns (main hidden
        after the final norm [T, H], MTP logits [T, V]); MTP row t uses the hidden at t and the
        next token seq[t + 1] (the model's own argmax at the last position)."""
        self._ensure({(1, True, 0, False)})
        self.reset()
        T, H = len(seq), self.cfg.hidden
        hid = torch.empty(T, H, dtype=BF16, device=self.dev)
        lg = torch.empty(T, self.cfg.vocab, dtype=BF16, device=self.dev)
        self.ctl[self.MODE].fill_(0)
        buf = torch.full((NMAX + 1,), -1, dtype=I32)
        for t in range(T):
            buf.fill_(-1)
            buf[0] = seq[t]
            if t + 1 < T:
                buf[1] = seq[t + 1]
            self.in_tok.copy_(buf)
            self.graph(1, True, 0).replay()
            hid[t].copy_(self.hid[0])
            lg[t].copy_(self.logits[0])
        torch.cuda.synchronize()
        return hid, lg
