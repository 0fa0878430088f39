"""Oracle (test infrastructure): the speculative decode cycle on CPU.

The reference has no CPU version of this part: acceptance, commit and MTP row selection exist
only as CUDA kernels (csrc/basic.cu:241-307) driven by the engine's pass structure
(python/qengine/engine.py:468-520 `_main` / `_mtp` / `_pass`, 558-573 `prefill`, 575-637
`generate` / `generate_spec`). This file restates them with Python integers and the CPU model of
oracle/model.py. Rows of a verify pass are run one after another through the same one-token
step as plain decoding, and rejected rows are undone by restoring a snapshot of the recurrent
state, so "speculative == plain" holds here by construction: what this oracle pins is the
integer bookkeeping (m, positions, logged tokens, next inputs, statistics) and the MTP input
conventions, which the CUDA path must reproduce bit for bit.

ctl layout (csrc/basic.cu:241-247): [0] pos, [1] pending, [2] mode (0 prefill, 1 verify),
[3] m, [4] cycles, [5] accepted drafts, [16 + m] histogram.
"""
from __future__ import annotations

import torch

from . import model as M

NMAX = 8  # rows per pass (python/qengine/engine.py:46)


def accept(in_tok, am, n, ctl, next_tok, log):
    """accept_kernel (csrc/basic.cu:256-279) on Python lists, in place."""
    P, mode = ctl[0], ctl[2]
    max_len = len(log)
    m = n - 1
    if mode == 1:
        m = 0
        while m < n - 1 and in_tok[m + 1] == am[m]:
            m += 1
        for i in range(m + 1):
            if P + 1 + i < max_len:
                log[P + 1 + i] = am[i]
        ctl[4] += 1
        ctl[5] += m
        ctl[16 + m] += 1
    elif in_tok[n] < 0 and P + n < max_len:
        log[P + n] = am[n - 1]
    for r in range(n):
        if mode == 1:
            next_tok[r] = am[r]
        elif r + 1 < n:
            next_tok[r] = in_tok[r + 1]
        else:
            next_tok[r] = in_tok[n] if in_tok[n] >= 0 else am[n - 1]
    ctl[3] = m


def commit(ctl, in_tok, am, drafts, k):
    """commit_kernel (csrc/basic.cu:283-291)."""
    m = ctl[3]
    ctl[0] += m + 1
    ctl[1] = m + 1
    in_tok[0] = am[m]
    for j in range(k):
        in_tok[1 + j] = drafts[j]


def mtp_position(ctl, off):
    """mtp_select_kernel's position rule (csrc/basic.cu:295-301)."""
    return ctl[0] if off < 0 else ctl[0] + ctl[3] + 1 + off


class Decoder:
    """Engine-shaped driver around the CPU model: same buffers and pass order as
    python/qengine/engine.py, one row at a time."""

    def __init__(self, W, cfg: M.Config, max_len: int, fused_swiglu: bool = False):
        self.W, self.cfg, self.max_len, self.fused = W, cfg, max_len, fused_swiglu
        self.has_mtp = "mtp" in W and W["mtp"] is not None
        self.reset()

    def reset(self):
        self.st = M.State(self.cfg, self.max_len, with_mtp=self.has_mtp)
        self.ctl = [0] * 32
        self.in_tok = [0] * (NMAX + 1)
        self.am = [0] * NMAX
        self.next_tok = [0] * NMAX
        self.drafts = [0] * NMAX
        self.mtp_am = [0] * NMAX
        self.log = [0] * self.max_len
        self.trace = []  # per pass: dict(n, pos, in_tok, am, m, drafts)
        self.last_logits = None

    # one pass = Engine._pass (engine.py:498-520)
    def run_pass(self, n, mtp_rows, k, override=None):
        ctl, st = self.ctl, self.st
        pos = ctl[0]
        if override is not None and ctl[2] == 1:
            override(self, pos, n)
        assert st.pos == pos, (st.pos, pos)
        snaps, hids, logits = [], [], []
        for r in range(n):  # _main: every row through the one-token step
            lg, hf = M.decode_step(self.W, st, self.in_tok[r], self.cfg, self.fused)
            snaps.append(st.snapshot())
            hids.append(hf)
            logits.append(lg)
            self.am[r] = int(torch.argmax(lg.float()))
        self.last_logits = logits
        accept(self.in_tok, self.am, n, ctl, self.next_tok, self.log)
        m = ctl[3]
        st.restore(snaps[m])  # rollback of the rejected rows (lazy replay on the GPU)
        if mtp_rows:
            mpos = mtp_position(ctl, -1)
            mout = []
            for r in range(n):  # _mtp over the n rows, positions mpos + r
                lg, hn = M.mtp_step(self.W, st, hids[r], self.next_tok[r], mpos + r, self.cfg, self.fused)
                self.mtp_am[r] = int(torch.argmax(lg.float()))
                mout.append(hn)
            if k > 0:
                self.drafts[0] = self.mtp_am[m]
                chain = mout[m]
            for j in range(1, k):  # chained drafts at positions pos + m + j
                mpos = mtp_position(ctl, j - 1)
                lg, chain = M.mtp_step(self.W, st, chain, self.drafts[j - 1], mpos, self.cfg, self.fused)
                self.drafts[j] = int(torch.argmax(lg.float()))
        self.trace.append({"n": n, "pos": pos, "in_tok": list(self.in_tok[:n + 1]), "am": list(self.am[:n]),
                           "m": m, "drafts": list(self.drafts[:k])})
        commit(ctl, self.in_tok, self.am, self.drafts, k)

    def prefill(self, prompt, mtp=False, k=0, chunk=NMAX):
        """engine.py:558-573"""
        chunks = [prompt[i:i + chunk] for i in range(0, len(prompt), chunk)]
        self.ctl[2] = 0
        for ci, c in enumerate(chunks):
            last = ci == len(chunks) - 1
            buf = [-1] * (NMAX + 1)
            buf[:len(c)] = c
            if not last:
                buf[len(c)] = chunks[ci + 1][0]
            self.in_tok = buf
            self.run_pass(len(c), mtp, k if last else 0)
        self.ctl[2] = 1

    def generate(self, prompt, n_new, chunk=NMAX):
        """Plain greedy (engine.py:575-597)."""
        P = len(prompt)
        assert P + n_new + 1 <= self.max_len
        self.reset()
        self.prefill(prompt, chunk=chunk)
        for _ in range(n_new - 1):
            self.run_pass(1, False, 0)
        return self.log[P:P + n_new]

    def generate_spec(self, prompt, n_new, k, chunk=NMAX, override=None):
        """Speculative greedy with k chained MTP drafts (engine.py:599-637). `override(dec, pos, n)`
        may rewrite dec.in_tok[1:n] before a verify pass (forced acceptance lengths)."""
        assert self.has_mtp and 1 <= k <= NMAX - 1
        P = len(prompt)
        assert P + n_new + 2 * NMAX + 2 <= self.max_len
        self.reset()
        self.prefill(prompt, mtp=True, k=k, chunk=chunk)
        self.ctl[4] = self.ctl[5] = 0
        for i in range(16, 32):
            self.ctl[i] = 0
        target = P + n_new - 1
        while self.ctl[0] < target:
            self.run_pass(k + 1, True, k, override)
        return self.log[P:P + n_new]


def forced_acceptance(truth, a, vocab):
    """Override hook: make exactly `a` drafts match. truth[p] = the plain-greedy token at
    position p. Draft j (input row j + 1, position pos + 1 + j) becomes the true token for j < a
    and (true + 1) mod vocab otherwise."""
    def hook(dec, pos, n):
        for j in range(n - 1):
            p = pos + 1 + j
            t = truth[p] if p < len(truth) else 0
            dec.in_tok[1 + j] = t if j < a else (t + 1) % vocab
    return hook
