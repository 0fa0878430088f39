"""End-to-end decode engine on the GPU against the CPU oracle, on the seeded tiny hybrid model
(4 layers: 3 Gated-DeltaNet + 1 gated attention, hidden 512, vocab 4096, 1 MTP layer).

Criteria (from the reference's real-weight tests restated on synthetic weights):
  - teacher-forced logits vs the oracle: cosine >= 0.9999 per position, max-abs reported,
    top-1 agreement >= 97 %;
  - MTP-row logits vs the oracle's mtp_step: cosine >= 0.9999;
  - chunked prefill == one-row-at-a-time, bit for bit;
  - speculative output token-identical to the engine's own plain greedy output for k = 1..4, with a
    pruned draft vocabulary, and at forced acceptance lengths 0..4;
  - run-to-run determinism.
"""
from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import model as OM
from util import cosine, dense_model, oracle_config

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def setup():
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    cfg = synth.tiny_config()
    Wp = synth.build_model(cfg, seed=7, device="cpu", scale_std=0.01)
    eng = Engine(cfg, synth.model_to(Wp, "cuda"), max_len=256)
    return cfg, Wp, eng


def test_teacher_forced_logits_vs_oracle(setup):
    cfg, Wp, eng = setup
    D, ocfg = dense_model(Wp), oracle_config(cfg)
    g = torch.load(G / "greedy.pt")
    seq = (g["prompt"] + g["tokens"])[:48]
    e_logits = eng.sequence_logits(seq).float().cpu()
    st = OM.State(ocfg, 64)
    worst_cos, worst_abs, agree = 1.0, 0.0, 0
    for t, tok in enumerate(seq):
        lg, _ = OM.decode_step(D, st, tok, ocfg, fused_swiglu=True)
        worst_cos = min(worst_cos, cosine(e_logits[t], lg))
        worst_abs = max(worst_abs, float((e_logits[t] - lg.float()).abs().max()))
        agree += int(e_logits[t].argmax()) == int(lg.float().argmax())
    print(f"\nlogits vs oracle over {len(seq)} positions: min cosine {worst_cos:.6f}, max|d| {worst_abs:.4f}, "
          f"top-1 agreement {agree}/{len(seq)}")
    assert worst_cos >= 0.9999
    assert agree / len(seq) >= 0.97


def test_teacher_forced_logits_vs_reference_golden(setup):
    """Same check against logits stored from the reference's own torch path (its SwiGLU rounds
    gate, up and silu to bf16, the engine's epilogue does not: a known, accepted difference)."""
    _, _, eng = setup
    g = torch.load(G / "decode.pt")
    e_logits = eng.sequence_logits(g["ids"]).float().cpu()
    cs = [cosine(e_logits[t], g["logits"][t]) for t in range(len(g["ids"]))]
    agree = sum(int(e_logits[t].argmax()) == int(g["logits"][t].float().argmax()) for t in range(len(g["ids"])))
    print(f"\nvs reference golden: min cosine {min(cs):.6f}, top-1 {agree}/{len(cs)}")
    # 0.9999 holds against the oracle with the kernel's epilogue definition (test above); against
    # the bf16-rounded SwiGLU of the torch path the floor is one notch lower on this tiny model.
    assert min(cs) >= 0.9998 and agree >= len(cs) - 1


def test_mtp_rows_vs_oracle(setup):
    cfg, Wp, eng = setup
    D, ocfg = dense_model(Wp), oracle_config(cfg)
    g = torch.load(G / "decode.pt")
    ids = g["ids"]
    hid, lg = eng.mtp_rows_logits(ids)
    hid, lg = hid.cpu(), lg.float().cpu()
    st = OM.State(ocfg, 64)
    for t in range(len(ids) - 1):  # the last row's next token is the engine's own argmax
        ml, _ = OM.mtp_step(D, st, hid[t], ids[t + 1], t, ocfg, fused_swiglu=True)
        assert cosine(lg[t], ml) >= 0.9999, t


def test_chunked_prefill_equals_one_by_one(setup):
    _, _, eng = setup
    g = torch.load(G / "greedy.pt")
    seq = g["prompt"][:21]
    a = eng.sequence_logits(seq, chunk=8)
    b = eng.sequence_logits(seq, chunk=1)
    c = eng.sequence_logits(seq, chunk=5)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert torch.equal(a.view(torch.int16), c.view(torch.int16))


@pytest.mark.parametrize("k", [1, 2, 3, 4])
def test_spec_equals_plain(setup, k):
    _, _, eng = setup
    g = torch.load(G / "greedy.pt")
    plain = eng.generate(g["prompt"], 160)
    spec, _, _, st = eng.generate_spec(g["prompt"], 160, k, timing=True)
    first = next((i for i, (a, b) in enumerate(zip(spec, plain)) if a != b), None)
    print(f"\nk={k}: accept rate {st['accept_rate']:.3f}, tokens/cycle {st['tokens_per_cycle']:.2f}, hist {st['hist']}")
    assert first is None, f"first difference at {first}"
    assert sum(st["hist"]) == st["cycles"]


@pytest.mark.parametrize("a", [0, 1, 2, 3, 4])
def test_forced_acceptance_lengths(setup, a):
    _, _, eng = setup
    g = torch.load(G / "greedy.pt")
    n_new = 120
    plain = eng.generate(g["prompt"], n_new + 16)
    truth = g["prompt"] + plain
    spec, _, _, st = eng.generate_spec(g["prompt"], n_new, 4, timing=True, force_accept=a, truth=truth)
    assert spec == plain[:n_new]
    assert st["hist"][a] == st["cycles"] and st["accepted"] == a * st["cycles"]
    assert abs(st["tokens_per_cycle"] - (a + 1)) < 1e-9


def test_draft_vocab_and_determinism(setup):
    cfg, Wp, _ = setup
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    g = torch.load(G / "greedy.pt")
    eng = Engine(cfg, synth.model_to(Wp, "cuda"), max_len=256, draft_vocab=1024)
    plain = eng.generate(g["prompt"], 100)
    assert eng.generate_spec(g["prompt"], 100, 4) == plain
    runs = [eng.generate(g["prompt"], 100) for _ in range(3)]
    assert all(r == plain for r in runs)


def test_oracle_greedy_agreement_reported(setup):
    """How far the engine's greedy continuation follows the reference's CPU continuation (fp32
    summation order differs, and near-ties in random-weight logits can flip): reported, and the
    first 8 tokens must agree."""
    _, _, eng = setup
    g = torch.load(G / "greedy.pt")
    gen = eng.generate(g["prompt"], 64)
    same = next((i for i, (a, b) in enumerate(zip(gen, g["tokens"])) if a != b), 64)
    print(f"\nengine greedy == reference CPU greedy for the first {same} of 64 tokens")
    assert same >= 8


def test_prefilled_context_spec_equals_plain(setup):
    """Long-cache harness: positions [0, 300) hold seeded K/V, the sequence starts at 300; the
    speculative output must still equal the plain output token for token (rollback indices,
    forced drafts and the log are all in absolute positions)."""
    from qengine_b200.engine import Engine
    from qengine_b200 import synth
    cfg, Wp, _ = setup
    eng = Engine(cfg, synth.model_to(Wp, "cuda"), max_len=512, attn_splits=8)
    eng.set_context(300)
    g = torch.load(G / "greedy.pt")
    plain = eng.generate(g["prompt"], 40)
    assert int(eng.ctl[eng.POS]) == 300 + 32 + 39
    assert eng.generate_spec(g["prompt"], 40, 3) == plain
    for a in (0, 2, 4):
        assert eng.generate_spec(g["prompt"], 40, 4, force_accept=a, truth=g["prompt"] + plain + [0] * 16) == plain
    base = Engine(cfg, synth.model_to(Wp, "cuda"), max_len=512, attn_splits=8).generate(g["prompt"], 40)
    assert base != plain  # the context is really attended to


# ---------------------------------------------------------------------------------------------
# The same checks at the 27B width (hidden 5120, head dim 256, DeltaNet d = 128, 48 value heads,
# fused projection offsets 16,480 / 14,336, 6 query heads per KV head): 3 DeltaNet layers + 1
# attention layer + the MTP layer, vocabulary cut to 16,384 rows so that the CPU oracle stays cheap.
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def wide():
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    from qengine_b200.quant import dequantize_w4
    cfg = synth.qwen27b_config(layers=4)
    cfg.vocab = 16384
    W = synth.build_model(cfg, seed=11, device="cuda", scale_std=0.01)
    eng = Engine(cfg, W, max_len=160)

    # dense fp32 weights for the oracle; dequantised on the GPU by the product dequantiser, which
    # test_w4_gpu.py::test_product_dequantiser_matches_oracle_dequantiser pins to the oracle's
    def dense(L):
        D = {k: v.cpu() for k, v in L.items() if isinstance(v, torch.Tensor)}
        D["type"] = L["type"]
        for k in ("in_proj", "out", "down", "fc"):
            if k in L:
                D[k] = dequantize_w4(L[k]).cpu()
        g, u = dequantize_w4(L["gate_up"])
        D["gate"], D["up"] = g.cpu(), u.cpu()
        return D

    D = {"embed": W["embed"].cpu(), "final_norm": W["final_norm"].cpu(), "lm_head": dequantize_w4(W["lm_head"]).cpu(),
         "layers": [dense(L) for L in W["layers"]], "mtp": dense(W["mtp"])}
    return cfg, D, eng


def test_wide_teacher_forced_logits_vs_oracle(wide):
    from qengine_b200 import synth
    cfg, D, eng = wide
    ocfg = oracle_config(cfg)
    seq = synth.prompt_ids(12, cfg.vocab, seed=21)
    e_logits = eng.sequence_logits(seq, chunk=5).float().cpu()   # passes of 5, 5 and 2 rows
    hid, m_logits = eng.mtp_rows_logits(seq[:6])
    st = OM.State(ocfg, 32)
    worst, worst_abs, agree, worst_m = 1.0, 0.0, 0, 1.0
    for t, tok in enumerate(seq):
        lg, hf = OM.decode_step(D, st, tok, ocfg, fused_swiglu=True)
        worst = min(worst, cosine(e_logits[t], lg))
        worst_abs = max(worst_abs, float((e_logits[t] - lg.float()).abs().max()))
        agree += int(e_logits[t].argmax()) == int(lg.float().argmax())
        if t < 5:
            ml, _ = OM.mtp_step(D, st, hid[t].cpu(), seq[t + 1], t, ocfg, fused_swiglu=True)
            worst_m = min(worst_m, cosine(m_logits[t].float().cpu(), ml))
    print(f"\n27B width, 4 layers: min cosine {worst:.6f} (MTP rows {worst_m:.6f}), max|d| {worst_abs:.4f}, "
          f"top-1 {agree}/{len(seq)}")
    assert worst >= 0.9999 and worst_m >= 0.9999 and agree >= len(seq) - 1


def test_wide_spec_equals_plain_and_chunking(wide):
    from qengine_b200 import synth
    cfg, _, eng = wide
    prompt = synth.prompt_ids(19, cfg.vocab, seed=22)
    plain = eng.generate(prompt, 40)
    for k in (1, 4):
        assert eng.generate_spec(prompt, 40, k) == plain, k
    for a in (0, 3, 4):
        assert eng.generate_spec(prompt, 40, 4, force_accept=a, truth=prompt + plain + [0] * 16) == plain, a
    a8 = eng.sequence_logits(prompt, chunk=8)
    a1 = eng.sequence_logits(prompt, chunk=1)
    assert torch.equal(a8.view(torch.int16), a1.view(torch.int16))


def test_engine_without_fused_norms_and_with_chains_agree(setup):
    """The three ways to run the same pass: norm fused into the GEMV launch (default), every norm
    as its own kernel, and consecutive GEMVs as one cooperative chain. Chains are bit-identical to
    the default; the unfused engine differs only by the order of the norm's sum of squares."""
    cfg, Wp, eng = setup
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    g = torch.load(G / "greedy.pt")
    seq = (g["prompt"] + g["tokens"])[:24]
    base = eng.sequence_logits(seq)
    W = synth.model_to(Wp, "cuda")
    chained = Engine(cfg, W, max_len=256, chain=True)
    assert torch.equal(chained.sequence_logits(seq).view(torch.int16), base.view(torch.int16))
    plain = eng.generate(g["prompt"], 60)
    assert chained.generate(g["prompt"], 60) == plain
    assert chained.generate_spec(g["prompt"], 60, 4) == plain
    unfused = Engine(cfg, W, max_len=256, fuse=False)
    lg = unfused.sequence_logits(seq)
    assert min(cosine(lg[t], base[t]) for t in range(len(seq))) >= 0.99999
    assert unfused.generate_spec(g["prompt"], 60, 3) == unfused.generate(g["prompt"], 60)


def _new_engine(cfg, Wp, **kw):
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    return Engine(cfg, synth.model_to(Wp, "cuda"), max_len=256, **kw)


def test_l2_window_around_the_draft_phase_changes_no_token(setup):
    """pin_mtp_l2 re-homes the draft layer's matrices into one arena and runs the draft phase of
    every graph under a persisting access-policy window (reference: python/qengine/engine.py:
    360-381, 502-519). It is a cache policy: tokens must not change, on or off."""
    from qengine_b200 import _C, _w4
    cfg, Wp, base = setup
    prompt = torch.load(G / "greedy.pt")["prompt"]
    plain = base.generate(prompt, 60)
    eng = _new_engine(cfg, Wp)
    names = ("fc", "in_proj", "out")
    before = {n: eng.mtp[n].qw.data_ptr() for n in names}
    eng.pin_mtp_l2(True)
    assert eng.l2_win is not None and eng.l2_win[1] >= sum(eng.mtp[n].nbytes for n in names)
    lo, hi = eng.l2_win[0], eng.l2_win[0] + eng.l2_win[1]
    assert all(lo <= eng.mtp[n].qw.data_ptr() < hi and eng.mtp[n].qw.data_ptr() != before[n] for n in names)
    for k in (1, 4):
        assert eng.generate_spec(prompt, 60, k) == plain, f"window on, k={k}"
    eng.pin_mtp_l2(False)
    assert eng.l2_win is None and not eng.graphs
    assert eng.generate_spec(prompt, 60, 4) == plain
    assert eng.generate(prompt, 60) == plain
    assert _C.attn_error() == 0 and _w4.ring_error() == 0


def test_engine_from_a_cache_directory(setup, tmp_path):
    """Weights written in the reference's cache layout load back into an engine that decodes the
    same tokens (qengine_b200.cache; reference python/qengine/engine.py:215-236)."""
    from qengine_b200 import cache
    from qengine_b200.engine import Engine
    cfg, Wp, base = setup
    prompt = torch.load(G / "greedy.pt")["prompt"]
    model_dir = tmp_path / "tiny-model"
    cache.write_config(model_dir, cfg)
    cache.save_cache(cache.cache_path(tmp_path / "c", "tiny-model"), Wp)
    eng = Engine.from_cache(model_dir, tmp_path / "c", device="cuda", max_len=256)
    assert eng.cfg == cfg
    want = base.generate(prompt, 48)
    assert eng.generate(prompt, 48) == want
    assert eng.generate_spec(prompt, 48, 3) == want


def test_bf16_lm_head_backend(setup):
    """lm_head kept in BF16 while the layers stay W4 (the reference's lm_head="bf16" choice,
    python/qengine/engine.py:195-208): the engine picks the BF16 GEMV for a dense head. With the
    dense head set to the packed head's own dequantised values, logits agree up to the summation
    order and speculative output still equals plain output."""
    from qengine_b200 import quant
    cfg, Wp, base = setup
    prompt = torch.load(G / "greedy.pt")["prompt"]
    Wd = dict(Wp)
    Wd["lm_head"] = quant.dequantize_w4(Wp["lm_head"]).to(torch.bfloat16).contiguous()
    eng = _new_engine(cfg, Wd)
    a = eng.sequence_logits(prompt[:12]).float()
    b = base.sequence_logits(prompt[:12]).float()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
    assert cos.min() > 0.9999, cos.min()
    plain = eng.generate(prompt, 48)
    assert eng.generate_spec(prompt, 48, 4) == plain


def test_norm_weights_too_large_for_fp16_rows_keep_bf16(setup):
    """GEMVs behind an RMSNorm take fp16 rows only while sqrt(H) * |1 + w| fits fp16 for every
    norm weight (Engine._norms_fit_fp16); one outsized weight sends the whole engine back to bf16
    rows, and both engines are self-consistent."""
    cfg, Wp, base = setup
    assert base.f16
    prompt = torch.load(G / "greedy.pt")["prompt"]
    Wb = dict(Wp)
    Wb["final_norm"] = Wp["final_norm"].clone()
    Wb["final_norm"][3] = 5000.0
    eng = _new_engine(cfg, Wb)
    assert not eng.f16
    plain = eng.generate(prompt, 40)
    assert eng.generate_spec(prompt, 40, 4) == plain
    # and the bf16-row engine on the unmodified weights decodes what the fp16-row engine decodes
    import os
    os.environ["QE_F16"] = "0"
    try:
        bf = _new_engine(cfg, Wp)
    finally:
        del os.environ["QE_F16"]
    assert not bf.f16
    assert bf.generate(prompt, 60) == base.generate(prompt, 60)
    a, b = bf.sequence_logits(prompt[:16]), base.sequence_logits(prompt[:16])
    assert torch.equal(a.view(torch.int16), b.view(torch.int16)), "fp16 rows changed logit bits"


# ---------------------------------------------------------------------------------------------
# Prefill in passes of up to 64 rows through the tensor-memory GEMM (Engine.prefill(wide=True); no
# counterpart in the reference, which prefills 8 rows at a time). The GEMM adds the groups of a tile
# in another order than the GEMV, so the state agrees with the 8-row passes to rounding only; what
# must hold exactly is everything downstream of a given prefill: spec == plain, determinism.
# ---------------------------------------------------------------------------------------------
def _prefill_and_snapshot(eng, prompt, wide, mtp=False, k=0):
    head = eng._wide_split(len(prompt), wide)
    eng._need_wide(head, mtp)
    eng._need(eng._prefill_keys(len(prompt), mtp, k, skip=head))
    eng.reset()
    eng.prefill(prompt, mtp=mtp, k=k, wide=wide)
    torch.cuda.synchronize()
    tail = len(prompt) - head if head else (len(prompt) - 1) % 8 + 1
    blocks = eng.layers + ([eng.mtp] if mtp else [])
    P = len(prompt)
    kv = [(L["kc"][:, :P].float().clone(), L["vc"][:, :P].float().clone()) for L in blocks if "kc" in L]
    return eng.logits[:tail].float().clone(), kv, int(eng.ctl[eng.POS].item()), int(eng.log[P].item()), head


@pytest.mark.parametrize("which,P", [("tiny", 33), ("tiny", 100), ("tiny", 137), ("27b", 75)])
def test_prefill_in_64_row_passes_agrees_with_8_row_passes(setup, wide, which, P):
    from qengine_b200 import synth
    cfg, _, eng = setup if which == "tiny" else wide
    prompt = synth.prompt_ids(P, cfg.vocab, seed=31)
    lg8, kv8, pos8, tok8, head8 = _prefill_and_snapshot(eng, prompt, False, mtp=True, k=2)
    lgw, kvw, posw, tokw, headw = _prefill_and_snapshot(eng, prompt, True, mtp=True, k=2)
    assert head8 == 0 and headw == ((P - 1) // 8) * 8 and posw == pos8 == P
    cs = min(cosine(lgw[t].cpu(), lg8[t].cpu()) for t in range(lgw.shape[0]))
    worst = float((lgw - lg8).abs().max())
    kv_err = max(float((a - b).abs().max() / (b.abs().max() + 1e-6)) for x, y in zip(kvw, kv8) for a, b in zip(x, y))
    print(f"\n{which} P={P}: last-pass logits cosine {cs:.7f}, max|d| {worst:.4f}, K/V rel err {kv_err:.2e}, "
          f"first token equal: {tokw == tok8}")
    assert cs >= 0.9999 and kv_err < 2e-2  # (the logits left in the buffer are the draft layer's)


def test_spec_equals_plain_after_a_wide_prefill(setup, wide):
    from qengine_b200 import synth
    for (cfg, _, eng), P, n_new in ((setup, 90, 80), (wide, 70, 40)):
        prompt = synth.prompt_ids(P, cfg.vocab, seed=32)
        plain = eng.generate(prompt, n_new, wide=True)
        assert eng.generate(prompt, n_new, wide=True) == plain  # run to run
        for k in (1, 4):
            assert eng.generate_spec(prompt, n_new, k, wide=True) == plain, (P, k)
        assert ("wide", 64, True) in eng.graphs and ("wide", 64, False) in eng.graphs


def test_wide_prefill_as_the_engines_default(setup):
    """Engine(wide_prefill=True) feeds every long enough prompt in 64-row passes without being asked
    per call; short prompts and wide=False still take the 8-row passes."""
    from qengine_b200 import synth
    from qengine_b200.engine import Engine
    cfg, Wp, eng = setup
    auto = Engine(cfg, synth.model_to(Wp, "cuda"), max_len=256, wide_prefill=True)
    prompt = synth.prompt_ids(80, cfg.vocab, seed=33)
    assert auto._wide_split(80, None) == 72 and auto._wide_split(80, False) == 0 and auto._wide_split(20, None) == 0
    assert auto._wide_blocks(72) == [64, 8] and eng._wide_split(80, None) == 0
    assert auto.generate(prompt, 24) == eng.generate(prompt, 24, wide=True)
    assert ("wide", 64, False) in auto.graphs and ("wide", 8, False) in auto.graphs
    assert auto.generate(prompt, 24, wide=False) == eng.generate(prompt, 24)
