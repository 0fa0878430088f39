"""Pin the CPU oracle (oracle/) and the host-side packer (qengine_b200.quant) against golden vectors
produced by the reference's own Python modules (tests/golden/make_golden.py). CPU only."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import model as OM
from oracle import spec as OS
from oracle import w4 as OW
from qengine_b200 import quant as Q
from qengine_b200 import synth
from util import cosine, dense_model, oracle_config

G = Path(__file__).resolve().parent / "golden"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def tiny():
    cfg = synth.tiny_config()
    Wp = synth.build_model(cfg, seed=7, device="cpu", scale_std=0.01)
    return cfg, Wp, dense_model(Wp), oracle_config(cfg)


# ------------------------------------------------------------------------------ wire format
def test_oracle_packer_matches_reference_bits():
    g = torch.load(G / "quant.pt")
    p = OW.quantize_w4(g["W"].float().numpy())
    assert np.array_equal(p["qw"], g["qw"].numpy())
    assert np.array_equal(p["scales"].view(np.uint16), g["scales"].view(torch.int16).numpy().view(np.uint16))
    deq = OW.dequantize(p["qw"], p["scales"], p["M"], p["K"])
    assert np.array_equal(deq, g["deq"].numpy())
    pg = OW.quantize_w4_gate_up(g["Wg"].float().numpy(), g["Wu"].float().numpy())
    assert np.array_equal(pg["qw"], g["gu_qw"].numpy())
    dg, du = OW.dequantize(pg["qw"], pg["scales"], pg["M"], pg["K"], True)
    assert np.array_equal(dg, g["gu_deq_g"].numpy()) and np.array_equal(du, g["gu_deq_u"].numpy())


def test_product_packer_matches_reference_bits():
    g = torch.load(G / "quant.pt")
    p = Q.quantize_w4(g["W"])
    assert torch.equal(p.qw, g["qw"]) and torch.equal(p.scales, g["scales"])
    assert torch.equal(Q.dequantize_w4(p), g["deq"])
    pg = Q.quantize_w4_gate_up(g["Wg"], g["Wu"])
    assert torch.equal(pg.qw, g["gu_qw"]) and torch.equal(pg.scales, g["gu_scales"])
    dg, du = Q.dequantize_w4(pg)
    assert torch.equal(dg, g["gu_deq_g"]) and torch.equal(du, g["gu_deq_u"])
    codes, sc = Q.unpack_codes(p)
    again = Q.pack_codes(codes, sc, p.M, p.K)
    assert torch.equal(again.qw, p.qw) and torch.equal(again.scales, p.scales)


def test_layout_against_bit_level_definition():
    """Every nibble of a small pack checked against the layout rule, written out longhand."""
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 16, size=(32, 256), dtype=np.uint8)
    scales = (np.abs(rng.standard_normal((32, 2))) * 0.01).astype(np.float16)
    qw, sc = OW.pack(codes, scales)
    for T in range(2):
        for c in range(4):
            for lane in range(32):
                r, t = lane // 4, lane % 4
                for s in range(4):
                    word = int(qw[T, c, lane, s]) & 0xFFFFFFFF
                    for j in range(8):
                        row = 16 * T + r + 8 * (j & 1)
                        k = 64 * c + 16 * t + 4 * s + 2 * ((j >> 1) & 1) + (j >> 2)
                        assert (word >> (4 * j)) & 15 == codes[row, k]
    assert np.array_equal(sc[1, 0], scales[16:32, 0])
    p = Q.pack_codes(torch.from_numpy(codes), torch.from_numpy(scales), 32, 256)
    assert np.array_equal(p.qw.numpy(), qw) and np.array_equal(p.scales.numpy(), sc)


# ------------------------------------------------------------------------------ elementary ops
def test_oracle_ops_match_reference(tiny):
    cfg, _, D, ocfg = tiny
    g = torch.load(G / "ops.pt")
    assert torch.equal(OM.rmsnorm1p(g["rms_x"], g["rms_w"], cfg.eps), g["rms_y"])
    assert torch.equal(OM.rmsnorm_gated(g["gn_x"], g["gn_z"], g["gn_w"], cfg.eps), g["gn_y"])
    for pos, (c, s) in g["rope"].items():
        oc, osn = OM.rope_cos_sin(pos, ocfg)
        assert torch.equal(oc, c) and torch.equal(osn, s)
    # DeltaNet core, state carried over 6 tokens
    L = D["layers"][0]
    conv = torch.zeros(cfg.conv_dim, cfg.conv_k - 1, dtype=BF)
    S = torch.zeros(cfg.hv, cfg.dk, cfg.dv)
    for (qkv, z, b, a), want in zip(g["gdn_rows"], g["gdn_out"]):
        assert torch.equal(OM.deltanet_core(qkv, z, b, a, L, conv, S, ocfg), want)
    assert torch.equal(S, g["gdn_S"]) and torch.equal(conv, g["gdn_conv"])
    # attention, 5 positions
    L = D["layers"][3]
    kc = torch.zeros(cfg.hkv, 16, cfg.head_dim, dtype=BF)
    vc = torch.zeros_like(kc)
    for pos, ((qg, k, v), wq, wo) in enumerate(zip(g["attn_rows"], g["attn_q"], g["attn_out"])):
        q, gate, kk, vv = OM.attention_qkv(qg, k, v, L, pos, ocfg)
        kc[:, pos], vc[:, pos] = kk, vv
        assert torch.equal(q, wq)
        assert torch.equal(OM.attention_core(q, gate, kc, vc, pos + 1, ocfg), wo)
    assert torch.equal(kc, g["attn_kc"]) and torch.equal(vc, g["attn_vc"])


# ------------------------------------------------------------------------------ whole model
def test_oracle_decode_and_mtp_match_reference(tiny):
    cfg, _, D, ocfg = tiny
    g = torch.load(G / "decode.pt")
    st = OM.State(ocfg, 64)
    for t, tok in enumerate(g["ids"]):
        lg, hf = OM.decode_step(D, st, tok, ocfg)
        assert cosine(lg, g["logits"][t]) > 0.99999
        assert (lg.float() - g["logits"][t].float()).abs().max() <= 0.0625
        assert int(lg.float().argmax()) == int(g["logits"][t].float().argmax())
        assert cosine(hf, g["hidden"][t]) > 0.99999
        nxt = g["ids"][t + 1] if t + 1 < len(g["ids"]) else int(lg.float().argmax())
        ml, mh = OM.mtp_step(D, st, g["hidden"][t], nxt, t, ocfg)
        assert cosine(ml, g["mtp_logits"][t]) > 0.99999
        assert cosine(mh, g["mtp_hidden"][t]) > 0.99999


def test_cpu_reference_run_plain_equals_golden_and_spec_equals_plain(tiny):
    """The CPU-runnable configuration: 32-token prompt, 64 greedy tokens; the oracle's plain greedy
    equals the reference's decode loop, and MTP k = 4 speculative output equals plain greedy."""
    cfg, _, D, ocfg = tiny
    g = torch.load(G / "greedy.pt")
    dec = OS.Decoder(D, ocfg, max_len=128)
    plain = dec.generate(g["prompt"], 64)
    assert plain == g["tokens"]
    spec = dec.generate_spec(g["prompt"], 64, 4)
    assert spec == plain
    assert dec.ctl[4] > 0 and sum(dec.ctl[16:21]) == dec.ctl[4]


@pytest.mark.parametrize("a", [0, 1, 2, 3, 4])
def test_forced_acceptance_lengths_on_cpu(tiny, a):
    cfg, _, D, ocfg = tiny
    g = torch.load(G / "greedy.pt")
    truth = g["prompt"] + g["tokens"]
    dec = OS.Decoder(D, ocfg, max_len=128)
    out = dec.generate_spec(g["prompt"], 40, 4, override=OS.forced_acceptance(truth, a, cfg.vocab))
    assert out == g["tokens"][:40]
    # every verify cycle whose window lies inside the known continuation accepted exactly `a`
    ms = [t["m"] for t in dec.trace if t["n"] == 5 and t["pos"] + 5 < len(truth)]
    assert ms and all(m == a for m in ms)


# ------------------------------------------------------------------------------ bookkeeping
def test_accept_commit_known_answers():
    """Hand-worked cases of the accept / commit rules (csrc/basic.cu:256-291 of the reference)."""
    ctl = [10, 0, 1, 0] + [0] * 28
    in_tok = [5, 7, 8, 9, 1, 0, 0, 0, 0]
    am = [7, 8, 3, 4, 6, 0, 0, 0]
    nxt, log = [0] * 8, [0] * 64
    OS.accept(in_tok, am, 5, ctl, nxt, log)
    assert ctl[3] == 2 and log[11:14] == [7, 8, 3] and log[14] == 0
    assert (ctl[4], ctl[5], ctl[18]) == (1, 2, 1) and nxt[:5] == am[:5]
    OS.commit(ctl, in_tok, am, [21, 22, 23, 24], 4)
    assert ctl[0] == 13 and ctl[1] == 3 and in_tok[:5] == [3, 21, 22, 23, 24]
    assert OS.mtp_position(ctl, -1) == 13 and OS.mtp_position(ctl, 1) == 13 + 2 + 1 + 1
    # all drafts accepted; log writes clipped at max_len
    ctl = [60, 0, 1, 0] + [0] * 28
    in_tok, am, log = [1, 2, 3, 0, 0, 0, 0, 0, 0], [2, 3, 9, 0, 0, 0, 0, 0], [0] * 63
    OS.accept(in_tok, am, 3, ctl, nxt, log)
    assert ctl[3] == 2 and log[61:63] == [2, 3] and ctl[18] == 1
    # prefill, more prompt follows: nothing logged, next_tok from the prompt
    ctl = [0, 0, 0, 0] + [0] * 28
    in_tok, am, log = [4, 5, 6, 7, -1, -1, -1, -1, -1], [9, 9, 9, 0, 0, 0, 0, 0], [0] * 64
    OS.accept(in_tok, am, 3, ctl, nxt, log)
    assert ctl[3] == 2 and nxt[:3] == [5, 6, 7] and log == [0] * 64 and ctl[4] == 0
    # prefill, last chunk: the last row's argmax is the first generated token
    in_tok = [4, 5, 6, -1, -1, -1, -1, -1, -1]
    OS.accept(in_tok, am, 3, ctl, nxt, log)
    assert nxt[:3] == [5, 6, 9] and log[3] == 9
