"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own Python modules
(`qengine.reference`, `qengine.quant` from a checkout of manaspros/qengine) on CPU.

    python tests/golden/make_golden.py --reference /path/to/qengine

The reference checkout is only needed to (re)generate; the tests read the committed files.
Inputs are the seeded tiny hybrid model of qengine_b200.synth (4 layers, hidden 512, vocab 4096,
W4 codes uniform, scales |N(0,1)| * 0.01) and seeded matrices for the packer. Everything runs
with the reference's fake-quant linear (tests/test_27b_w4.py:70-71 of the reference).

Files written (torch.save, a few hundred KB in total):
  quant.pt    reference quantize_w4 / quantize_w4_gate_up / dequantize_w4 on seeded matrices
  ops.pt      rmsnorm1p, rmsnorm_gated, rope, deltanet_core, attention on seeded inputs
  decode.pt   decode_step logits + hidden for 12 teacher-forced tokens, mtp_step rows
  greedy.pt   32-token prompt, 64 greedy tokens (reference decode loop)
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

BF = torch.bfloat16


def fq_lin(x, w):
    return torch.nn.functional.linear(x.float(), w.float()).to(BF)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of manaspros/qengine")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "python"))
    from qengine import quant as RQ
    from qengine import reference as R

    from qengine_b200 import synth
    from oracle.convert import dense_model, reference_named

    torch.manual_seed(0)
    torch.set_num_threads(1)

    # ---- quant.pt --------------------------------------------------------------------------
    g = torch.Generator().manual_seed(11)
    Wm = (torch.randn(37, 300, generator=g) * 0.02).to(BF)
    Wm[2, :128] = 0          # an all-zero group
    Wm[3, 5] = 50.0          # an outlier
    Wg = (torch.randn(21, 200, generator=g) * 0.02).to(BF)
    Wu = (torch.randn(21, 200, generator=g) * 0.02).to(BF)
    p, pg = RQ.quantize_w4(Wm), RQ.quantize_w4_gate_up(Wg, Wu)
    dg, du = RQ.dequantize_w4(pg)
    torch.save({"W": Wm, "qw": p.qw, "scales": p.scales, "deq": RQ.dequantize_w4(p),
                "Wg": Wg, "Wu": Wu, "gu_qw": pg.qw, "gu_scales": pg.scales, "gu_deq_g": dg, "gu_deq_u": du},
               HERE / "quant.pt")

    # ---- model ------------------------------------------------------------------------------
    cfg = synth.tiny_config()
    Wp = synth.build_model(cfg, seed=7, device="cpu", scale_std=0.01)
    D = dense_model(Wp)
    W = reference_named(D, cfg)
    rcfg = R.Config(hidden=cfg.hidden, layers=cfg.layers, inter=cfg.inter, vocab=cfg.vocab, eps=cfg.eps,
                    layer_types=cfg.layer_types, hq=cfg.hq, hkv=cfg.hkv, head_dim=cfg.head_dim,
                    rope_theta=cfg.rope_theta, rotary_dim=cfg.rotary_dim, hk=cfg.hk, hv=cfg.hv, dk=cfg.dk,
                    dv=cfg.dv, conv_k=cfg.conv_k, tied=False, mtp_layers=1)

    # ---- ops.pt -----------------------------------------------------------------------------
    g = torch.Generator().manual_seed(12)
    ops = {}
    x = (torch.randn(3, cfg.hidden, generator=g) * 2).to(BF)
    w = (torch.randn(cfg.hidden, generator=g) * 0.3).to(BF)
    ops["rms_x"], ops["rms_w"], ops["rms_y"] = x, w, R.rmsnorm1p(x, w, cfg.eps)
    xo = torch.randn(cfg.hv, cfg.dv, generator=g).to(BF)
    zz = torch.randn(cfg.hv, cfg.dv, generator=g).to(BF)
    nw = (1 + 0.2 * torch.randn(cfg.dv, generator=g)).to(BF)
    ops["gn_x"], ops["gn_z"], ops["gn_w"], ops["gn_y"] = xo, zz, nw, R.rmsnorm_gated(xo, zz, nw, cfg.eps)
    ops["rope"] = {}
    for pos in (0, 1, 5, 127, 2047, 32768):
        c, s = R.rope_cos_sin(pos, rcfg, "cpu")
        ops["rope"][pos] = (c, s)
    # DeltaNet core over 6 tokens of layer 0 (state carried), incl. the softplus threshold branch
    L0 = "layers.0.linear_attn."
    conv = torch.zeros(cfg.conv_dim, cfg.conv_k - 1, dtype=BF)
    S = torch.zeros(cfg.hv, cfg.dk, cfg.dv)
    rows, outs = [], []
    for t in range(6):
        qkv = (torch.randn(cfg.conv_dim, generator=g) * 2).to(BF)
        z = torch.randn(cfg.value_dim, generator=g).to(BF)
        b = (torch.randn(cfg.hv, generator=g) * 2).to(BF)
        aa = (torch.randn(cfg.hv, generator=g) * 3).to(BF)
        if t == 3:
            aa[0] = 30.0
        rows.append((qkv, z, b, aa))
        outs.append(R.deltanet_core(qkv, z, b, aa, W, L0, conv, S, rcfg))
    ops["gdn_rows"], ops["gdn_out"], ops["gdn_S"], ops["gdn_conv"] = rows, outs, S.clone(), conv.clone()
    # attention: 5 positions of layer 3
    L3 = "layers.3.self_attn."
    kc = torch.zeros(cfg.hkv, 16, cfg.head_dim, dtype=BF)
    vc = torch.zeros_like(kc)
    arows, aouts, aq = [], [], []
    for pos in range(5):
        qg = (torch.randn(cfg.hq * 2 * cfg.head_dim, generator=g) * 3).to(BF)
        k = (torch.randn(cfg.hkv * cfg.head_dim, generator=g) * 3).to(BF)
        v = torch.randn(cfg.hkv * cfg.head_dim, generator=g).to(BF)
        q, gate, kk, vv = R.attention_qkv_from_proj(qg, k, v, W, L3, pos, rcfg)
        kc[:, pos], vc[:, pos] = kk, vv
        arows.append((qg, k, v))
        aq.append(q.clone())
        aouts.append(R.attention_core(q, gate, kc, vc, pos + 1, rcfg))
    ops["attn_rows"], ops["attn_q"], ops["attn_out"] = arows, aq, aouts
    ops["attn_kc"], ops["attn_vc"] = kc.clone(), vc.clone()
    torch.save(ops, HERE / "ops.pt")

    # ---- decode.pt: teacher-forced tokens + MTP rows -----------------------------------------
    ids = synth.prompt_ids(12, cfg.vocab, seed=99)
    st = R.State(rcfg, 64, device="cpu")
    mst = R.MTPState(rcfg, 64, device="cpu")
    logits, hidden, mlogits, mhidden = [], [], [], []
    for t, tok in enumerate(ids):
        lg, hf = R.decode_step(W, st, tok, rcfg, lin=fq_lin, return_hidden=True)
        logits.append(lg)
        hidden.append(hf)
        nxt = ids[t + 1] if t + 1 < len(ids) else int(lg.float().argmax())
        ml, mh = R.mtp_step(W, mst, hf, nxt, t, rcfg, lin=fq_lin)
        mlogits.append(ml)
        mhidden.append(mh)
    torch.save({"ids": ids, "logits": torch.stack(logits), "hidden": torch.stack(hidden),
                "mtp_logits": torch.stack(mlogits), "mtp_hidden": torch.stack(mhidden)}, HERE / "decode.pt")

    # ---- greedy.pt: the CPU reference run of the tiny configuration --------------------------
    prompt = synth.prompt_ids(32, cfg.vocab, seed=1234)
    st = R.State(rcfg, 128, device="cpu")
    for t in prompt[:-1]:
        R.decode_step(W, st, t, rcfg, lin=fq_lin)
    tok, gen = prompt[-1], []
    for _ in range(64):
        tok = int(R.decode_step(W, st, tok, rcfg, lin=fq_lin).float().argmax())
        gen.append(tok)
    torch.save({"prompt": prompt, "tokens": gen, "model_seed": 7, "scale_std": 0.01}, HERE / "greedy.pt")
    print("golden vectors written to", HERE)
    print("distinct greedy tokens:", len(set(gen)))


if __name__ == "__main__":
    main()
