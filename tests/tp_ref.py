"""Tensor-parallel restatement of the CPU oracle's one-token step, for the world_size > 1 tests.

Each rank holds the shard `qengine_b200.tp.shard_model` gives it (dequantised by the oracle) and
runs the oracle's own mixer functions on the local head counts; the matrices split along K
(out / o_proj, down, mtp.fc) produce fp32 partial rows that are gathered and summed in rank order
before the single bf16 rounding, exactly what the engine's exchange + rmsnorm1p_parts does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from oracle import model as OM

BF16 = torch.bfloat16


def reduce_parts(part: torch.Tensor) -> torch.Tensor:
    """Gather every rank's fp32 partial row, sum in ascending rank order, round once."""
    parts = [torch.empty_like(part) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, part.contiguous())
    s = parts[0].clone()
    for p in parts[1:]:
        s += p
    return s.to(BF16)


def tp_layer(h, L, st, key, pos, lc):
    x = OM.rmsnorm1p(h, L["in_norm"], lc.eps)
    pr = OM.lin(x, L["in_proj"])
    if L["type"] == "linear_attention":
        mix = OM.deltanet_core(*OM.split_gdn_proj(pr, lc), L, st.conv[key], st.S[key], lc)
    else:
        qg, k, v = OM.split_attn_proj(pr, lc)
        q, gate, kk, vv = OM.attention_qkv(qg, k, v, L, pos, lc)
        st.k[key][:, pos] = kk
        st.v[key][:, pos] = vv
        mix = OM.attention_core(q, gate, st.k[key], st.v[key], pos + 1, lc)
    h = h + reduce_parts(F.linear(mix.float(), L["out"].float()))
    x = OM.rmsnorm1p(h, L["post_norm"], lc.eps)
    g, u = F.linear(x.float(), L["gate"].float()), F.linear(x.float(), L["up"].float())
    act = (F.silu(g) * u).to(BF16)
    return h + reduce_parts(F.linear(act.float(), L["down"].float()))


@torch.no_grad()
def tp_decode_step(W, st, tok, lc):
    """Returns (this rank's logits slice [V / t] bf16, hidden after the final norm)."""
    h = W["embed"][tok]
    for l, L in enumerate(W["layers"]):
        h = tp_layer(h, L, st, l, st.pos, lc)
    st.pos += 1
    hf = OM.rmsnorm1p(h, W["final_norm"], lc.eps)
    return OM.lin(hf, W["lm_head"]), hf


@torch.no_grad()
def tp_mtp_step(W, st, h_prev, next_tok, pos, lc):
    M = W["mtp"]
    rank, t = dist.get_rank(), dist.get_world_size()
    e = OM.rmsnorm1p(W["embed"][next_tok], M["pre_e"], lc.eps)
    hh = OM.rmsnorm1p(h_prev, M["pre_h"], lc.eps)
    cat = torch.cat([e, hh])
    w = cat.numel() // t
    u = reduce_parts(F.linear(cat[rank * w:(rank + 1) * w].float(), M["fc"].float()))
    u = tp_layer(u, M, st, "mtp", pos, lc)
    hn = OM.rmsnorm1p(u, M["norm"], lc.eps)
    return OM.lin(hn, W["lm_head"]), hn


def merge_argmax(local_logits: torch.Tensor, base: int) -> int:
    """Vocabulary-split greedy token: local first-max, exchange (value, id), keep the larger value
    and on equal values the lower id."""
    i = int(torch.argmax(local_logits.float()))
    cand = torch.tensor([float(local_logits[i]), float(base + i)], dtype=torch.float64)
    allc = [torch.empty_like(cand) for _ in range(dist.get_world_size())]
    dist.all_gather(allc, cand)
    bv, bi = allc[0].tolist()
    for v, j in (c.tolist() for c in allc[1:]):
        if v > bv or (v == bv and j < bi):
            bv, bi = v, j
    return int(bi)


def gather_logits(local_logits: torch.Tensor) -> torch.Tensor:
    parts = [torch.empty_like(local_logits) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local_logits.contiguous())
    return torch.cat(parts, dim=-1)
