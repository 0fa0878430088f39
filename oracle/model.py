"""Oracle (test infrastructure): the hybrid Gated-DeltaNet / gated-attention model on CPU torch,
one token per step, restating python/qengine/reference.py of the reference with every bf16
rounding point kept. Linear layers use the reference's fake-quant definition for W4 weights
(tests/test_27b_w4.py:70-71): bf16 activations, fp32 dequantised weights, fp32 accumulation, one
rounding to bf16.

Weights are a plain dict in the fused layout the engine uses (python/qengine/engine.py:307-331):

  W = {"embed": bf16 [V, H], "final_norm": bf16 [H], "lm_head": fp32 [V, H],
       "layers": [layer, ...], "mtp": layer + {"fc": fp32 [H, 2H], "norm", "pre_e", "pre_h"}}
  DeltaNet layer : type "linear_attention", in_norm, post_norm, in_proj fp32 [C + Vd + 2 Hv, H]
                   (rows [qkv | z | b | a]), out fp32 [H, Vd], gate, up fp32 [I, H], down fp32
                   [H, I], conv_w bf16 [C, 1, 4], A_log, dt_bias bf16 [Hv], norm_w bf16 [dv]
  attention layer: type "full_attention", in_proj fp32 [Hq 2 hd + 2 Hkv hd, H] (rows
                   [per-head q|gate, k, v]), out fp32 [H, Hq hd], q_norm, k_norm bf16 [hd]
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

BF16, F32 = torch.bfloat16, torch.float32


@dataclass
class Config:
    """Same fields as the reference Config (reference.py:27-61)."""
    hidden: int
    layers: int
    inter: int
    vocab: int
    eps: float
    layer_types: list
    hq: int
    hkv: int
    head_dim: int
    rope_theta: float
    rotary_dim: int
    hk: int
    hv: int
    dk: int
    dv: int
    conv_k: int = 4
    mtp_layers: int = 1
    tied: bool = False
    eos: list = field(default_factory=list)

    @property
    def key_dim(self):
        return self.hk * self.dk

    @property
    def value_dim(self):
        return self.hv * self.dv

    @property
    def conv_dim(self):
        return 2 * self.key_dim + self.value_dim


def lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Fake-quant linear (tests/test_27b_w4.py:70-71)."""
    return F.linear(x.float(), w.float()).to(BF16)


def rmsnorm1p(x, w, eps):
    """Zero-centred RMSNorm in fp32, one rounding (reference.py:132-136)."""
    xf = x.float()
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    return (y * (1.0 + w.float())).to(x.dtype)


def rmsnorm_gated(x, z, w, eps):
    """bf16(norm(x)) -> bf16(w * .) -> bf16(. * silu(z_f32)) (reference.py:139-146)."""
    xf = x.float()
    n = (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)).to(x.dtype)
    y = w * n
    return (y * F.silu(z.float())).to(x.dtype)


def l2norm(x, eps=1e-6):
    """reference.py:149-150"""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def inv_freq(cfg: Config) -> torch.Tensor:
    rd = cfg.rotary_dim
    return 1.0 / (cfg.rope_theta ** (torch.arange(0, rd, 2, dtype=F32) / rd))


def rope_cos_sin(pos: int, cfg: Config):
    """cos/sin over rotary_dim dims in fp32, cast to bf16 (reference.py:158-166)."""
    fr = torch.tensor(float(pos)) * inv_freq(cfg)
    emb = torch.cat([fr, fr])
    return emb.cos().to(BF16), emb.sin().to(BF16)


def apply_rope(x, cos, sin):
    """Rotate-half on the first rotary_dim dims, bf16 elementwise (reference.py:169-176)."""
    rd = cos.shape[-1]
    xr, rest = x[..., :rd], x[..., rd:]
    a, b = xr[..., :rd // 2], xr[..., rd // 2:]
    rot = torch.cat([-b, a], dim=-1)
    return torch.cat([xr * cos + rot * sin, rest], dim=-1)


class State:
    """Per-sequence state (reference.py:182-195): conv history bf16 [C, conv_k - 1] oldest first,
    S fp32 [hv, dk, dv], K/V caches bf16 [hkv, max_len, head_dim]. Key = layer index ("mtp" for
    the draft head's attention layer)."""

    def __init__(self, cfg: Config, max_len: int, with_mtp: bool = True):
        self.pos = 0
        self.max_len = max_len
        self.conv, self.S, self.k, self.v = {}, {}, {}, {}
        for l, t in enumerate(cfg.layer_types):
            if t == "linear_attention":
                self.conv[l] = torch.zeros(cfg.conv_dim, cfg.conv_k - 1, dtype=BF16)
                self.S[l] = torch.zeros(cfg.hv, cfg.dk, cfg.dv, dtype=F32)
            else:
                self.k[l] = torch.zeros(cfg.hkv, max_len, cfg.head_dim, dtype=BF16)
                self.v[l] = torch.zeros(cfg.hkv, max_len, cfg.head_dim, dtype=BF16)
        if with_mtp:
            self.k["mtp"] = torch.zeros(cfg.hkv, max_len, cfg.head_dim, dtype=BF16)
            self.v["mtp"] = torch.zeros(cfg.hkv, max_len, cfg.head_dim, dtype=BF16)

    def snapshot(self):
        """Recurrent part only (K/V rows past pos are never read, so they need no undo)."""
        return (self.pos, {l: c.clone() for l, c in self.conv.items()},
                {l: s.clone() for l, s in self.S.items()})

    def restore(self, snap):
        self.pos = snap[0]
        for l in self.conv:
            self.conv[l].copy_(snap[1][l])
            self.S[l].copy_(snap[2][l])


def deltanet_core(qkv, z, b, a, L, conv_state, S, cfg: Config):
    """Everything between in_proj and out_proj of a DeltaNet layer for one token
    (reference.py:211-242). qkv [C], z [hv*dv], b, a [hv] bf16. Updates conv_state and S."""
    z = z.view(cfg.hv, cfg.dv)
    wc = L["conv_w"].view(cfg.conv_dim, cfg.conv_k)
    window = torch.cat([conv_state, qkv[:, None]], dim=-1)
    conv_state.copy_(window[:, 1:])
    conv = (window.float() * wc.float()).sum(-1).to(BF16)
    act = F.silu(conv)
    q, k, v = torch.split(act, [cfg.key_dim, cfg.key_dim, cfg.value_dim])
    q, k, v = q.view(cfg.hk, cfg.dk), k.view(cfg.hk, cfg.dk), v.view(cfg.hv, cfg.dv)
    beta = b.sigmoid()
    g = -L["A_log"].float().exp() * F.softplus(a.float() + L["dt_bias"])
    rep = cfg.hv // cfg.hk
    if rep > 1:  # value head j reads q/k head j // rep
        q, k = q.repeat_interleave(rep, dim=0), k.repeat_interleave(rep, dim=0)
    qf = l2norm(q.float()) / math.sqrt(cfg.dk)
    kf = l2norm(k.float())
    vf, bf = v.float(), beta.float()
    S.mul_(g.exp()[:, None, None])
    kv = (S * kf[:, :, None]).sum(dim=1)
    delta = (vf - kv) * bf[:, None]
    S.add_(kf[:, :, None] * delta[:, None, :])
    o = (S * qf[:, :, None]).sum(dim=1).to(BF16)
    return rmsnorm_gated(o, z, L["norm_w"], cfg.eps).reshape(-1)


def split_gdn_proj(pr, cfg: Config):
    c0, c1 = cfg.conv_dim, cfg.conv_dim + cfg.value_dim
    return pr[:c0], pr[c0:c1], pr[c1:c1 + cfg.hv], pr[c1 + cfg.hv:c1 + 2 * cfg.hv]


def split_attn_proj(pr, cfg: Config):
    q0 = cfg.hq * 2 * cfg.head_dim
    k1 = q0 + cfg.hkv * cfg.head_dim
    return pr[:q0], pr[q0:k1], pr[k1:k1 + cfg.hkv * cfg.head_dim]


def attention_qkv(qg, k, v, L, pos, cfg: Config):
    """Per-head q/k norm and RoPE from the projection rows (reference.py:252-260). Returns
    q [hq, hd], gate [hq*hd], k [hkv, hd], v [hkv, hd]."""
    hd = cfg.head_dim
    qg = qg.view(cfg.hq, 2 * hd)
    q, gate = qg[:, :hd], qg[:, hd:].reshape(-1)
    q = rmsnorm1p(q, L["q_norm"], cfg.eps)
    k = rmsnorm1p(k.view(cfg.hkv, hd), L["k_norm"], cfg.eps)
    cos, sin = rope_cos_sin(pos, cfg)
    return apply_rope(q, cos, sin), gate, apply_rope(k, cos, sin), v.view(cfg.hkv, hd)


def attention_core(q, gate, kc, vc, n, cfg: Config):
    """softmax(q K^T / sqrt(hd)) V over cache rows [0, n), fp32 softmax, output rounded to bf16
    then multiplied by bf16 sigmoid(gate) (reference.py:263-272)."""
    grp = cfg.hq // cfg.hkv
    K = kc[:, :n].float().repeat_interleave(grp, 0)
    V = vc[:, :n].float().repeat_interleave(grp, 0)
    s = torch.einsum("hd,hnd->hn", q.float(), K) * cfg.head_dim ** -0.5
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hn,hnd->hd", p, V).to(BF16).reshape(-1)
    return o * torch.sigmoid(gate)


def mlp(x, L, fused_swiglu=False):
    """SwiGLU MLP (reference.py:283-287). fused_swiglu=True models the GEMV epilogue instead
    (csrc/gemv_w4.cu:188-193): silu(g) * u on the unrounded fp32 sums, one rounding."""
    if fused_swiglu:
        g, u = F.linear(x.float(), L["gate"].float()), F.linear(x.float(), L["up"].float())
        act = (F.silu(g) * u).to(BF16)
    else:
        act = F.silu(lin(x, L["gate"])) * lin(x, L["up"])
    return lin(act, L["down"])


def decoder_layer(h, L, st: State, key, pos, cfg: Config, fused_swiglu=False):
    """One layer on one token (reference.py:290-299). key selects the layer's state."""
    x = rmsnorm1p(h, L["in_norm"], cfg.eps)
    pr = lin(x, L["in_proj"])
    if L["type"] == "linear_attention":
        mix = deltanet_core(*split_gdn_proj(pr, cfg), L, st.conv[key], st.S[key], cfg)
    else:
        qg, k, v = split_attn_proj(pr, cfg)
        q, gate, kk, vv = attention_qkv(qg, k, v, L, pos, cfg)
        st.k[key][:, pos] = kk
        st.v[key][:, pos] = vv
        mix = attention_core(q, gate, st.k[key], st.v[key], pos + 1, cfg)
    h = h + lin(mix, L["out"])
    x = rmsnorm1p(h, L["post_norm"], cfg.eps)
    return h + mlp(x, L, fused_swiglu)


@torch.no_grad()
def decode_step(W, st: State, tok: int, cfg: Config, fused_swiglu=False):
    """One token through the main model (reference.py:306-315). Returns (bf16 logits [V],
    hidden after the final norm [H])."""
    h = W["embed"][tok]
    for l, L in enumerate(W["layers"]):
        h = decoder_layer(h, L, st, l, st.pos, cfg, fused_swiglu)
    st.pos += 1
    hf = rmsnorm1p(h, W["final_norm"], cfg.eps)
    return lin(hf, W["lm_head"]), hf


@torch.no_grad()
def mtp_step(W, st: State, h_prev, next_tok: int, pos: int, cfg: Config, fused_swiglu=False):
    """One draft row (reference.py:354-367): h_prev = hidden after the final norm at `pos` (or,
    when chaining, the previous draft row's hidden after mtp.norm), next_tok = token at pos + 1;
    the draft head's attention layer runs at `pos`. Returns (logits, hidden after mtp.norm)."""
    M = W["mtp"]
    e = rmsnorm1p(W["embed"][next_tok], M["pre_e"], cfg.eps)
    hh = rmsnorm1p(h_prev, M["pre_h"], cfg.eps)
    u = lin(torch.cat([e, hh]), M["fc"])
    u = decoder_layer(u, M, st, "mtp", pos, cfg, fused_swiglu)
    hn = rmsnorm1p(u, M["norm"], cfg.eps)
    return lin(hn, W["lm_head"]), hn
