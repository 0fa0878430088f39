"""Shared test helpers: conversions between the engine's packed weights and the oracle's dense
fp32 weights, comparison metrics."""
from __future__ import annotations

import numpy as np
import torch

from oracle import model as OM
from oracle import w4 as OW


def dequant_oracle(p):
    """W4Packed -> fp32 torch weights through the ORACLE's dequantiser (numpy)."""
    r = OW.dequantize(p.qw.cpu().numpy(), p.scales.cpu().numpy(), p.M, p.K, p.gate_up)
    if p.gate_up:
        return torch.from_numpy(r[0]), torch.from_numpy(r[1])
    return torch.from_numpy(r)


def oracle_config(cfg) -> OM.Config:
    return OM.Config(**{f: getattr(cfg, f) for f in (
        "hidden", "layers", "inter", "vocab", "eps", "layer_types", "hq", "hkv", "head_dim", "rope_theta",
        "rotary_dim", "hk", "hv", "dk", "dv", "conv_k", "mtp_layers", "tied")})


def _dense_layer(L):
    D = {"type": L["type"], "in_norm": L["in_norm"].cpu(), "post_norm": L["post_norm"].cpu(),
         "in_proj": dequant_oracle(L["in_proj"]), "out": dequant_oracle(L["out"]),
         "down": dequant_oracle(L["down"])}
    D["gate"], D["up"] = dequant_oracle(L["gate_up"])
    for k in ("conv_w", "A_log", "dt_bias", "norm_w", "q_norm", "k_norm", "norm", "pre_e", "pre_h"):
        if k in L:
            D[k] = L[k].cpu()
    if "fc" in L:
        D["fc"] = dequant_oracle(L["fc"])
    return D


def dense_model(W) -> dict:
    """Engine weights dict (packed) -> oracle weights dict (dense fp32, CPU)."""
    return {"embed": W["embed"].cpu(), "final_norm": W["final_norm"].cpu(),
            "lm_head": dequant_oracle(W["lm_head"]),
            "layers": [_dense_layer(L) for L in W["layers"]],
            "mtp": _dense_layer(W["mtp"]) if W.get("mtp") else None}


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-300))


def bf16_ulp_close(a, b, ulps=1):
    """|a - b| <= ulps * bf16 spacing at max(|a|, |b|); NaN must match NaN. Returns (ok, max err)."""
    a, b = a.float(), b.float()
    m = torch.maximum(a.abs(), b.abs())
    spacing = torch.where(m > 0, 2.0 ** (torch.floor(torch.log2(m.clamp_min(1e-38))) - 7),
                          torch.full_like(m, 1e-38))
    both_nan = torch.isnan(a) & torch.isnan(b)
    ok = ((a - b).abs() <= ulps * spacing) | (a == b) | both_nan
    ok &= torch.isnan(a) == torch.isnan(b)
    return bool(ok.all()), float((a - b).abs().nan_to_num().max())
