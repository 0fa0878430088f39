"""Conversions between the engine's packed weights and the dense fp32 weights the CPU oracle (and
the reference's torch model) multiply with -- TEST INFRASTRUCTURE, like the rest of oracle/.

  dequant_oracle   W4Packed -> fp32 weights through the oracle's own dequantiser (oracle/w4.py)
  oracle_config    engine Config -> oracle Config (same field names)
  dense_model      engine weights dict -> oracle weights dict (fused rows kept fused)
  reference_named  oracle weights dict -> the reference's HF-style names, the fusion of
                   python/qengine/engine.py:307-331 undone (python/qengine/reference.py reads these)
"""
from __future__ import annotations

import torch

from . import model as OM
from . import w4 as OW


def dequant_oracle(p):
    r = OW.dequantize(p.qw.cpu().numpy(), p.scales.cpu().numpy(), p.M, p.K, p.gate_up)
    if p.gate_up:
        return torch.from_numpy(r[0]), torch.from_numpy(r[1])
    return torch.from_numpy(r)


def oracle_config(cfg) -> OM.Config:
    return OM.Config(**{f: getattr(cfg, f) for f in (
        "hidden", "layers", "inter", "vocab", "eps", "layer_types", "hq", "hkv", "head_dim", "rope_theta",
        "rotary_dim", "hk", "hv", "dk", "dv", "conv_k", "mtp_layers", "tied")})


def dense_layer(L) -> dict:
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
    return {"embed": W["embed"].cpu(), "final_norm": W["final_norm"].cpu(),
            "lm_head": dequant_oracle(W["lm_head"]),
            "layers": [dense_layer(L) for L in W["layers"]],
            "mtp": dense_layer(W["mtp"]) if W.get("mtp") else None}


def reference_named(D, cfg) -> dict:
    W = {"embed_tokens.weight": D["embed"], "norm.weight": D["final_norm"], "lm_head.weight": D["lm_head"]}

    def put(L, p, kind):
        W[p + "input_layernorm.weight"] = L["in_norm"]
        W[p + "post_attention_layernorm.weight"] = L["post_norm"]
        W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"] = L["gate"], L["up"]
        W[p + "mlp.down_proj.weight"] = L["down"]
        ip = L["in_proj"]
        if kind == "linear_attention":
            q = p + "linear_attn."
            c0, c1 = cfg.conv_dim, cfg.conv_dim + cfg.value_dim
            W[q + "in_proj_qkv.weight"], W[q + "in_proj_z.weight"] = ip[:c0], ip[c0:c1]
            W[q + "in_proj_b.weight"], W[q + "in_proj_a.weight"] = ip[c1:c1 + cfg.hv], ip[c1 + cfg.hv:]
            W[q + "out_proj.weight"] = L["out"]
            W[q + "conv1d.weight"], W[q + "A_log"] = L["conv_w"], L["A_log"]
            W[q + "dt_bias"], W[q + "norm.weight"] = L["dt_bias"], L["norm_w"]
        else:
            q = p + "self_attn."
            q0 = cfg.hq * 2 * cfg.head_dim
            k1 = q0 + cfg.hkv * cfg.head_dim
            W[q + "q_proj.weight"], W[q + "k_proj.weight"], W[q + "v_proj.weight"] = ip[:q0], ip[q0:k1], ip[k1:]
            W[q + "o_proj.weight"] = L["out"]
            W[q + "q_norm.weight"], W[q + "k_norm.weight"] = L["q_norm"], L["k_norm"]

    for l, L in enumerate(D["layers"]):
        put(L, f"layers.{l}.", L["type"])
    if D.get("mtp"):
        M = D["mtp"]
        put(M, "mtp.layers.0.", "full_attention")
        W["mtp.fc.weight"], W["mtp.norm.weight"] = M["fc"], M["norm"]
        W["mtp.pre_fc_norm_embedding.weight"], W["mtp.pre_fc_norm_hidden.weight"] = M["pre_e"], M["pre_h"]
    return W
