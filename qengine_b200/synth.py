"""Model configuration and seeded synthetic weights in the engine's fused W4 layout.

No checkpoint, tokenizer or dataset is available offline, so every measurement and parity test
runs on random-init weights of the right shapes: int4 codes uniform in 0..15, one fp16 scale per
(row, group) drawn as |N(0,1)| * scale_std, bf16 norms and embedding. One torch.Generator per
tensor, seeded from (seed, tensor index) in a fixed order, so CPU and GPU builds of the tiny
model are bit-identical and the 27B-shape model is reproducible on the GPU.

Layer dictionaries follow the reference engine's fused layout (python/qengine/engine.py:307-331):
DeltaNet in_proj rows [qkv | z | b | a], attention in_proj rows [per-head q|gate | k | v],
MLP gate/up interleaved in blocks of 8 rows for the fused SwiGLU epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .quant import W4Packed

BF16 = torch.bfloat16


@dataclass
class Config:
    """Same fields as the reference Config (python/qengine/reference.py:27-61)."""
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

    @property
    def gdn_proj_rows(self):
        return self.conv_dim + self.value_dim + 2 * self.hv

    @property
    def attn_proj_rows(self):
        return self.hq * 2 * self.head_dim + 2 * self.hkv * self.head_dim


def _pattern(layers: int) -> list:
    """3:1 DeltaNet : attention, attention at l % 4 == 3."""
    return ["full_attention" if l % 4 == 3 else "linear_attention" for l in range(layers)]


def tiny_config() -> Config:
    """The CPU-runnable case: 4 layers, hidden 512, vocab 4096."""
    return Config(hidden=512, layers=4, inter=1536, vocab=4096, eps=1e-6, layer_types=_pattern(4),
                  hq=8, hkv=2, head_dim=64, rope_theta=1e7, rotary_dim=16, hk=4, hv=8, dk=64, dv=64)


def shardable8_config() -> Config:
    """A small configuration that an 8-way tensor-parallel engine can shard: 16 query / 4 KV heads
    (KV heads shared by rank pairs at t = 8), 8 key / 16 value DeltaNet heads, every K split a
    multiple of 128."""
    return Config(hidden=512, layers=4, inter=2048, vocab=4096, eps=1e-6, layer_types=_pattern(4),
                  hq=16, hkv=4, head_dim=64, rope_theta=1e7, rotary_dim=16, hk=8, hv=16, dk=64, dv=64)


def qwen27b_config(layers: int = 64) -> Config:
    """27B shape: 64 layers (48 DeltaNet + 16 attention), hidden 5120, vocab 248,320."""
    return Config(hidden=5120, layers=layers, inter=17408, vocab=248320, eps=1e-6,
                  layer_types=_pattern(layers), hq=24, hkv=4, head_dim=256, rope_theta=1e7,
                  rotary_dim=64, hk=16, hv=48, dk=128, dv=128)


class _Seeds:
    def __init__(self, seed: int, device):
        self.seed, self.i, self.device = seed, 0, torch.device(device)

    def gen(self) -> torch.Generator:
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 1_000_003 + self.i)
        self.i += 1
        return g


def random_w4(rows: int, K: int, g: torch.Generator, device, scale_std: float, M: int | None = None,
              gate_up: bool = False) -> W4Packed:
    """Packed matrix with uniform codes and |N(0,1)| * scale_std scales; rows % 16 == 0 and
    K % 128 == 0 (true for every matrix of both configurations), so no padding nibbles exist."""
    assert rows % 16 == 0 and K % 128 == 0
    T, Cn, G = rows // 16, K // 64, K // 128
    words = torch.randint(0, 2**32, (T, Cn, 32, 4), generator=g, device=device, dtype=torch.int64)
    qw = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    del words
    sc = (torch.randn(T, G, 16, generator=g, device=device).abs() * scale_std).to(torch.float16)
    return W4Packed(qw, sc, M if M is not None else (rows // 2 if gate_up else rows), K, gate_up)


def _small(shape, g, device, std=1.0, mean=0.0):
    return (torch.randn(*shape, generator=g, device=device) * std + mean).to(BF16)


def _layer(cfg: Config, kind: str, S: _Seeds, scale_std: float) -> dict:
    dev, H, I = S.device, cfg.hidden, cfg.inter
    L = {"type": kind,
         "in_norm": _small((H,), S.gen(), dev, 0.1), "post_norm": _small((H,), S.gen(), dev, 0.1)}
    if kind == "linear_attention":
        L["in_proj"] = random_w4(cfg.gdn_proj_rows, H, S.gen(), dev, scale_std)
        L["out"] = random_w4(H, cfg.value_dim, S.gen(), dev, scale_std)
        L["conv_w"] = _small((cfg.conv_dim, 1, cfg.conv_k), S.gen(), dev, 0.5)
        g = S.gen()
        L["A_log"] = (torch.rand(cfg.hv, generator=g, device=dev) * 5.7 - 3.0).to(BF16)
        L["dt_bias"] = _small((cfg.hv,), S.gen(), dev, 1.0)
        L["norm_w"] = _small((cfg.dv,), S.gen(), dev, 0.2, 1.0)
    else:
        L["in_proj"] = random_w4(cfg.attn_proj_rows, H, S.gen(), dev, scale_std)
        L["out"] = random_w4(H, cfg.hq * cfg.head_dim, S.gen(), dev, scale_std)
        L["q_norm"] = _small((cfg.head_dim,), S.gen(), dev, 0.3)
        L["k_norm"] = _small((cfg.head_dim,), S.gen(), dev, 0.3)
    L["gate_up"] = random_w4(2 * I, H, S.gen(), dev, scale_std, M=I, gate_up=True)
    L["down"] = random_w4(H, I, S.gen(), dev, scale_std)
    L["fused_swiglu"] = True
    return L


@torch.no_grad()
def build_model(cfg: Config, seed: int = 0, device="cpu", scale_std: float = 0.01, mtp: bool = True) -> dict:
    """Weights dict: embed, final_norm, lm_head, layers[], mtp (or None)."""
    S = _Seeds(seed, device)
    dev = S.device
    W = {"embed": _small((cfg.vocab, cfg.hidden), S.gen(), dev, 1.0),
         "final_norm": _small((cfg.hidden,), S.gen(), dev, 0.1),
         "lm_head": random_w4(cfg.vocab, cfg.hidden, S.gen(), dev, scale_std),
         "layers": [_layer(cfg, t, S, scale_std) for t in cfg.layer_types], "mtp": None}
    if mtp and cfg.mtp_layers > 0:
        Mt = _layer(cfg, "full_attention", S, scale_std)
        Mt["fc"] = random_w4(cfg.hidden, 2 * cfg.hidden, S.gen(), dev, scale_std)
        Mt["norm"] = _small((cfg.hidden,), S.gen(), dev, 0.1)
        Mt["pre_e"] = _small((cfg.hidden,), S.gen(), dev, 0.1)
        Mt["pre_h"] = _small((cfg.hidden,), S.gen(), dev, 0.1)
        W["mtp"] = Mt
    return W


def model_to(W: dict, device) -> dict:
    """Copy a weights dict to another device (packed matrices included)."""
    def mv(v):
        if isinstance(v, (torch.Tensor, W4Packed)):
            return v.to(device)
        if isinstance(v, dict):
            return {k: mv(x) for k, x in v.items()}
        if isinstance(v, list):
            return [mv(x) for x in v]
        return v
    return mv(W)


def packed_bytes(W: dict) -> dict:
    """Bytes of packed weights a decode step streams: decoder, lm_head, mtp."""
    def layer_bytes(L):
        return sum(L[k].nbytes for k in ("in_proj", "out", "gate_up", "down"))
    out = {"decoder": sum(layer_bytes(L) for L in W["layers"]), "lm_head": W["lm_head"].nbytes, "mtp": 0}
    if W.get("mtp"):
        out["mtp"] = layer_bytes(W["mtp"]) + W["mtp"]["fc"].nbytes
    return out


def prompt_ids(n: int, vocab: int, seed: int = 1234) -> list:
    """Seeded-uniform token ids."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
