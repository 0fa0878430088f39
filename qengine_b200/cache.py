"""Prepared-weights cache on disk, in the reference's directory layout, and the GPTQ-grid repack.

Layout (python/qengine/engine.py:215-236, 281-292, 307-331 of the reference): one directory
`<cache_dir>/<model name>-<tag>/` holding

    top.pt        {"embed": bf16 [V, H], "norm": bf16 [H], "lm_head_bf16": bf16 [V, H] or a stub}
    lm_head.pt    the packed lm_head (W4Packed)
    layerNN.pt    one dict per decoder layer: type, in_norm, post_norm, in_proj, out, gate_up, down,
                  fused_swiglu and the mixer's small tensors (conv_w, A_log, dt_bias, norm_w or
                  q_norm, k_norm); matrices are W4Packed
    mtp.pt        the draft layer: a full-attention layer dict plus fc, norm, pre_e, pre_h
    COMPLETE      written last; a directory without it is ignored (all or nothing)

The files are `torch.save` pickles that name the class `qengine.quant.W4Packed`. Reading maps
that name onto qengine_b200.quant.W4Packed (same five fields, same wire format); writing registers
an alias module for the duration of the dump, so a cache written here loads in the reference and
the other way round. `config_from_dir` / `write_config` cover the `config.json` keys the reference
reads (python/qengine/reference.py:63-85).
"""
from __future__ import annotations

import json
import pickle
import sys
import types
from contextlib import contextmanager
from pathlib import Path

import torch

from . import quant
from .quant import GROUP, W4Packed, pack_codes
from .synth import Config

CACHE_TAG = "w4-rtn-g128-v1"  # the reference's tag for this wire format (engine.py:85)
_FOREIGN = ("qengine.quant", "W4Packed")


def cache_path(cache_dir, model_name: str, tag: str = CACHE_TAG) -> Path:
    return Path(cache_dir) / f"{model_name}-{tag}"


# ---- pickle plumbing ---------------------------------------------------------------------------
class _Unpickler(pickle.Unpickler):
    def find_class(self, module, name):
        if (module, name) == _FOREIGN:
            return W4Packed
        return super().find_class(module, name)


class _pickle_reader:
    """The `pickle_module` torch.load wants: the stock module with the class name mapped."""
    __name__ = "pickle"
    Unpickler = _Unpickler
    load = staticmethod(lambda f, **kw: _Unpickler(f, **kw).load())
    loads = staticmethod(pickle.loads)


@contextmanager
def _reference_class_names():
    """While active, W4Packed pickles under the reference's module path."""
    saved = {k: sys.modules.get(k) for k in ("qengine", "qengine.quant")}
    old = (W4Packed.__module__, W4Packed.__qualname__)
    try:
        if saved["qengine.quant"] is None:
            pkg = saved["qengine"] or types.ModuleType("qengine")
            mod = types.ModuleType("qengine.quant")
            mod.W4Packed = W4Packed
            pkg.quant = mod
            sys.modules["qengine"], sys.modules["qengine.quant"] = pkg, mod
            W4Packed.__module__ = "qengine.quant"
        yield
    finally:
        W4Packed.__module__, W4Packed.__qualname__ = old
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _load(f: Path, device):
    return torch.load(f, map_location=device, weights_only=False, pickle_module=_pickle_reader)


def _cpu(obj):
    """Host copy of a weights subtree; packed matrices become whatever class currently answers to
    the reference's name (this module's alias, or the reference's own class when its package is
    imported in the same process)."""
    if isinstance(obj, W4Packed):
        cls = getattr(sys.modules.get("qengine.quant"), "W4Packed", W4Packed)
        return cls(obj.qw.cpu(), obj.scales.cpu(), int(obj.M), int(obj.K), bool(obj.gate_up))
    if isinstance(obj, torch.Tensor):
        return obj.cpu()
    if isinstance(obj, dict):
        return {k: _cpu(v) for k, v in obj.items()}
    return obj


# ---- directory <-> weights dict ----------------------------------------------------------------
def is_complete(directory) -> bool:
    return (Path(directory) / "COMPLETE").exists()


def save_cache(directory, weights: dict, lm_head_bf16: torch.Tensor | None = None, note: str = "") -> Path:
    """Write a weights dict (qengine_b200.synth.build_model layout) as a cache directory.
    lm_head_bf16: the unquantised head for `top.pt`; the reference drops it right after loading
    when a packed lm_head.pt exists, so a one-row stub is stored when it is not given."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "COMPLETE").unlink(missing_ok=True)
    H = weights["embed"].shape[1]
    stub = torch.zeros(1, H, dtype=torch.bfloat16) if lm_head_bf16 is None else lm_head_bf16
    with _reference_class_names():
        torch.save(_cpu({"embed": weights["embed"], "norm": weights["final_norm"], "lm_head_bf16": stub}),
                   d / "top.pt")
        if isinstance(weights["lm_head"], W4Packed):
            torch.save(_cpu(weights["lm_head"]), d / "lm_head.pt")
        for i, L in enumerate(weights["layers"]):
            torch.save(_cpu(L), d / f"layer{i:02d}.pt")
        if weights.get("mtp"):
            torch.save(_cpu(weights["mtp"]), d / "mtp.pt")
    packed = isinstance(weights["lm_head"], W4Packed)
    (d / "COMPLETE").write_text(
        f"{CACHE_TAG} lm_head={'same' if packed else 'bf16'} mtp={bool(weights.get('mtp'))} {note}\n")
    return d


def load_cache(directory, cfg: Config, device="cpu", mtp: bool = True) -> dict:
    """Read a complete cache directory into a weights dict for `Engine`. Raises FileNotFoundError
    for a directory without its COMPLETE marker or with a layer file missing."""
    d = Path(directory)
    if not is_complete(d):
        raise FileNotFoundError(f"{d}: no COMPLETE marker (partial caches are not used)")
    top = _load(d / "top.pt", device)
    W = {"embed": top["embed"], "final_norm": top["norm"], "layers": [], "mtp": None}
    if (d / "lm_head.pt").exists():
        W["lm_head"] = _load(d / "lm_head.pt", device)
    elif (d / "lm_head_w4gptq.pt").exists():  # the reference's GPTQ head: {"packed", "stats", "src"}
        W["lm_head"] = _load(d / "lm_head_w4gptq.pt", device)["packed"]
    else:
        W["lm_head"] = top["lm_head_bf16"].contiguous()
    for i, kind in enumerate(cfg.layer_types):
        L = _load(d / f"layer{i:02d}.pt", device)
        if L["type"] != kind:
            raise ValueError(f"{d}/layer{i:02d}.pt is a {L['type']} layer, the config says {kind}")
        W["layers"].append(L)
    if mtp and cfg.mtp_layers > 0 and (d / "mtp.pt").exists():
        W["mtp"] = _load(d / "mtp.pt", device)
    return W


# ---- config.json -------------------------------------------------------------------------------
def config_from_dir(path) -> Config:
    """The fields of a checkpoint's config.json that the decode step needs."""
    raw = json.loads((Path(path) / "config.json").read_text())
    t = raw.get("text_config", raw)
    rope = t["rope_parameters"]
    eos = t.get("eos_token_id", [])
    gen = Path(path) / "generation_config.json"
    if gen.exists():
        eos = json.loads(gen.read_text()).get("eos_token_id", eos)
    hd = t["head_dim"]
    return Config(hidden=t["hidden_size"], layers=t["num_hidden_layers"], inter=t["intermediate_size"],
                  vocab=t["vocab_size"], eps=t["rms_norm_eps"], layer_types=list(t["layer_types"]),
                  hq=t["num_attention_heads"], hkv=t["num_key_value_heads"], head_dim=hd,
                  rope_theta=float(rope["rope_theta"]),
                  rotary_dim=int(hd * rope.get("partial_rotary_factor", 1.0)),
                  hk=t["linear_num_key_heads"], hv=t["linear_num_value_heads"],
                  dk=t["linear_key_head_dim"], dv=t["linear_value_head_dim"],
                  conv_k=t["linear_conv_kernel_dim"], mtp_layers=t.get("mtp_num_hidden_layers", 0),
                  tied=bool(raw.get("tie_word_embeddings", t.get("tie_word_embeddings", False))),
                  eos=eos if isinstance(eos, list) else [eos])


def write_config(path, cfg: Config) -> Path:
    """config.json with the keys `config_from_dir` (and the reference's Config.from_dir) read."""
    p = Path(path)
    p.mkdir(parents=True, exist_ok=True)
    t = {"hidden_size": cfg.hidden, "num_hidden_layers": cfg.layers, "intermediate_size": cfg.inter,
         "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps, "layer_types": list(cfg.layer_types),
         "num_attention_heads": cfg.hq, "num_key_value_heads": cfg.hkv, "head_dim": cfg.head_dim,
         "rope_parameters": {"rope_theta": cfg.rope_theta,
                             "partial_rotary_factor": cfg.rotary_dim / cfg.head_dim},
         "linear_num_key_heads": cfg.hk, "linear_num_value_heads": cfg.hv,
         "linear_key_head_dim": cfg.dk, "linear_value_head_dim": cfg.dv,
         "linear_conv_kernel_dim": cfg.conv_k, "mtp_num_hidden_layers": cfg.mtp_layers,
         "eos_token_id": list(cfg.eos)}
    (p / "config.json").write_text(json.dumps({"text_config": t, "tie_word_embeddings": cfg.tied}, indent=1))
    return p / "config.json"


# ---- GPTQ-grid repack --------------------------------------------------------------------------
@torch.no_grad()
def pack_from_grid(Wq: torch.Tensor, rows_per_step: int = 2048):
    """Pack a matrix whose values already lie on the W4 grid (code * scale with code in -8..7 and
    one fp16 scale per 128-group, stored rounded to bf16; e.g. a GPTQ-quantised lm_head) WITHOUT
    quantising again. Serves the reference's `W4Linear.prepare_from_grid`
    (python/qengine/engine.py:117-180).

    Per group the scale is recovered by trial: absmax is |code| * scale for some |code| in 1..8,
    seen through one bf16 rounding (up to four fp16 steps, plus the division), so the fp16 numbers within six steps
    of absmax / 8, absmax / 7, ... absmax / 1 are tried and the one whose grid reproduces the
    stored bf16 values best is kept (ties: the first in the order tried, which starts with the
    reference's own candidates, / 7 and / 8 with two steps). The wider search also recovers groups
    whose extreme codes are not in use or whose scale lies more than two steps off. The codes
    and scales found go straight into the packer, so the packed matrix holds exactly the grid
    point chosen (the reference has only a quantiser to pack with and builds an fp32 matrix that
    its quantiser maps onto the same grid point). Returns (W4Packed, {"exact_frac": fraction of
    stored values reproduced bit for bit after bf16 rounding})."""
    M, K = Wq.shape
    if K % GROUP:
        raise ValueError("grid repack needs K to be a multiple of 128")
    Mp = -(-M // 16) * 16
    G = K // GROUP
    dev = Wq.device
    codes = torch.full((Mp, K), 8, dtype=torch.uint8, device=dev)
    scales = torch.zeros(Mp, G, dtype=torch.float16, device=dev)
    hits = 0
    for r0 in range(0, M, rows_per_step):
        v = Wq[r0:r0 + rows_per_step].float().view(-1, G, GROUP)
        top = v.abs().amax(-1, keepdim=True)
        best_s = torch.ones_like(top)
        best_err = torch.full_like(top, float("inf"))
        # candidates in the reference's order first (absmax / 7 then / 8, two steps either way), so
        # that a group it reproduces exactly gets the same scale here; then the wider search
        trials = [(fs, st) for fs in (7.0, 8.0) for st in (-2, -1, 0, 1, 2)]
        trials += [(fs, st) for fs in (7.0, 8.0) for st in (-6, -5, -4, -3, 3, 4, 5, 6)]
        trials += [(fs, st) for fs in (6.0, 5.0, 4.0, 3.0, 2.0, 1.0) for st in range(-6, 7)]
        for full_scale, step in trials:
            est = (top / full_scale).to(torch.float16)
            s = (est.view(torch.int16) + step).view(torch.float16).float()
            s = torch.where((s > 0) & torch.isfinite(s), s, torch.ones_like(s))
            q = torch.clamp(torch.round(v / s), -8, 7)
            err = ((q * s).to(torch.bfloat16).float() - v).abs().sum(-1, keepdim=True)
            take = err < best_err
            best_s = torch.where(take, s, best_s)
            best_err = torch.where(take, err, best_err)
        empty = top == 0
        best_s = torch.where(empty, torch.zeros_like(best_s), best_s)
        div = torch.where(empty, torch.ones_like(best_s), best_s)
        q = torch.clamp(torch.round(v / div), -8, 7)
        hits += ((q * best_s).to(torch.bfloat16).float() == v).sum().item()
        n = v.shape[0]
        codes[r0:r0 + n] = (q + 8).to(torch.uint8).view(n, K)
        scales[r0:r0 + n] = best_s.squeeze(-1).to(torch.float16)
    packed = pack_codes(codes, scales, M, K)
    return packed, {"exact_frac": hits / max(1, M * K)}


__all__ = ["CACHE_TAG", "cache_path", "save_cache", "load_cache", "is_complete", "config_from_dir",
           "write_config", "pack_from_grid", "quant"]
