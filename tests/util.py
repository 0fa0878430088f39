"""Shared test helpers: comparison metrics, and the packed -> dense weight conversions of
oracle/convert.py under their short names."""
from __future__ import annotations

import numpy as np
import torch

from oracle.convert import dense_model, dequant_oracle, oracle_config, reference_named  # noqa: F401  (re-exported)


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
