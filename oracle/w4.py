"""Oracle (test infrastructure): the W4 wire format restated with numpy loops-free integer code.

Follows python/qengine/quant.py of the reference:
  - quantiser `_scales_and_codes` (quant.py:65-75): scale = fp16(2 absmax / 15),
    code = clamp(round_half_even(w / scale) + 8, 0, 15), all-zero group -> scale 0, codes 8;
  - layout `_index_map` / `_pack` (quant.py:54-62, 78-104): lane l = 4 g + t of tile/chunk holds
    rows g, g + 8 and k = 64 c + 16 t + 4 s + {0..3} in word s; nibble j = row g + 8 (j & 1),
    k0 + 2 ((j >> 1) & 1) + (j >> 2); scales stored [tile, group, row-in-tile];
  - gate/up interleave `quantize_w4_gate_up` (quant.py:114-125);
  - `dequantize_w4` (quant.py:128-148).
Arrays are numpy; fp16 scales are numpy float16 (same IEEE format as torch.float16).
"""
from __future__ import annotations

import numpy as np

GROUP = 128


def ceil_to(a: int, b: int) -> int:
    return (a + b - 1) // b * b


def lane_map():
    """row_in_tile[32, 4, 8], k_in_chunk[32, 4, 8] for (lane, word, nibble)."""
    lane = np.arange(32).reshape(32, 1, 1)
    s = np.arange(4).reshape(1, 4, 1)
    j = np.arange(8).reshape(1, 1, 8)
    g, t = lane // 4, lane % 4
    row = g + 8 * (j & 1) + 0 * s
    k = 16 * t + 4 * s + 2 * ((j >> 1) & 1) + (j >> 2)
    return np.broadcast_to(row, (32, 4, 8)), np.broadcast_to(k, (32, 4, 8))


def quantize_codes(W: np.ndarray):
    """W float32 [Mp, Kp] (already padded) -> (codes uint8 [Mp, Kp], scales float16 [Mp, Kp/128])."""
    Mp, Kp = W.shape
    g = W.reshape(Mp, Kp // GROUP, GROUP).astype(np.float32)
    absmax = np.abs(g).max(axis=-1)
    s16 = (absmax * np.float32(2.0 / 15.0)).astype(np.float16)
    s = s16.astype(np.float32)
    safe = np.where(s > 0, s, np.float32(1.0))
    q = np.rint(g / safe[..., None]) + 8          # rint = round half to even, like torch.round
    q = np.clip(q, 0, 15)
    q = np.where((s > 0)[..., None], q, 8.0)
    return q.astype(np.uint8).reshape(Mp, Kp), s16


def pack(codes: np.ndarray, scales: np.ndarray):
    """codes uint8 [Mp, Kp], scales float16 [Mp, Kp/128] -> (qw int32 [Mp/16, Kp/64, 32, 4],
    scales float16 [Mp/16, Kp/128, 16])."""
    Mp, Kp = codes.shape
    T, Cn, G = Mp // 16, Kp // 64, Kp // GROUP
    row, k = lane_map()
    u = codes.reshape(T, 16, Cn, 64).astype(np.uint64)
    nib = u[:, row, :, k]                       # [32, 4, 8, T, Cn]
    nib = np.transpose(nib, (3, 4, 0, 1, 2))    # [T, Cn, 32, 4, 8]
    shifts = (4 * np.arange(8)).astype(np.uint64)
    word = (nib << shifts).sum(axis=-1).astype(np.uint32)
    qw = word.view(np.int32).reshape(T, Cn, 32, 4)
    sc = np.ascontiguousarray(np.transpose(scales.reshape(T, 16, G), (0, 2, 1)))
    return np.ascontiguousarray(qw), sc


def unpack(qw: np.ndarray, sc: np.ndarray):
    """Inverse of pack: (codes uint8 [Mp, Kp], scales float16 [Mp, Kp/128])."""
    T, Cn = qw.shape[0], qw.shape[1]
    row, k = lane_map()
    w = qw.view(np.uint32).astype(np.uint64)
    shifts = (4 * np.arange(8)).astype(np.uint64)
    nib = ((w[..., None] >> shifts) & np.uint64(15)).astype(np.uint8)   # [T, Cn, 32, 4, 8]
    codes = np.zeros((T, 16, Cn, 64), dtype=np.uint8)
    codes[:, row, :, k] = np.transpose(nib, (2, 3, 4, 0, 1))
    scales = np.transpose(sc, (0, 2, 1)).reshape(T * 16, -1)
    return codes.reshape(T * 16, Cn * 64), np.ascontiguousarray(scales)


def quantize_w4(W: np.ndarray):
    """W float [M, K] -> dict(qw, scales, M, K, gate_up=False)."""
    M, K = W.shape
    Wp = np.zeros((ceil_to(M, 16), ceil_to(K, GROUP)), dtype=np.float32)
    Wp[:M, :K] = W.astype(np.float32)
    qw, sc = pack(*quantize_codes(Wp))
    return {"qw": qw, "scales": sc, "M": M, "K": K, "gate_up": False}


def quantize_w4_gate_up(Wg: np.ndarray, Wu: np.ndarray):
    I, K = Wg.shape
    Ip = ceil_to(I, 8)
    both = np.zeros((Ip // 8, 2, 8, K), dtype=np.float32)
    g = np.zeros((Ip, K), dtype=np.float32)
    u = np.zeros((Ip, K), dtype=np.float32)
    g[:I], u[:I] = Wg, Wu
    both[:, 0], both[:, 1] = g.reshape(Ip // 8, 8, K), u.reshape(Ip // 8, 8, K)
    p = quantize_w4(both.reshape(2 * Ip, K))
    p.update(M=I, gate_up=True)
    return p


def dequantize(qw: np.ndarray, sc: np.ndarray, M: int, K: int, gate_up: bool = False):
    """float32 [M, K] = (code - 8) * scale, or (gate, up) for an interleaved gate/up pack."""
    codes, scales = unpack(qw, sc)
    Mp, Kp = codes.shape
    w = (codes.astype(np.float32) - 8.0).reshape(Mp, Kp // GROUP, GROUP)
    w = (w * scales.astype(np.float32)[..., None]).reshape(Mp, Kp)
    if gate_up:
        o = w.reshape(Mp // 16, 2, 8, Kp)
        return o[:, 0].reshape(Mp // 2, Kp)[:M, :K].copy(), o[:, 1].reshape(Mp // 2, Kp)[:M, :K].copy()
    return w[:M, :K].copy()
