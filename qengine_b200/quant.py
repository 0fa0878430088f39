"""W4 wire format: int4 symmetric round-to-nearest quantiser and packer, group 128 along K, one
fp16 scale per (row, group). This is the format qe_w4_gemv reads; it is the reference's format
(python/qengine/quant.py:1-30, 41-148) so packed checkpoints are interchangeable.

    scale[m, g] = fp16(2 * max|W[m, 128g:128g+128]| / 15)
    u[m, k]     = clamp(round(W[m, k] / scale) + 8, 0, 15)       stored nibble
    W~[m, k]    = (u - 8) * scale                                 what the kernel multiplies

    qw     int32 [Mp/16, Kp/64, 32, 4]    Mp = ceil16(M), Kp = ceil128(K), padding nibble 8
    scales fp16  [Mp/16, Kp/128, 16]

Bit layout of one 32-bit word, for tile T, chunk c, lane = 4 r + t, word s:
nibble j = j0 + 2 j1 + 4 j2 holds row 16 T + r + 8 j0 and k = 64 c + 16 t + 4 s + 2 j1 + j2.
The packer below builds the words with a reshape of the code matrix to
[T, j0, r, c, t, s, j1, j2] and a weighted sum over (j0, j1, j2); no gather is involved.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

GROUP = 128


def _ceil(a: int, b: int) -> int:
    return -(-a // b) * b


@dataclass
class W4Packed:
    qw: torch.Tensor      # int32 [Mp/16, Kp/64, 32, 4]
    scales: torch.Tensor  # fp16  [Mp/16, Kp/128, 16]
    M: int                # logical rows (gate_up: intermediate size I)
    K: int
    gate_up: bool = False

    @property
    def nbytes(self) -> int:
        return self.qw.numel() * 4 + self.scales.numel() * 2

    def to(self, device) -> "W4Packed":
        return W4Packed(self.qw.to(device), self.scales.to(device), self.M, self.K, self.gate_up)


def _nibble_weights(device) -> torch.Tensor:
    """2^(4 j) for j = j0 + 2 j1 + 4 j2, shaped [j0, j1, j2] (int64)."""
    j0 = torch.arange(2, device=device).view(2, 1, 1)
    j1 = torch.arange(2, device=device).view(1, 2, 1)
    j2 = torch.arange(2, device=device).view(1, 1, 2)
    return torch.ones((), dtype=torch.int64, device=device) << (4 * (j0 + 2 * j1 + 4 * j2))


def pack_codes(codes: torch.Tensor, scales: torch.Tensor, M: int, K: int, gate_up: bool = False) -> W4Packed:
    """Pack given nibbles. codes: integer [Mp, Kp] in 0..15 (padding must be 8); scales: fp16
    [Mp, Kp/128]."""
    Mp, Kp = codes.shape
    assert Mp % 16 == 0 and Kp % GROUP == 0 and scales.shape == (Mp, Kp // GROUP)
    T, Cn = Mp // 16, Kp // 64
    u = codes.to(torch.int64).view(T, 2, 8, Cn, 4, 4, 2, 2)        # T j0 r c t s j1 j2
    u = u.permute(0, 3, 2, 4, 5, 1, 6, 7)                            # T c r t s j0 j1 j2
    word = (u * _nibble_weights(codes.device)).sum(dim=(-1, -2, -3))  # [T, c, r, t, s]
    word = torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
    qw = word.reshape(T, Cn, 32, 4).contiguous()
    sc = scales.to(torch.float16).view(T, 16, Kp // GROUP).permute(0, 2, 1).contiguous()
    return W4Packed(qw, sc, M, K, gate_up)


def unpack_codes(p: W4Packed) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of pack_codes: (codes uint8 [Mp, Kp], scales fp16 [Mp, Kp/128])."""
    T, Cn = p.qw.shape[0], p.qw.shape[1]
    dev = p.qw.device
    w = (p.qw.to(torch.int64) & 0xFFFFFFFF).view(T, Cn, 8, 4, 4)     # T c r t s
    j0 = torch.arange(2, device=dev).view(2, 1, 1)
    j1 = torch.arange(2, device=dev).view(1, 2, 1)
    j2 = torch.arange(2, device=dev).view(1, 1, 2)
    sh = 4 * (j0 + 2 * j1 + 4 * j2)
    nib = (w[..., None, None, None] >> sh) & 0xF                       # T c r t s j0 j1 j2
    codes = nib.permute(0, 5, 2, 1, 3, 4, 6, 7).reshape(T * 16, Cn * 64).to(torch.uint8)
    scales = p.scales.permute(0, 2, 1).reshape(T * 16, -1)
    return codes, scales


@torch.no_grad()
def _quantize_rows(Wp: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Wp fp32 [rows, Kp] -> (codes uint8 [rows, Kp], scales fp16 [rows, Kp/128])."""
    rows, Kp = Wp.shape
    g = Wp.view(rows, Kp // GROUP, GROUP)
    s16 = (g.abs().amax(dim=-1) * (2.0 / 15.0)).to(torch.float16)
    s = s16.float()
    live = s > 0
    q = torch.round(g / torch.where(live, s, torch.ones_like(s)).unsqueeze(-1)) + 8
    q = torch.where(live.unsqueeze(-1), q.clamp_(0, 15), torch.full_like(q, 8.0))
    return q.to(torch.uint8).view(rows, Kp), s16


@torch.no_grad()
def _quantize_pack(W: torch.Tensor, M: int, K: int, gate_up: bool, rows_per_step: int = 4096) -> W4Packed:
    Mp, Kp = _ceil(W.shape[0], 16), _ceil(K, GROUP)
    dev = W.device
    qw = torch.empty(Mp // 16, Kp // 64, 32, 4, dtype=torch.int32, device=dev)
    sc = torch.empty(Mp // 16, Kp // GROUP, 16, dtype=torch.float16, device=dev)
    for r0 in range(0, Mp, rows_per_step):  # bounded memory for the 248,320-row head
        r1 = min(Mp, r0 + rows_per_step)
        Wp = torch.zeros(r1 - r0, Kp, dtype=torch.float32, device=dev)
        if r0 < W.shape[0]:
            blk = W[r0:min(r1, W.shape[0]), :K].float()
            Wp[:blk.shape[0], :K] = blk
        codes, s16 = _quantize_rows(Wp)
        part = pack_codes(codes, s16, 0, 0)
        qw[r0 // 16:r1 // 16] = part.qw
        sc[r0 // 16:r1 // 16] = part.scales
    return W4Packed(qw, sc, M, K, gate_up)


def quantize_w4(W: torch.Tensor) -> W4Packed:
    """RTN symmetric int4, group 128 along K, fp16 scales. W: [M, K], any float dtype."""
    assert W.dim() == 2
    return _quantize_pack(W, W.shape[0], W.shape[1], False)


def interleave_gate_up(Wg: torch.Tensor, Wu: torch.Tensor) -> torch.Tensor:
    """Rows in blocks of 8: tile T rows 0..7 = gate[8T..8T+7], rows 8..15 = up[8T..8T+7]
    (zero rows pad I to a multiple of 8), so a lane of the GEMV holds gate and up of one output."""
    assert Wg.shape == Wu.shape and Wg.dim() == 2
    I, K = Wg.shape
    Ip = _ceil(I, 8)
    both = torch.zeros(Ip // 8, 2, 8, K, dtype=Wg.dtype, device=Wg.device)
    g = torch.zeros(Ip, K, dtype=Wg.dtype, device=Wg.device)
    u = torch.zeros(Ip, K, dtype=Wg.dtype, device=Wg.device)
    g[:I], u[:I] = Wg, Wu
    both[:, 0], both[:, 1] = g.view(Ip // 8, 8, K), u.view(Ip // 8, 8, K)
    return both.view(2 * Ip, K)


def quantize_w4_gate_up(Wg: torch.Tensor, Wu: torch.Tensor) -> W4Packed:
    """Pack gate [I, K] and up [I, K] for gemv_swiglu (out = silu(x Wg^T) * x Wu^T)."""
    I, K = Wg.shape
    return _quantize_pack(interleave_gate_up(Wg, Wu), I, K, True)


@torch.no_grad()
def dequantize_w4(p: W4Packed):
    """fp32 weights the kernel effectively multiplies with: [M, K], or (gate, up) each [I, K]."""
    codes, scales = unpack_codes(p)
    Mp, Kp = codes.shape
    w = (codes.float() - 8.0).view(Mp, Kp // GROUP, GROUP) * scales.float().unsqueeze(-1)
    w = w.view(Mp, Kp)
    if p.gate_up:
        o = w.view(Mp // 16, 2, 8, Kp)
        return (o[:, 0].reshape(Mp // 2, Kp)[:p.M, :p.K].contiguous(),
                o[:, 1].reshape(Mp // 2, Kp)[:p.M, :p.K].contiguous())
    return w[:p.M, :p.K].contiguous()


def gemv(x: torch.Tensor, p: W4Packed, out: torch.Tensor | None = None, **kw) -> torch.Tensor:
    """out[N, M] = x[N, K] @ W~^T, or silu(gate) * up for gate_up packs, through `_w4`."""
    from . import _w4

    if out is None:
        out = torch.empty(x.shape[0], p.M, dtype=torch.bfloat16, device=x.device)
    (_w4.gemv_swiglu if p.gate_up else _w4.gemv)(x, p.qw, p.scales, out, p.M, **kw)
    return out


def gemm(x: torch.Tensor, p: W4Packed, out: torch.Tensor | None = None, **kw) -> torch.Tensor:
    """The same product for up to 64 rows with the matrix read once (`_w4.gemm`; prefill passes)."""
    from . import _w4

    if out is None:
        out = torch.empty(x.shape[0], p.M, dtype=torch.bfloat16, device=x.device)
    _w4.gemm(x, p.qw, p.scales, out, p.M, swiglu=p.gate_up, **kw)
    return out
