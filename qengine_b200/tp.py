"""Tensor parallelism for the decode path: one process per GPU, `torch.distributed` (NCCL over
NVLink) for the exchanges. The reference is single-GPU; this layer follows the model's natural
shards:

  in_proj      split by heads (DeltaNet: q/k heads and value heads in the same ratio, so value head
               j still reads q/k head j // r locally; attention: query heads, KV heads split up to
               Hkv ranks and shared by t / Hkv ranks beyond), rows re-fused per rank
  out / o_proj, down, mtp.fc   split along K -> fp32 partial sums, one exchange each
  gate_up      split by output tiles (8 outputs per tile), matching down's K slices
  lm_head      split by vocabulary rows -> local argmax -> exchange of (value, index)
  norms, embedding, control words   replicated; accept / commit run redundantly on every rank

Exchange = all-gather of the ranks' fp32 partial rows followed by a fixed-order sum fused into the
consuming RMSNorm (`_C.rmsnorm1p_parts`): deterministic and independent of how many rows a pass has,
which a ring all-reduce is not.
"""
from __future__ import annotations

from dataclasses import replace

import torch

from .quant import GROUP, W4Packed, pack_codes, unpack_codes
from .synth import Config


def local_config(cfg: Config, t: int) -> Config:
    """Per-rank shapes. `vocab` becomes the local slice; `hidden` stays whole."""
    assert cfg.hk % t == 0 and cfg.hv % t == 0 and cfg.hq % t == 0 and cfg.inter % (8 * t) == 0
    assert cfg.vocab % (16 * t) == 0 and (cfg.hkv % t == 0 or t % cfg.hkv == 0)
    return replace(cfg, hk=cfg.hk // t, hv=cfg.hv // t, hq=cfg.hq // t, hkv=max(1, cfg.hkv // t),
                   inter=cfg.inter // t, vocab=cfg.vocab // t)


# ---------------------------------------------------------------------------------------------
# Shards of packed matrices
# ---------------------------------------------------------------------------------------------
def select_rows(p: W4Packed, rows: torch.Tensor) -> W4Packed:
    """Packed matrix made of the given output rows of `p` (any order), padded to 16 rows."""
    assert not p.gate_up
    codes, scales = unpack_codes(p)
    rows = rows.to(codes.device)
    M = rows.numel()
    Mp = -(-M // 16) * 16
    c = torch.full((Mp, codes.shape[1]), 8, dtype=torch.uint8, device=codes.device)
    s = torch.zeros(Mp, scales.shape[1], dtype=scales.dtype, device=codes.device)
    c[:M], s[:M] = codes[rows], scales[rows]
    return pack_codes(c, s, M, p.K)


def slice_tiles(p: W4Packed, t0: int, t1: int) -> W4Packed:
    """Rows of 16-row tiles [t0, t1) (for a gate/up pack: outputs 8 t0 .. 8 t1)."""
    rows = (t1 - t0) * (8 if p.gate_up else 16)
    return W4Packed(p.qw[t0:t1].contiguous(), p.scales[t0:t1].contiguous(), rows, p.K, p.gate_up)


def slice_k(p: W4Packed, k0: int, k1: int) -> W4Packed:
    """Columns [k0, k1) of the reduction dimension (multiples of the group size)."""
    assert k0 % GROUP == 0 and k1 % GROUP == 0 and not p.gate_up
    return W4Packed(p.qw[:, k0 // 64:k1 // 64].contiguous(), p.scales[:, k0 // GROUP:k1 // GROUP].contiguous(),
                    p.M, k1 - k0)


def _arange(a, b, dev):
    return torch.arange(a, b, device=dev)


def shard_layer(L: dict, cfg: Config, t: int, g: int) -> dict:
    """Rank g's shard of one decoder (or MTP) layer dict."""
    dev = L["in_proj"].qw.device
    lc = local_config(cfg, t)
    S = {k: v for k, v in L.items() if k not in ("in_proj", "out", "gate_up", "down", "conv_w", "A_log", "dt_bias", "fc")}
    if L["type"] == "linear_attention":
        D, kd = cfg.dk, cfg.key_dim
        q = _arange(g * lc.hk * D, (g + 1) * lc.hk * D, dev)
        v = _arange(g * lc.hv * cfg.dv, (g + 1) * lc.hv * cfg.dv, dev)
        hv = _arange(g * lc.hv, (g + 1) * lc.hv, dev)
        conv_rows = torch.cat([q, kd + q, 2 * kd + v])
        c0, c1 = cfg.conv_dim, cfg.conv_dim + cfg.value_dim
        rows = torch.cat([conv_rows, c0 + v, c1 + hv, c1 + cfg.hv + hv])
        S["in_proj"] = select_rows(L["in_proj"], rows)
        S["conv_w"] = L["conv_w"][conv_rows].contiguous()
        S["A_log"], S["dt_bias"] = L["A_log"][hv].contiguous(), L["dt_bias"][hv].contiguous()
        S["out"] = slice_k(L["out"], g * lc.hv * cfg.dv, (g + 1) * lc.hv * cfg.dv)
    else:
        hd = cfg.head_dim
        q0 = cfg.hq * 2 * hd
        k1 = q0 + cfg.hkv * hd
        qrows = _arange(g * lc.hq * 2 * hd, (g + 1) * lc.hq * 2 * hd, dev)
        if t <= cfg.hkv:
            kv = _arange(g * lc.hkv * hd, (g + 1) * lc.hkv * hd, dev)
        else:  # a KV head is shared by t / Hkv consecutive ranks
            head = g // (t // cfg.hkv)
            kv = _arange(head * hd, (head + 1) * hd, dev)
        S["in_proj"] = select_rows(L["in_proj"], torch.cat([qrows, q0 + kv, k1 + kv]))
        S["out"] = slice_k(L["out"], g * lc.hq * hd, (g + 1) * lc.hq * hd)
    tiles = L["gate_up"].qw.shape[0]
    S["gate_up"] = slice_tiles(L["gate_up"], g * tiles // t, (g + 1) * tiles // t)
    S["down"] = slice_k(L["down"], g * lc.inter, (g + 1) * lc.inter)
    if "fc" in L:
        H2 = L["fc"].K
        S["fc"] = slice_k(L["fc"], g * H2 // t, (g + 1) * H2 // t)
    return S


def shard_model(W: dict, cfg: Config, t: int, g: int) -> dict:
    """Rank g's shard of a weights dict (see qengine_b200.synth.build_model)."""
    tiles = W["lm_head"].qw.shape[0]
    return {"embed": W["embed"], "final_norm": W["final_norm"],
            "lm_head": slice_tiles(W["lm_head"], g * tiles // t, (g + 1) * tiles // t),
            "layers": [shard_layer(L, cfg, t, g) for L in W["layers"]],
            "mtp": shard_layer(W["mtp"], cfg, t, g) if W.get("mtp") else None}


def build_sharded_model(cfg: Config, t: int, g: int, seed=0, device="cuda", scale_std=0.01, mtp=True) -> dict:
    """Same weights as synth.build_model(cfg, seed, ...) but only rank g's shard is kept: every
    full matrix is generated (same seeds, same order), sharded and dropped layer by layer."""
    from . import synth
    S = synth._Seeds(seed, device)
    dev = S.device
    W = {"embed": synth._small((cfg.vocab, cfg.hidden), S.gen(), dev, 1.0),
         "final_norm": synth._small((cfg.hidden,), S.gen(), dev, 0.1)}
    head = synth.random_w4(cfg.vocab, cfg.hidden, S.gen(), dev, scale_std)
    tiles = head.qw.shape[0]
    W["lm_head"] = slice_tiles(head, g * tiles // t, (g + 1) * tiles // t)
    del head
    W["layers"] = []
    for kind in cfg.layer_types:
        W["layers"].append(shard_layer(synth._layer(cfg, kind, S, scale_std), cfg, t, g))
    W["mtp"] = None
    if mtp and cfg.mtp_layers > 0:
        Mt = synth._layer(cfg, "full_attention", S, scale_std)
        Mt["fc"] = synth.random_w4(cfg.hidden, 2 * cfg.hidden, S.gen(), dev, scale_std)
        Mt["norm"] = synth._small((cfg.hidden,), S.gen(), dev, 0.1)
        Mt["pre_e"] = synth._small((cfg.hidden,), S.gen(), dev, 0.1)
        Mt["pre_h"] = synth._small((cfg.hidden,), S.gen(), dev, 0.1)
        W["mtp"] = shard_layer(Mt, cfg, t, g)
    return W


# ---------------------------------------------------------------------------------------------
# Communicator
# ---------------------------------------------------------------------------------------------
class TPGroup:
    """Rank, size and the exchanges of the decode path over a torch.distributed process group.

    transport "peer" (default): the library's own exchange kernels over NVLink peer memory
    (qe_tp_exchange_norm / qe_tp_exchange_argmax): one launch per exchange, fused with the
    consuming norm; the process group is only used once, on the host, to swap the IPC handles of
    the exchange blocks. transport "nccl": all-gather through torch.distributed followed by
    `_C.rmsnorm1p_parts` / `_C.argmax_merge` (the library-collective baseline).
    All calls enqueue on the current CUDA stream and can be captured in CUDA graphs."""

    def __init__(self, group=None, transport: str = "peer", timeout_ms: int | None = None):
        import torch.distributed as dist
        assert transport in ("peer", "nccl")
        self.dist, self.group, self.transport = dist, group, transport
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.timeout_ms = timeout_ms
        self.comm = self._block = None
        self._maps = []

    # -- peer transport -------------------------------------------------------------------------
    def open(self, hidden: int):
        """Allocate this rank's exchange block, map every peer's (CUDA IPC) and build the
        communicator. Collective: every rank of the group must call it."""
        import ctypes as C
        from ._lib import check, lib
        if self.comm is not None or self.transport != "peer":
            return
        nbytes = lib.qe_tp_block_bytes(int(hidden), self.size)
        if nbytes < 0:
            raise RuntimeError(f"tensor parallel exchange: hidden {hidden} / world {self.size} not supported")
        blk = C.c_void_p()
        check(lib.qe_tp_alloc(nbytes, C.byref(blk)), "tp alloc", kernels=0)
        handle = (C.c_ubyte * 64)()
        check(lib.qe_tp_export(blk, handle), "tp export", kernels=0)
        handles = [None] * self.size
        self.dist.all_gather_object(handles, bytes(handle), group=self.group)
        blocks = (C.c_void_p * self.size)()
        for r, h in enumerate(handles):
            if r == self.rank:
                blocks[r] = blk.value
            else:
                m = C.c_void_p()
                check(lib.qe_tp_import((C.c_ubyte * 64).from_buffer_copy(h), C.byref(m)), "tp import", kernels=0)
                blocks[r] = m.value
                self._maps.append(m)
        comm = C.c_void_p()
        check(lib.qe_tp_comm_create(blocks, self.rank, self.size, int(hidden), C.byref(comm)), "tp comm", kernels=0)
        if self.timeout_ms:
            check(lib.qe_tp_set_timeout_ms(comm, int(self.timeout_ms)), "tp timeout", kernels=0)
        self._block, self.comm = blk, comm
        self.dist.barrier(group=self.group)  # nobody pushes before every block is mapped

    def close(self):
        """Collective: unmap the peers' blocks, then free our own."""
        from ._lib import lib
        if self.comm is None:
            return
        torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        for m in self._maps:
            lib.qe_tp_unmap(m)
        self._maps = []
        self.dist.barrier(group=self.group)
        lib.qe_tp_comm_destroy(self.comm)
        lib.qe_tp_free(self._block)
        self.comm = self._block = None

    def error(self):
        """Sticky error word of the peer transport after a device sync: None, or a dict naming the
        rank that was late."""
        import ctypes as C
        from ._lib import lib
        if self.comm is None:
            return None
        info = (C.c_int * 4)()
        e = lib.qe_tp_error(self.comm, info)
        if e == 0:
            return None
        return {"error": e, "late_rank": info[1], "row": info[2], "kind": "argmax" if info[3] else "norm"}

    def exchange_norm(self, x, part, w, out, eps, out16=None):
        """x += bf16(sum over ranks of part); out = rmsnorm1p(x) -- one launch. out16 (fp16, same
        shape, optional) receives the normed rows as fp16 as well."""
        from ._lib import check, lib
        assert part.dtype == torch.float32 and part.stride(1) == 1 and x.stride(1) == 1 and out.stride(1) == 1
        assert x.shape == part.shape == out.shape
        assert out16 is None or (out16.dtype == torch.float16 and out16.shape == out.shape and out16.stride(1) == 1)
        check(lib.qe_tp_exchange_norm(self.comm, x.data_ptr(), part.data_ptr(), w.data_ptr(), out.data_ptr(),
                                      out16.data_ptr() if out16 is not None else None,
                                      x.shape[0], x.stride(0), part.stride(0), out.stride(0),
                                      out16.stride(0) if out16 is not None else 0, float(eps),
                                      torch.cuda.current_stream().cuda_stream), "tp exchange_norm")

    def exchange_argmax(self, cand_v, cand_i, rows, out):
        from ._lib import check, lib
        check(lib.qe_tp_exchange_argmax(self.comm, cand_v.data_ptr(), cand_i.data_ptr(), int(rows), out.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream), "tp exchange_argmax")

    # -- library collective -----------------------------------------------------------------------
    def all_gather(self, out: torch.Tensor, inp: torch.Tensor):
        self.dist.all_gather_into_tensor(out, inp, group=self.group)

    def barrier(self):
        self.dist.barrier(group=self.group)
