"""Tensor-parallel path on the GPU.

One-GPU part: the device pieces of the exchange (fp32 partial-sum GEMV, residual norm over gathered
parts, vocabulary-shard argmax + merge) against torch, and the tensor-parallel engine on a group
of one rank, which must reproduce the single-GPU engine bit for bit.
Two-GPU part (skipped on a one-GPU box): ranks over NCCL against the single-GPU engine and the
oracle, speculative output identical to plain output.
"""
from __future__ import annotations

import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent
G = HERE / "golden"
BF16 = torch.bfloat16


# ---------------------------------------------------------------------------------------------
# device pieces
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(512, 1024), (5120, 2176), (1024, 17408)])
@pytest.mark.parametrize("n", [1, 5])
@pytest.mark.parametrize("mode", [-1, 0, 2, 3, 4])
def test_gemv_fp32_partial_equals_rounded_bf16_output(shape, n, mode):
    from qengine_b200 import _w4, synth
    M, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + K + n)
    p = synth.random_w4(M, K, g, "cuda", 0.02)
    x = torch.randn(n, K, generator=g, device="cuda").to(BF16)
    o16 = torch.empty(n, M, dtype=BF16, device="cuda")
    o32 = torch.empty(n, M, dtype=torch.float32, device="cuda")
    _w4.gemv(x, p.qw, p.scales, o16, M, mode=mode)
    _w4.gemv_partial(x, p.qw, p.scales, o32, M, mode=mode)
    assert torch.equal(o32.to(BF16), o16)
    wide = torch.randn(n, 2 * K, generator=g, device="cuda").to(BF16)  # a K slice of a wider row
    wide[:, K:] = x
    _w4.gemv_partial(wide[:, K:], p.qw, p.scales, o32, M, mode=mode)
    assert torch.equal(o32.to(BF16), o16)


@pytest.mark.parametrize("nparts", [1, 2, 8])
@pytest.mark.parametrize("n,H", [(1, 512), (8, 5120), (3, 1000)])
def test_rmsnorm1p_parts(nparts, n, H):
    from qengine_b200 import _C
    g = torch.Generator(device="cuda").manual_seed(nparts * 100 + n)
    x = torch.randn(n, H, generator=g, device="cuda").to(BF16)
    parts = torch.randn(nparts, n, H, generator=g, device="cuda")
    w = (torch.randn(H, generator=g, device="cuda") * 0.1).to(BF16)
    out = torch.empty_like(x)
    x0 = x.clone()
    _C.rmsnorm1p_parts(x, parts, w, out, 1e-6)
    d = parts[0].clone()
    for p in range(1, nparts):
        d += parts[p]
    xr = (x0.float() + d.to(BF16).float()).to(BF16)
    assert torch.equal(x, xr)
    xf = xr.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + w.float())).to(BF16)
    err = (out.float() - ref.float()).abs()
    assert float((err / ref.float().abs().clamp_min(1e-2)).max()) < 2 ** -6
    # one part: the same result as the two-operand norm on the rounded delta
    if nparts == 1:
        x2, out2 = x0.clone(), torch.empty_like(x)
        _C.rmsnorm1p(x2, parts[0].to(BF16), w, out2, 1e-6)
        assert torch.equal(x2, x) and torch.equal(out2, out)


def test_argmax_shards_and_merge():
    from qengine_b200 import _C
    g = torch.Generator(device="cuda").manual_seed(1)
    n, V, t = 6, 4096, 4
    full = torch.randn(n, V, generator=g, device="cuda").to(BF16)
    full[1, [9, 1030, 3000]] = 50.0      # ties across shards: lowest id
    full[2, [2050, 2051]] = 50.0         # tie inside one shard
    full[3] = float("-inf")              # no finite value: id 0
    Vl = V // t
    ws_v = torch.empty(n * 256, device="cuda")
    ws_i = torch.empty(n * 256, dtype=torch.int32, device="cuda")
    vals = torch.empty(t, n, device="cuda")
    idx = torch.empty(t, n, dtype=torch.int32, device="cuda")
    for r in range(t):
        _C.argmax_v(full[:, r * Vl:(r + 1) * Vl], ws_v, ws_i, idx[r], vals[r], base=r * Vl)
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    _C.argmax_merge(vals, idx, out)
    assert out.tolist() == full.float().argmax(-1).tolist()
    assert torch.equal(vals.max(0).values, full.float().max(-1).values)


# ---------------------------------------------------------------------------------------------
# peer-memory exchange kernels on one GPU: the peer is a second local block that the test fills
# (or leaves empty) BEFORE the launch, so no kernel ever waits for another kernel
# ---------------------------------------------------------------------------------------------
class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class _FakeWorld:
    """Communicator of `rank` in a world of `world` ranks whose blocks all live on this GPU."""

    def __init__(self, H, world, rank, timeout_ms=200):
        import ctypes as C
        from qengine_b200._lib import lib
        self.lib, self.H, self.world, self.rank = lib, H, world, rank
        self.nbytes = lib.qe_tp_block_bytes(H, world)
        assert self.nbytes > 0
        self.ptrs = []
        for _ in range(world):
            p = C.c_void_p()
            assert lib.qe_tp_alloc(self.nbytes, C.byref(p)) == 0
            self.ptrs.append(p)
        arr = (C.c_void_p * world)(*[p.value for p in self.ptrs])
        self.comm = C.c_void_p()
        assert lib.qe_tp_comm_create(arr, rank, world, H, C.byref(self.comm)) == 0
        assert lib.qe_tp_set_timeout_ms(self.comm, timeout_ms) == 0
        self.blocks = [torch.as_tensor(_Raw(p.value, self.nbytes), device="cuda") for p in self.ptrs]

    def norm_slot(self, owner, seq, src):
        """int32 view [8 rows, H, 2] of the slot in `owner`'s block that `src` writes for exchange `seq`."""
        off = 4096 + ((seq & 1) * self.world + src) * 8 * self.H * 8
        return self.blocks[owner][off:off + 8 * self.H * 8].view(torch.int32).view(8, self.H, 2)

    def am_slot(self, owner, seq, src):
        off = 256 + ((seq & 1) * 8 + src) * 8 * 16
        return self.blocks[owner][off:off + 8 * 16].view(torch.int32).view(8, 4)

    def error(self):
        import ctypes as C
        info = (C.c_int * 4)()
        return self.lib.qe_tp_error(self.comm, info), list(info)

    def close(self):
        torch.cuda.synchronize()
        self.lib.qe_tp_comm_destroy(self.comm)
        del self.blocks
        for p in self.ptrs:
            self.lib.qe_tp_free(p)


def _norm_ref(x0, parts, w, eps=1e-6):
    d = parts[0].clone()
    for p in parts[1:]:
        d += p
    xr = (x0.float() + d.to(BF16).float()).to(BF16)
    xf = xr.float()
    return xr, (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(BF16)


@pytest.mark.parametrize("H,world,rank", [(512, 2, 0), (5120, 2, 1), (5120, 8, 3), (2048, 4, 0)])
def test_exchange_norm_against_prefilled_peers(H, world, rank):
    from qengine_b200 import _C
    from qengine_b200._lib import lib
    fw = _FakeWorld(H, world, rank)
    g = torch.Generator(device="cuda").manual_seed(H + world)
    w = (torch.randn(H, generator=g, device="cuda") * 0.1).to(BF16)
    s = torch.cuda.current_stream().cuda_stream
    try:
        for seq, n in [(1, 1), (2, 5), (3, 8), (4, 1)]:  # rows 1..: each row has its own sequence number
            x = torch.randn(n, H, generator=g, device="cuda").to(BF16)
            parts = [torch.randn(n, H, generator=g, device="cuda") for _ in range(world)]
            x0, out = x.clone(), torch.empty_like(x)
            # per-row sequence numbers differ (row 0 took part in every exchange, row 7 in one)
            seqs = [sum(1 for (q, m) in [(1, 1), (2, 5), (3, 8), (4, 1)][:seq] if r < m) for r in range(n)]
            for src in range(world):
                if src == rank:
                    continue
                for r in range(n):
                    sl = fw.norm_slot(rank, seqs[r], src)
                    sl[r, :, 0] = parts[src][r].view(torch.int32)
                    sl[r, :, 1] = seqs[r]
            torch.cuda.synchronize()
            out16 = torch.empty(n, H, dtype=torch.float16, device="cuda")
            assert lib.qe_tp_exchange_norm(fw.comm, x.data_ptr(), parts[rank].data_ptr(), w.data_ptr(), out.data_ptr(),
                                           out16.data_ptr(), n, x.stride(0), parts[rank].stride(0), out.stride(0),
                                           out16.stride(0), 1e-6, s) == 0
            assert fw.error()[0] == 0
            assert torch.equal(out16.float(), out.float()), "the fp16 copy of the normed rows"
            xr, ref = _norm_ref(x0, parts, w)
            assert torch.equal(x, xr)
            # the norm over gathered parts (library-collective transport) sums the squares in another
            # order: same residual rows, normed rows within one ulp; every peer received our row
            from util import bf16_ulp_close
            x2, out2 = x0.clone(), torch.empty_like(x)
            _C.rmsnorm1p_parts(x2, torch.stack(parts), w, out2, 1e-6)
            assert torch.equal(x, x2) and bf16_ulp_close(out, out2, ulps=1)[0]
            assert float(((out.float() - ref.float()).abs() / ref.float().abs().clamp_min(1e-2)).max()) < 2 ** -6
            for peer in range(world):
                if peer == rank:
                    continue
                for r in range(n):
                    got = fw.norm_slot(peer, seqs[r], rank)[r]
                    assert torch.equal(got[:, 0], parts[rank][r].view(torch.int32)) and bool((got[:, 1] == seqs[r]).all())
    finally:
        fw.close()


def test_exchange_argmax_against_prefilled_peers():
    from qengine_b200._lib import lib
    world, rank, n = 4, 2, 6
    fw = _FakeWorld(512, world, rank)
    s = torch.cuda.current_stream().cuda_stream
    try:
        vals = torch.tensor([[1.0, 5.0, 2.0, float("-inf"), 3.0, 0.5],
                             [4.0, 5.0, 2.0, float("-inf"), float("nan"), 0.5],
                             [2.0, 5.0, 7.0, float("-inf"), 9.0, 0.5],
                             [3.0, 1.0, 7.0, float("-inf"), 1.0, 0.25]], device="cuda")
        idx = (torch.arange(world, device="cuda", dtype=torch.int32)[:, None] * 1000
               + torch.tensor([5, 6, 7, 0, 9, 1], device="cuda", dtype=torch.int32)[None])
        for seq in (1, 2, 3):
            for src in range(world):
                if src != rank:
                    sl = fw.am_slot(rank, seq, src)
                    sl[:n, 0] = vals[src].view(torch.int32)
                    sl[:n, 2] = idx[src]
                    sl[:n, 1] = seq
                    sl[:n, 3] = seq
            out = torch.full((8,), -1, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            assert lib.qe_tp_exchange_argmax(fw.comm, vals[rank].contiguous().data_ptr(), idx[rank].contiguous().data_ptr(),
                                             n, out.data_ptr(), s) == 0
            assert fw.error()[0] == 0
            #            max 4.0@r1  tie 5.0 -> rank 0   tie 7.0 -> rank 2   all -inf -> first   NaN wins   tie -> rank 0
            assert out[:n].tolist() == [1005, 6, 2007, 0, 1009, 1]
            for peer in range(world):
                if peer != rank:
                    got = fw.am_slot(peer, seq, rank)[:n]
                    assert torch.equal(got[:, 2], idx[rank]) and bool((got[:, 1] == seq).all())
    finally:
        fw.close()


def test_exchange_wait_runs_out_and_reports_the_late_rank():
    """Failure detection without a fault: the peer's slot is never filled, the bounded wait gives
    up, the kernel returns, the error word names the late rank, and the context stays usable."""
    import time
    from qengine_b200._lib import lib
    H = 512
    fw = _FakeWorld(H, 2, 0, timeout_ms=50)
    s = torch.cuda.current_stream().cuda_stream
    try:
        x = torch.ones(1, H, device="cuda", dtype=BF16)
        part = torch.ones(1, H, device="cuda")
        w = torch.zeros(H, device="cuda", dtype=BF16)
        out = torch.empty_like(x)
        args = (fw.comm, x.data_ptr(), part.data_ptr(), w.data_ptr(), out.data_ptr(), None, 1, H, H, H, 0, 1e-6, s)
        t0 = time.perf_counter()
        assert lib.qe_tp_exchange_norm(*args) == 0
        err, info = fw.error()
        dt = time.perf_counter() - t0
        assert err == 1 and info[1:] == [1, 0, 0], (err, info)
        assert 0.04 < dt < 2.0, dt
        t0 = time.perf_counter()               # sticky: later exchanges do not spin at all
        for _ in range(20):
            assert lib.qe_tp_exchange_norm(*args) == 0
        assert fw.error()[0] == 1
        assert time.perf_counter() - t0 < 0.04
        assert lib.qe_tp_clear_error(fw.comm) == 0 and fw.error()[0] == 0
        assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0   # context still usable
    finally:
        fw.close()


# ---------------------------------------------------------------------------------------------
# engine under torch.distributed
# ---------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, *extra):
    for p in (str(HERE), str(HERE.parent)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import os
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    import threading
    fn(rank, world, *extra)
    torch.cuda.synchronize()
    dist.barrier()
    # a teardown that stalls (graphs holding collectives) must not hold the GPUs: leave after 20 s
    threading.Timer(20.0, lambda: os._exit(0)).start()
    dist.destroy_process_group()
    os._exit(0)


def _spawn(fn, world, *extra):
    import torch.multiprocessing as mp
    mp.spawn(_entry, args=(world, _free_port(), fn) + extra, nprocs=world, join=True)


def _gather_cols(local):
    import torch.distributed as dist
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=-1)


def _engine_worker(rank, world, transport, small8=False):
    from oracle import model as OM
    from qengine_b200 import synth, tp
    from qengine_b200.engine import Engine
    from util import cosine, dense_model, oracle_config
    cfg = synth.shardable8_config() if small8 else synth.tiny_config()
    Wp = synth.build_model(cfg, seed=7, device="cpu", scale_std=0.01)
    W = synth.model_to(Wp, "cuda")
    eng = Engine(cfg, tp.shard_model(W, cfg, world, rank), max_len=256, tp=tp.TPGroup(transport=transport))
    if small8:  # no stored continuation for this configuration: a seeded prompt, teacher-forced
        prompt = synth.prompt_ids(32, cfg.vocab, seed=1234)
        seq = prompt + synth.prompt_ids(8, cfg.vocab, seed=4321)
    else:
        g = torch.load(G / "greedy.pt")
        prompt, seq = g["prompt"], (g["prompt"] + g["tokens"])[:40]

    lg = _gather_cols(eng.sequence_logits(seq))
    hid, mlg_l = eng.mtp_rows_logits(seq[:12])
    mlg = _gather_cols(mlg_l)
    plain = eng.generate(prompt, 40)
    for k in (1, 3, 4):
        assert eng.generate_spec(prompt, 40, k) == plain, k          # rollback exact under TP
    for a in (0, 2, 4):
        got = eng.generate_spec(prompt, 40, 4, force_accept=a, truth=prompt + plain + [0] * 16)
        assert got == plain, a
    assert eng.generate(prompt, 40) == plain                          # run-to-run identical
    dv = Engine(cfg, tp.shard_model(W, cfg, world, rank), max_len=256, tp=tp.TPGroup(transport=transport),
                draft_vocab=1024)
    assert dv.generate_spec(prompt, 40, 3) == plain
    assert eng.tp.error() is None and dv.tp.error() is None

    # every rank must hold the same tokens (control words are replicated, never exchanged)
    import torch.distributed as dist
    mine = torch.tensor(plain, device="cuda")
    allp = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allp, mine)
    assert all(torch.equal(a, mine) for a in allp)

    if rank == 0:
        # fuse=False: the same kernels as the tensor-parallel engine (norm as a launch of its own);
        # the fused single-GPU engine computes the norm statistics in another order (1 ulp)
        one = Engine(cfg, W, max_len=256, fuse=False)
        ref_lg = one.sequence_logits(seq)
        _, ref_mlg = one.mtp_rows_logits(seq[:12])
        ref_plain = one.generate(prompt, 40)
        if world == 1 and transport == "nccl":  # same kernels, no exchange: the same bits
            assert torch.equal(lg, ref_lg) and torch.equal(mlg, ref_mlg) and plain == ref_plain
        cs = min(cosine(lg[t], ref_lg[t]) for t in range(len(seq)))
        cm = min(cosine(mlg[t], ref_mlg[t]) for t in range(12))
        agree = sum(int(lg[t].float().argmax()) == int(ref_lg[t].float().argmax()) for t in range(len(seq)))
        same = next((i for i, (a, b) in enumerate(zip(plain, ref_plain)) if a != b), len(plain))
        print(f"\nTP={world} ({transport}) vs single GPU: min cosine logits {cs:.6f}, mtp {cm:.6f}, top-1 {agree}/{len(seq)}, "
              f"greedy identical for {same}/40 tokens")
        assert cs >= 0.9999 and cm >= 0.9999 and agree >= len(seq) - 1
        D, oc = dense_model(Wp), oracle_config(cfg)
        st = OM.State(oc, 64)
        worst = 1.0
        for t, tok in enumerate(seq):
            ref, _ = OM.decode_step(D, st, tok, oc, fused_swiglu=True)
            worst = min(worst, cosine(lg[t].cpu(), ref))
        print(f"TP={world} vs oracle: min cosine {worst:.6f}")
        assert worst >= 0.9999


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_tp_engine_group_of_one(transport):
    """One rank: with the library-collective transport the kernels are those of the unfused single-GPU
    engine (bit-identical); the peer transport's exchange kernel sums the squares of the norm in its
    own order (cosine, token checks)."""
    _spawn(_engine_worker, 1, transport)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_tp_engine_two_gpus(transport):
    _spawn(_engine_worker, 2, transport)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp_engine_four_gpus_shared_kv_heads():
    _spawn(_engine_worker, 4, "peer")  # tiny model: 2 KV heads over 4 ranks


def test_tp_engine_shardable8_config_group_of_one():
    """The 8-way shardable configuration through the same checks on one GPU (logits vs the single-GPU
    engine and the oracle, speculative == plain), so that the 8-GPU test below differs only in t."""
    _spawn(_engine_worker, 1, "peer", True)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp_engine_eight_gpus():
    _spawn(_engine_worker, 8, "peer", True)  # 4 KV heads over 8 ranks: each shared by a pair
