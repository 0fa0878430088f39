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
    _w4.gemv_act16(x, p.qw, p.scales, o32, M, mode=mode)
    assert torch.equal(o32.to(BF16), o16)
    wide = torch.randn(n, 2 * K, generator=g, device="cuda").to(BF16)  # a K slice of a wider row
    wide[:, K:] = x
    _w4.gemv_act16(wide[:, K:], p.qw, p.scales, o32, M, mode=mode)
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
# engine under torch.distributed
# ---------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn):
    for p in (str(HERE), str(HERE.parent)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import os
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        fn(rank, world)
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _spawn(fn, world):
    import torch.multiprocessing as mp
    mp.spawn(_entry, args=(world, _free_port(), fn), nprocs=world, join=True)


def _gather_cols(local):
    import torch.distributed as dist
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=-1)


def _engine_worker(rank, world):
    from oracle import model as OM
    from qengine_b200 import synth, tp
    from qengine_b200.engine import Engine
    from util import cosine, dense_model, oracle_config
    cfg = synth.tiny_config()
    Wp = synth.build_model(cfg, seed=7, device="cpu", scale_std=0.01)
    W = synth.model_to(Wp, "cuda")
    eng = Engine(cfg, tp.shard_model(W, cfg, world, rank), max_len=256, tp=tp.TPGroup())
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
    dv = Engine(cfg, tp.shard_model(W, cfg, world, rank), max_len=256, tp=tp.TPGroup(), draft_vocab=1024)
    assert dv.generate_spec(prompt, 40, 3) == plain

    # every rank must hold the same tokens (control words are replicated, never exchanged)
    import torch.distributed as dist
    mine = torch.tensor(plain, device="cuda")
    allp = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allp, mine)
    assert all(torch.equal(a, mine) for a in allp)

    if rank == 0:
        one = Engine(cfg, W, max_len=256)
        ref_lg = one.sequence_logits(seq)
        _, ref_mlg = one.mtp_rows_logits(seq[:12])
        ref_plain = one.generate(prompt, 40)
        if world == 1:  # a group of one rank adds the exchange but no arithmetic
            assert torch.equal(lg, ref_lg) and torch.equal(mlg, ref_mlg) and plain == ref_plain
        cs = min(cosine(lg[t], ref_lg[t]) for t in range(len(seq)))
        cm = min(cosine(mlg[t], ref_mlg[t]) for t in range(12))
        agree = sum(int(lg[t].float().argmax()) == int(ref_lg[t].float().argmax()) for t in range(len(seq)))
        same = next((i for i, (a, b) in enumerate(zip(plain, ref_plain)) if a != b), len(plain))
        print(f"\nTP={world} vs single GPU: min cosine logits {cs:.6f}, mtp {cm:.6f}, top-1 {agree}/{len(seq)}, "
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


def test_tp_engine_group_of_one_is_bit_identical():
    _spawn(_engine_worker, 1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_engine_two_gpus():
    _spawn(_engine_worker, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp_engine_four_gpus_shared_kv_heads():
    _spawn(_engine_worker, 4)  # tiny model: 2 KV heads over 4 ranks
