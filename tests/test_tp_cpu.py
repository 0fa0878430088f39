"""Tensor-parallel host logic on the CPU: shard construction, and a world_size-2 `gloo` run of the
sharded oracle step against the unsharded oracle (same seeded tiny model)."""
from __future__ import annotations

import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import model as OM
from qengine_b200 import quant as Q
from qengine_b200 import synth, tp
from util import cosine, dense_model, dequant_oracle, oracle_config

HERE = Path(__file__).resolve().parent
SEED, STD = 7, 0.01  # the model of tests/golden/greedy.pt


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(fn, world, *args):
    port = _free_port()
    mp.spawn(_entry, args=(world, port, fn, args), nprocs=world, join=True)


def _entry(rank, world, port, fn, args):
    for p in (str(HERE), str(HERE.parent)):
        if p not in sys.path:
            sys.path.insert(0, p)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# shards (single process)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("t", [2, 4])
def test_local_config_and_kv_sharing(t):
    cfg = synth.tiny_config()
    lc = tp.local_config(cfg, t)
    assert (lc.hq, lc.hk, lc.hv, lc.inter, lc.vocab) == (cfg.hq // t, cfg.hk // t, cfg.hv // t, cfg.inter // t, cfg.vocab // t)
    assert lc.hkv == max(1, cfg.hkv // t) and lc.hidden == cfg.hidden
    assert lc.hq % lc.hkv == 0 and lc.hv % lc.hk == 0 and lc.hv // lc.hk == cfg.hv // cfg.hk
    big = tp.local_config(synth.qwen27b_config(), 8)
    assert (big.hq, big.hkv, big.hk, big.hv, big.inter, big.vocab) == (3, 1, 2, 6, 2176, 31040)


def test_select_rows_slice_k_slice_tiles_roundtrip():
    g = torch.Generator().manual_seed(3)
    p = synth.random_w4(96, 256, g, "cpu", 0.02)
    full = dequant_oracle(p)
    rows = torch.tensor([5, 0, 17, 95, 33, 34, 35, 64, 2])
    sel = tp.select_rows(p, rows)
    assert sel.M == 9 and sel.qw.shape[0] == 1
    assert torch.equal(dequant_oracle(sel), full[rows])
    assert torch.equal(torch.cat([dequant_oracle(tp.slice_k(p, 0, 128)), dequant_oracle(tp.slice_k(p, 128, 256))], 1), full)
    assert torch.equal(torch.cat([dequant_oracle(tp.slice_tiles(p, 0, 2)), dequant_oracle(tp.slice_tiles(p, 2, 6))], 0), full)
    gu = synth.random_w4(64, 128, g, "cpu", 0.02, M=32, gate_up=True)
    G, U = dequant_oracle(gu)
    G0, U0 = dequant_oracle(tp.slice_tiles(gu, 0, 2))
    G1, U1 = dequant_oracle(tp.slice_tiles(gu, 2, 4))
    assert torch.equal(torch.cat([G0, G1]), G) and torch.equal(torch.cat([U0, U1]), U)


@pytest.mark.parametrize("t,small8", [(2, False), (4, False), (2, True), (8, True)])
def test_shards_reassemble_to_the_full_layer(t, small8):
    """Row shards of in_proj are the head slices, K shards of out / down concatenate to the full
    matrix, and attention KV heads are shared once t exceeds their number (t = 4 on the tiny
    configuration, t = 8 on the 8-way shardable one)."""
    cfg = synth.shardable8_config() if small8 else synth.tiny_config()
    W = synth.build_model(cfg, SEED, "cpu", STD)
    lc = tp.local_config(cfg, t)
    for li in (0, 3):
        L = W["layers"][li]
        full_in, full_out = dequant_oracle(L["in_proj"]), dequant_oracle(L["out"])
        shards = [tp.shard_layer(L, cfg, t, g) for g in range(t)]
        assert torch.equal(torch.cat([dequant_oracle(s["out"]) for s in shards], 1), full_out)
        assert torch.equal(torch.cat([dequant_oracle(s["down"]) for s in shards], 1), dequant_oracle(L["down"]))
        Gf, Uf = dequant_oracle(L["gate_up"])
        assert torch.equal(torch.cat([dequant_oracle(s["gate_up"])[0] for s in shards]), Gf)
        assert torch.equal(torch.cat([dequant_oracle(s["gate_up"])[1] for s in shards]), Uf)
        for g, s in enumerate(shards):
            loc = dequant_oracle(s["in_proj"])
            if L["type"] == "linear_attention":
                assert loc.shape[0] == lc.gdn_proj_rows
                kd, D = cfg.key_dim, cfg.dk
                assert torch.equal(loc[:lc.key_dim], full_in[g * lc.hk * D:(g + 1) * lc.hk * D])
                assert torch.equal(loc[lc.key_dim:2 * lc.key_dim], full_in[kd + g * lc.hk * D:kd + (g + 1) * lc.hk * D])
                a_local = loc[lc.conv_dim + lc.value_dim + lc.hv:]
                a0 = cfg.conv_dim + cfg.value_dim + cfg.hv + g * lc.hv
                assert torch.equal(a_local, full_in[a0:a0 + lc.hv])
                assert torch.equal(s["A_log"], L["A_log"][g * lc.hv:(g + 1) * lc.hv])
                assert s["conv_w"].shape[0] == lc.conv_dim
            else:
                assert loc.shape[0] == lc.attn_proj_rows
                hd, q0 = cfg.head_dim, cfg.hq * 2 * cfg.head_dim
                kv_head = g * lc.hkv if t <= cfg.hkv else g // (t // cfg.hkv)
                kl = loc[lc.hq * 2 * hd:lc.hq * 2 * hd + lc.hkv * hd]
                assert torch.equal(kl, full_in[q0 + kv_head * hd:q0 + (kv_head + lc.hkv) * hd])
                # every local query head reads a KV head this rank holds
                grp = cfg.hq // cfg.hkv
                for j in range(lc.hq):
                    assert (g * lc.hq + j) // grp - kv_head == j // (lc.hq // lc.hkv)


def test_build_sharded_model_equals_shard_of_built_model():
    cfg = synth.tiny_config()
    W = synth.build_model(cfg, SEED, "cpu", STD)
    a = tp.shard_model(W, cfg, 2, 1)
    b = tp.build_sharded_model(cfg, 2, 1, SEED, "cpu", STD)
    assert torch.equal(a["lm_head"].qw, b["lm_head"].qw)
    for La, Lb in zip(a["layers"] + [a["mtp"]], b["layers"] + [b["mtp"]]):
        for k in ("in_proj", "out", "gate_up", "down"):
            assert torch.equal(La[k].qw, Lb[k].qw) and torch.equal(La[k].scales, Lb[k].scales)
    assert torch.equal(a["mtp"]["fc"].qw, b["mtp"]["fc"].qw)


# ---------------------------------------------------------------------------------------------
# world_size 2 over gloo
# ---------------------------------------------------------------------------------------------
def _tp_step_worker(rank, world, steps):
    import tp_ref
    cfg = synth.tiny_config()
    W = synth.build_model(cfg, SEED, "cpu", STD)
    lc = oracle_config(tp.local_config(cfg, world))
    Wl = dense_model(tp.shard_model(W, cfg, world, rank))
    st = OM.State(lc, 64)
    if rank == 0:
        oc = oracle_config(cfg)
        Wd = dense_model(W)
        st0 = OM.State(oc, 64)
    tok = 11
    for s in range(steps):
        lg_l, hf = tp_ref.tp_decode_step(Wl, st, tok, lc)
        nxt = tp_ref.merge_argmax(lg_l, rank * lc.vocab)
        lg = tp_ref.gather_logits(lg_l)
        assert nxt == int(torch.argmax(lg.float()))
        # the draft head on the same row (position s, next token = the greedy one)
        mlg_l, _ = tp_ref.tp_mtp_step(Wl, st, hf, nxt, s, lc)
        mlg = tp_ref.gather_logits(mlg_l)
        if rank == 0:
            ref, hf0 = OM.decode_step(Wd, st0, tok, oc, fused_swiglu=True)
            assert cosine(lg, ref) > 0.9999, (s, cosine(lg, ref))
            assert int(torch.argmax(ref.float())) == nxt, s
            mref, _ = OM.mtp_step(Wd, st0, hf0, nxt, s, oc, fused_swiglu=True)
            assert cosine(mlg, mref) > 0.9999, (s, cosine(mlg, mref))
        tok = nxt


def test_sharded_oracle_step_matches_unsharded_world2():
    _spawn(_tp_step_worker, 2, 6)


def _argmax_worker(rank, world):
    import tp_ref
    g = torch.Generator().manual_seed(5)
    V = 64
    for case in range(8):
        full = torch.randn(world * V, generator=g).to(torch.bfloat16)
        if case % 2:  # equal maxima in both shards and twice inside one: the lowest id wins
            full[[7, 40, V + 3]] = 9.0
        if case == 7:
            full[:] = float("-inf")
        got = tp_ref.merge_argmax(full[rank * V:(rank + 1) * V], rank * V)
        assert got == int(torch.argmax(full.float())), case


def test_vocabulary_split_argmax_tie_rule_world2():
    _spawn(_argmax_worker, 2)


def _partial_sum_worker(rank, world):
    """K-split W4 GEMV through the numpy oracle: rank-ordered fp32 sum of the partial rows equals
    the full product up to fp32 reassociation, and is identical on every rank."""
    import numpy as np
    import tp_ref
    from oracle import w4 as OW
    g = torch.Generator().manual_seed(9)
    p = synth.random_w4(64, 512, g, "cpu", 0.02)
    x = torch.randn(3, 512, generator=g).to(torch.bfloat16)
    w = 512 // world
    ps = tp.slice_k(p, rank * w, (rank + 1) * w)
    Wl = OW.dequantize(ps.qw.numpy(), ps.scales.numpy(), ps.M, ps.K, False)
    part = torch.from_numpy(x[:, rank * w:(rank + 1) * w].float().numpy() @ Wl.T.astype(np.float32))
    got = tp_ref.reduce_parts(part)
    full = x.float() @ dequant_oracle(p).T
    assert torch.allclose(got.float(), full, rtol=2e-2, atol=1e-3)
    both = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(both, got)
    assert all(torch.equal(both[0], b) for b in both)


def test_ksplit_partial_sums_world2():
    _spawn(_partial_sum_worker, 2)
