"""Benchmark of the batch-1 decode path on B200: 27B-shape W4A16 model, random-init weights,
128-token seeded prompt, 1,024 greedy tokens per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0). `value` = decode tokens per second (plain greedy, inputs
resident on the device, CUDA-event time of the decode replays); `e2e` = the same through
Engine.generate() with the prompt coming from host memory and the tokens read back to the host,
prefill included; `roofline` = the W4 GEMV kernel timed alone on this model's own matrices in
token order (every matrix distinct, 13 GB, far larger than L2) against the measured HBM copy
bandwidth; `mtp_k4` = speculative decoding with k = 4 at forced acceptance lengths 0..4 and natural
acceptance; `cpu_baseline` = whole tokens of the same model shape on the host cores through the
reference's own torch path (oracle/_ref, else the oracle's restatement of it); at N > 1
`tp_parity` compares the tensor-parallel engine's logits with the single-GPU engine's.

--impl reference times that CPU path as an arm of its own (rank 0 only).
--impl reference-gpu (one GPU) runs the unmodified reference engine on its own kernels, built for
sm_100a by baseline/build_ref.py, on the same synthetic model, and this library beside it.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN, N_NEW = 128, 1024
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
WORKLOAD = "27B-shape W4A16 plain greedy decode ({layers} layers, hidden 5120, vocab 248320), " \
           "{prompt}-token seeded prompt, {tokens} tokens per step"


def ncu_traffic_ratio():
    """DRAM bytes / algorithmic bytes of the W4 kernel from the kept ncu summary (a line
    `traffic_ratio: <float>` in profiles/w4_chain_kernel_27b_shapes.md); None if there is none."""
    f = ROOT / "profiles" / "w4_chain_kernel_27b_shapes.md"
    if f.exists():
        m = re.search(r"traffic_ratio:\s*([0-9.]+)", f.read_text())
        if m:
            return float(m.group(1))
    return None


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.idx)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            # under load = the upper half of the samples (idle gaps between steps clock down)
            sm.sort()
            out["sm_mhz"] = statistics.median(sm[len(sm) // 2:])
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ----------------------------------------------------------------------------------------------
# CPU arm: whole tokens of the model shape on the host cores, through the reference's torch path
# ----------------------------------------------------------------------------------------------
def _dense_on_grid(rows, K, g, scale_std):
    """Dense fp32 weights on the int4 grid: what dequantising a packed matrix of uniform codes and
    |N(0,1)| * scale_std group scales yields, built without the detour through the packer."""
    import torch
    codes = torch.randint(0, 16, (rows, K // 128, 128), generator=g, dtype=torch.int8)
    scales = (torch.randn(rows, K // 128, 1, generator=g).abs() * scale_std).to(torch.float16).float()
    return ((codes.float() - 8.0) * scales).view(rows, K)


def cpu_reference_tokens(steps: int, warmup: int, layers: int = 64, distinct: int = 4, vocab: int | None = None):
    """Times `steps` whole decode tokens (after `warmup`) of the 27B-shape model on the host cores
    with all host threads. The dense fp32 model would be 108 GB, so the `layers` layers cycle
    through `distinct` distinct weight sets (3 DeltaNet + 1 attention: 6 GB, far beyond any CPU
    cache, so the memory traffic of a token is that of the full model); every layer keeps its own
    recurrent state and KV cache. Uses the reference's own decode_step with its fake-quant linear
    when oracle/_ref has been built, else the oracle's restatement.
    Returns (tok_s, threads, kind, sample description, seconds per token)."""
    import torch
    from oracle import build_ref
    from oracle import model as OM
    from oracle.convert import oracle_config, reference_named
    from qengine_b200 import synth

    torch.set_num_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1
    cfg = synth.qwen27b_config(layers=layers)
    if vocab:
        cfg.vocab = vocab
    g = torch.Generator().manual_seed(1)
    H, I = cfg.hidden, cfg.inter

    def small(shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def dense_layer(kind):
        D = {"type": kind, "in_norm": small((H,), 0.1), "post_norm": small((H,), 0.1)}
        if kind == "linear_attention":
            D["in_proj"] = _dense_on_grid(cfg.gdn_proj_rows, H, g, 0.01)
            D["out"] = _dense_on_grid(H, cfg.value_dim, g, 0.01)
            D["conv_w"] = small((cfg.conv_dim, 1, cfg.conv_k), 0.5)
            D["A_log"] = (torch.rand(cfg.hv, generator=g) * 5.7 - 3.0).to(torch.bfloat16)
            D["dt_bias"], D["norm_w"] = small((cfg.hv,)), small((cfg.dv,), 0.2, 1.0)
        else:
            D["in_proj"] = _dense_on_grid(cfg.attn_proj_rows, H, g, 0.01)
            D["out"] = _dense_on_grid(H, cfg.hq * cfg.head_dim, g, 0.01)
            D["q_norm"], D["k_norm"] = small((cfg.head_dim,), 0.3), small((cfg.head_dim,), 0.3)
        D["gate"], D["up"] = _dense_on_grid(I, H, g, 0.01), _dense_on_grid(I, H, g, 0.01)
        D["down"] = _dense_on_grid(H, I, g, 0.01)
        return D

    sets = [dense_layer(cfg.layer_types[i]) for i in range(min(distinct, layers))]
    D = {"embed": small((cfg.vocab, H)), "final_norm": small((H,), 0.1),
         "lm_head": _dense_on_grid(cfg.vocab, H, g, 0.01),
         "layers": [sets[l % len(sets)] for l in range(layers)], "mtp": None}
    ref = build_ref.load()
    ocfg = oracle_config(cfg)
    if ref is not None:
        R, _ = ref
        rcfg = R.Config(hidden=cfg.hidden, layers=cfg.layers, inter=cfg.inter, vocab=cfg.vocab, eps=cfg.eps,
                        layer_types=cfg.layer_types, hq=cfg.hq, hkv=cfg.hkv, head_dim=cfg.head_dim,
                        rope_theta=cfg.rope_theta, rotary_dim=cfg.rotary_dim, hk=cfg.hk, hv=cfg.hv, dk=cfg.dk,
                        dv=cfg.dv, conv_k=cfg.conv_k, tied=False, mtp_layers=0)
        Wn = reference_named(D, cfg)
        st = R.State(rcfg, 64, device="cpu")
        fq = lambda x, w: torch.nn.functional.linear(x.float(), w.float()).to(torch.bfloat16)
        step = lambda tok: R.decode_step(Wn, st, tok, rcfg, lin=fq)
        kind = "reference"
    else:
        st = OM.State(ocfg, 64, with_mtp=False)
        step = lambda tok: OM.decode_step(D, st, tok, ocfg, fused_swiglu=False)[0]
        kind = "port"
    tok, times = 17, []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            lg = step(tok)
            tok = int(lg.float().argmax())
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    per_tok = statistics.mean(times)
    desc = (f"{steps} whole tokens ({layers} layers + lm_head of {cfg.vocab} rows) of the 27B-shape model, dense fp32 "
            f"weights on the int4 grid; the layers cycle through {len(sets)} distinct weight sets "
            f"({sum(t.numel() for s_ in sets for t in s_.values() if hasattr(t, 'numel')) * 4 / 1e9:.1f} GB) because the "
            f"whole dense model does not fit host memory; greedy, context <= {warmup + steps}")
    return 1.0 / per_tok, torch.get_num_threads(), kind, desc, per_tok


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tok_s, cores, kind, desc, per_tok = cpu_reference_tokens(max(1, a.steps), max(0, a.warmup), layers=a.layers,
                                                              vocab=a.ref_vocab or None)
    line = {
        "impl": "reference", "metric": "batch-1 decode tok/s (plain)", "value": tok_s, "unit": "tok/s",
        "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": per_tok * 1e3,
        "higher_is_better": True, "scaling": "weak" if a.gpus == 1 else "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD.format(layers=a.layers, prompt=a.prompt, tokens=a.tokens),
                   "step": "one whole token on the host cores (bounded sample of the workload)",
                   "timing": "host wall clock, CPU only"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def run_reference_gpu(a):
    """Same-box comparator: the unmodified reference engine on its own kernels, compiled for
    sm_100a by baseline/build_ref.py, decoding the same synthetic 27B-shape model. The model is
    handed over through the reference's public route for prepared weights: a cache directory in
    its layout (qengine_b200.cache.save_cache) plus a config.json. The same directory is then
    loaded into this repository's engine, so both engines multiply with the same bytes."""
    import shutil
    import tempfile
    import torch
    from qengine_b200 import cache, synth
    from qengine_b200.engine import Engine as Ours

    native = str(ROOT / "baseline" / "_ref" / "native" / "python")
    if not os.path.exists(os.path.join(native, "qengine", "engine.py")):
        print(json.dumps({"impl": "reference-gpu", "unavailable": "baseline/_ref/native is not built "
                          "(python baseline/build_ref.py needs the reference checkout)"}), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = synth.qwen27b_config(layers=a.layers)
    n_new, P = a.tokens, a.prompt
    tmp = tempfile.mkdtemp(prefix="qe_cache_")
    try:
        model_dir = os.path.join(tmp, "synthetic-27b")
        cache.write_config(model_dir, cfg)
        W = synth.build_model(cfg, seed=1, device=dev, scale_std=0.01)
        t0 = time.perf_counter()
        cdir = cache.save_cache(cache.cache_path(os.path.join(tmp, "cache"), "synthetic-27b"), W)
        save_s = time.perf_counter() - t0
        del W
        torch.cuda.empty_cache()
        prompt = synth.prompt_ids(P, cfg.vocab, seed=1234)

        sys.path.insert(0, native)
        from qengine.engine import Engine as Ref, W4Linear as RefW4  # the reference's own classes
        t0 = time.perf_counter()
        ref = Ref(model_dir, max_len=P + n_new + 32, linear=RefW4(), device="cuda",
                  cache_dir=os.path.join(tmp, "cache"))
        load_s = time.perf_counter() - t0
        for _ in range(max(1, a.warmup)):
            ref.generate(prompt, n_new)
        sampler = ClockSampler(0)
        sampler.start()
        dec, e2e = [], []
        for _ in range(a.steps):
            t0 = time.perf_counter()
            gen_ref, _, d = ref.generate(prompt, n_new, timing=True)
            e2e.append(time.perf_counter() - t0)
            dec.append(d)
        clocks = sampler.stop()
        ref_tok_s = a.steps * (n_new - 1) / sum(dec)
        spec = {}
        if not a.no_mtp:
            ref.generate_spec(prompt, n_new, 4)
            out, _, d, st = ref.generate_spec(prompt, n_new, 4, timing=True)
            spec = {"tok_s": (n_new - 1) / d, "tokens_per_cycle": st["tokens_per_cycle"],
                    "ms_per_cycle": d * 1e3 / max(1, st["cycles"]), "identical_to_plain": out == gen_ref}
        del ref
        torch.cuda.empty_cache()

        ours = Ours.from_cache(model_dir, os.path.join(tmp, "cache"), device=dev, max_len=P + n_new + 32)
        for _ in range(max(1, a.warmup)):
            ours.generate(prompt, n_new)
        dec2 = []
        for _ in range(a.steps):
            gen_ours, _, d = ours.generate(prompt, n_new, timing=True)
            dec2.append(d)
        ours_tok_s = a.steps * (n_new - 1) / sum(dec2)
        same = 0
        for x, y in zip(gen_ref, gen_ours):
            if x != y:
                break
            same += 1
        print(json.dumps({
            "impl": "reference-gpu", "metric": "batch-1 decode tok/s (plain)", "value": ref_tok_s,
            "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": 1e3 * sum(dec) / a.steps, "higher_is_better": True, "dtype": "bf16 x int4 (W4A16)",
            "data": "synthetic", "config": {"workload": WORKLOAD.format(layers=a.layers, prompt=P, tokens=n_new),
                                            "route": "cache directory in the reference's layout"},
            "e2e": {"value": a.steps * n_new / sum(e2e), "unit": "tok/s", "h2d_bytes_per_step": 4 * P,
                    "d2h_bytes_per_step": 4 * n_new},
            "reference_mtp_k4": spec, "clocks": clocks,
            "this_library_same_cache": {"tok_s": ours_tok_s, "ratio_to_reference": ours_tok_s / ref_tok_s,
                                        "leading_tokens_equal": same, "of": len(gen_ref)},
            "cache": {"bytes": sum(os.path.getsize(os.path.join(cdir, f)) for f in os.listdir(cdir)),
                      "save_s": save_s, "reference_load_s": load_s}}), flush=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def w4_sequence_timing(eng, n_rows, reps=10):
    """Every W4 GEMV of one token (all layers in order, then the lm_head) as one CUDA graph on the
    model's own weights: the dominant kernel timed alone, in situ shapes, nothing reused in L2.
    The GEMVs that follow an RMSNorm in the engine (in_proj, gate_up, lm_head) take fp16 rows when
    the engine runs them that way, the others bf16. Returns (ms per token, launches, bytes)."""
    import torch
    from qengine_b200 import _w4
    cfg = eng.cfg
    lin = eng.linear
    H = cfg.hidden
    xs = {k: torch.randn(n_rows, k, device=eng.dev).to(torch.bfloat16) for k in
          {H, cfg.value_dim, cfg.hq * cfg.head_dim, cfg.inter}}
    x16 = xs[H].to(torch.float16)
    outs, plan, nbytes = {}, [], 0
    for L in eng.layers:
        for key in ("in_proj", "out", "gate_up", "down"):
            p = L[key]
            outs.setdefault(p.M, torch.empty(n_rows, p.M, device=eng.dev, dtype=torch.bfloat16))
            plan.append((p, key in ("in_proj", "gate_up")))
            nbytes += p.nbytes + n_rows * (p.K + p.M) * 2
    p = eng.lm_head
    outs.setdefault(p.M, torch.empty(n_rows, p.M, device=eng.dev, dtype=torch.bfloat16))
    plan.append((p, True))
    nbytes += p.nbytes + n_rows * (p.K + p.M) * 2
    f16 = bool(getattr(eng, "f16", False))

    def body():
        for p, normed in plan:
            x = x16 if (f16 and normed) else xs[p.K]
            _w4.gemv_chain([lin.job(x, p, outs[p.M])], **lin.kw)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return statistics.median(ms), len(plan), nbytes


def mlp_pair_timing(eng, n_rows, reps=20):
    """W4 microbench: fused gate/up (5120 -> 2 x 17408, SwiGLU) then down (17408 -> 5120), rotating
    over the layers' distinct weights so L2 cannot hold them. Returns (us per pair, GB/s)."""
    import torch
    cfg, lin = eng.cfg, eng.linear
    x = torch.randn(n_rows, cfg.hidden, device=eng.dev).to(torch.bfloat16)
    act = torch.empty(n_rows, cfg.inter, device=eng.dev, dtype=torch.bfloat16)
    out = torch.empty(n_rows, cfg.hidden, device=eng.dev, dtype=torch.bfloat16)
    Ls = eng.layers
    nbytes = Ls[0]["gate_up"].nbytes + Ls[0]["down"].nbytes + n_rows * (cfg.hidden * 2 + cfg.inter * 2) * 2

    def body():
        for L in Ls:
            lin.gate_up(x, L["gate_up"], act)
            lin(act, L["down"], out)

    body()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    us = statistics.median(ms) * 1e3 / len(Ls)
    return us, nbytes / (us * 1e-6) / 1e9


def exchange_timing(eng, reps=10, count=128):
    """One tensor-parallel exchange (every rank's fp32 partial row to every rank, summed inside the
    residual norm) timed as a graph of `count` of them. Every rank must call this."""
    import torch
    from qengine_b200 import _C
    h, w = eng.h[:1], eng.final_norm

    def body():
        for _ in range(count):
            if eng.tp.transport == "nccl":
                eng.tp.all_gather(eng.parts[1], eng.part32[:1])
                _C.rmsnorm1p_parts(h, eng.parts[1], w, eng.xn[:1], eng.cfg.eps)
            else:
                eng.tp.exchange_norm(h, eng.part32[:1], w, eng.xn[:1], eng.cfg.eps)

    eng.part32.zero_()
    body()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        body()
    ms = []
    for i in range(reps + 3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            ms.append(e0.elapsed_time(e1))
    return statistics.median(ms) * 1e3 / count


def tp_parity(world, rank, dev, transport, positions=16):
    """Tensor-parallel logits against the single-GPU engine on the same seeded weights: a 4-layer
    model of the 27B width (3 DeltaNet + 1 attention layer, full vocabulary), `positions`
    teacher-forced tokens. Every rank runs its shard; rank 0 also runs the whole model on its own
    GPU and compares. Returns the comparison on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    from qengine_b200 import synth, tp
    from qengine_b200.engine import Engine
    cfg = synth.qwen27b_config(layers=4)
    seq = synth.prompt_ids(positions, cfg.vocab, seed=77)
    Wr = tp.build_sharded_model(cfg, world, rank, seed=3, device=dev, scale_std=0.01, mtp=False)
    eng = Engine(cfg, Wr, max_len=64, device=dev, tp=tp.TPGroup(transport=transport), mtp=False)
    local = eng.sequence_logits(seq).contiguous()
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    err = eng.tp.error()
    eng.graphs.clear()
    del eng, Wr
    torch.cuda.empty_cache()
    out = None
    if rank == 0:
        full = torch.cat(parts, dim=-1).float()
        W1 = synth.build_model(cfg, seed=3, device=dev, scale_std=0.01, mtp=False)
        ref = Engine(cfg, W1, max_len=64, device=dev, mtp=False).sequence_logits(seq).float()
        cos = torch.nn.functional.cosine_similarity(full.double(), ref.double(), dim=-1)
        out = {"model": "4 layers of the 27B width, full vocabulary", "positions": positions,
               "min_cosine": float(cos.min()), "max_abs": float((full - ref).abs().max()),
               "top1_agree": int((full.argmax(-1) == ref.argmax(-1)).sum()), "exchange_error": err,
               "against": "the single-GPU engine of this library on the same seeded weights"}
        del W1, ref
        torch.cuda.empty_cache()
    dist.barrier()
    return out


def bytes_per_token(eng, mean_ctx):
    """Algorithmic HBM bytes of one plain decode step at context length mean_ctx."""
    from qengine_b200 import synth
    cfg = eng.cfg
    pb = synth.packed_bytes({"layers": eng.layers, "lm_head": eng.lm_head, "mtp": eng.mtp})
    n_gdn = sum(t == "linear_attention" for t in cfg.layer_types)
    n_att = cfg.layers - n_gdn
    state = n_gdn * 2 * cfg.hv * cfg.dk * cfg.dv * 4
    staged = n_gdn * 2 * (cfg.hv * (cfg.dk + cfg.dv + 2)) * 4
    norms = (2 * cfg.layers + 1) * cfg.hidden * 2
    kv_row = n_att * 2 * cfg.hkv * cfg.head_dim * 2
    total = pb["decoder"] + pb["lm_head"] + state + staged + norms + cfg.hidden * 2 + kv_row * mean_ctx + kv_row
    return total, pb


def run_ours(a):
    import torch
    import torch.distributed as dist
    from qengine_b200 import synth
    from qengine_b200.engine import Engine

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    parity_early = None
    if world > 1 and not a.no_tp_parity:
        parity_early = tp_parity(world, rank, dev, a.transport)
    cfg = synth.qwen27b_config(layers=a.layers)
    n_new, P = a.tokens, a.prompt
    if world == 1:
        W = synth.build_model(cfg, seed=1, device=dev, scale_std=0.01)
        eng = Engine(cfg, W, max_len=P + n_new + 32, device=dev)
    else:  # tensor parallel: one sequence, every matrix sharded over the ranks
        from qengine_b200 import tp
        W = tp.build_sharded_model(cfg, world, rank, seed=1, device=dev, scale_std=0.01)
        eng = Engine(cfg, W, max_len=P + n_new + 32, device=dev, tp=tp.TPGroup(transport=a.transport))
    prompt = synth.prompt_ids(P, cfg.vocab, seed=1234)

    # ---- warm-up (captures the graphs) and timed plain decode ------------------------------
    for _ in range(max(1, a.warmup)):
        eng.generate(prompt, n_new)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    dec_s, e2e_s = [], []
    for _ in range(a.steps):
        t0 = time.perf_counter()
        gen, _, d = eng.generate(prompt, n_new, timing=True)   # host prompt in, host tokens out
        e2e_s.append(time.perf_counter() - t0)
        dec_s.append(d)
    barrier()
    clocks = sampler.stop()
    t_dec = torch.tensor([sum(dec_s), sum(e2e_s)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_dec, op=dist.ReduceOp.MAX)
    dec_total, e2e_total = t_dec.tolist()
    value = a.steps * (n_new - 1) / dec_total
    e2e = a.steps * n_new / e2e_total
    kernels_per_token = eng.graph_kernels[(1, False, 0, False)]
    launches = a.steps * ((n_new - 1) * kernels_per_token +
                          sum(eng.graph_kernels[k] for k in eng._prefill_keys(P, False, 0)) * (P // 8))

    # ---- MTP k = 4 (every rank takes part: the passes hold collectives) -----------------------
    mtp = {}
    if not a.no_mtp:
        truth = prompt + gen + [0] * 64
        for label, fa in [("natural", None)] + [(f"a{i}", i) for i in range(5)]:
            kw = dict(force_accept=fa, truth=truth) if fa is not None else {}
            eng.generate_spec(prompt, n_new, 4, **kw)  # capture + warm
            barrier()
            out, _, d, st = eng.generate_spec(prompt, n_new, 4, timing=True, **kw)
            td = torch.tensor([d], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(td, op=dist.ReduceOp.MAX)
            d = float(td.item())
            mtp[label] = {"tok_s": (n_new - 1) / d, "tokens_per_cycle": st["tokens_per_cycle"],
                          "ms_per_cycle": d * 1e3 / max(1, st["cycles"]), "identical_to_plain": out == gen}
    # ---- the same cycle with a pruned draft head (drafts scored over the first --draft-vocab ids) ----
    if not a.no_mtp and a.draft_vocab > 0:
        kw = dict(max_len=P + n_new + 32, device=dev, draft_vocab=a.draft_vocab)
        if world > 1:
            kw["tp"] = tp.TPGroup(transport=a.transport)
        eng_d = Engine(cfg, W, **kw)
        for label, fa in (("a0", 0), ("a4", 4)):
            eng_d.generate_spec(prompt, n_new, 4, force_accept=fa, truth=truth)
            barrier()
            out, _, d, st = eng_d.generate_spec(prompt, n_new, 4, timing=True, force_accept=fa, truth=truth)
            td = torch.tensor([d], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(td, op=dist.ReduceOp.MAX)
            d = float(td.item())
            mtp[f"draft_vocab_{a.draft_vocab}_{label}"] = {
                "tok_s": (n_new - 1) / d, "tokens_per_cycle": st["tokens_per_cycle"],
                "ms_per_cycle": d * 1e3 / max(1, st["cycles"]), "identical_to_plain": out == gen}
        del eng_d
        gc.collect()  # engines hold reference cycles; their graphs and buffers go with the collection
        torch.cuda.empty_cache()
    # ---- the draft layer's fc + in_proj + o_proj pinned in L2 for the draft phase (A/B) ---------
    if not a.no_mtp and world == 1:
        eng_p = Engine(cfg, W, max_len=P + n_new + 32, device=dev)
        eng_p.pin_mtp_l2(True)
        window_bytes = eng_p.l2_win[1]
        for label, fa in (("a0", 0), ("a4", 4)):
            eng_p.generate_spec(prompt, n_new, 4, force_accept=fa, truth=truth)
            barrier()
            out, _, d, st = eng_p.generate_spec(prompt, n_new, 4, timing=True, force_accept=fa, truth=truth)
            mtp[f"l2_window_{label}"] = {
                "tok_s": (n_new - 1) / d, "ms_per_cycle": d * 1e3 / max(1, st["cycles"]),
                "identical_to_plain": out == gen, "window_bytes": window_bytes,
                "without_window_ms_per_cycle": mtp[label]["ms_per_cycle"]}
        eng_p.pin_mtp_l2(False)
        del eng_p
        gc.collect()
        torch.cuda.empty_cache()
    # ---- prompt processing: 8-row passes through the GEMV vs 64-row passes through the GEMM ------
    prefill = {}
    if world == 1 and a.prefill_tokens >= 64:
        eng_f = Engine(cfg, W, max_len=a.prefill_tokens + 64, device=dev, mtp=False)
        long_prompt = synth.prompt_ids(a.prefill_tokens, cfg.vocab, seed=4321)
        firsts = {}
        for label, wide_pass in (("rows8", False), ("rows64", True)):
            firsts[label] = eng_f.generate(long_prompt, 2, wide=wide_pass)[0]  # captures the graphs
            secs = []
            for _ in range(3):
                barrier()
                secs.append(eng_f.generate(long_prompt, 2, timing=True, wide=wide_pass)[1])
            sec = statistics.median(secs)
            prefill[label] = {"tok_s": a.prefill_tokens / sec, "ms": sec * 1e3}
        prefill.update(prompt_tokens=a.prefill_tokens, speedup=prefill["rows64"]["tok_s"] / prefill["rows8"]["tok_s"],
                       first_token_equal=firsts["rows8"] == firsts["rows64"],
                       what="host feed + graph replays of a whole prompt; rows64 = passes of 64 rows through "
                            "qe_w4_gemm (tcgen05), the mixers in sub-passes of 8 rows")
        del eng_f
        gc.collect()
        torch.cuda.empty_cache()
    exchange_us = exchange_timing(eng) if world > 1 else None
    parity = parity_early

    # ---- verify pass alone vs plain step (one graph replay each, same weights) -----------------
    verify = {}
    if not a.no_mtp:
        for n_rows in (1, 5):
            g = eng.graph(n_rows, False, 0)
            eng.reset()
            eng.ctl[eng.MODE].fill_(1)
            eng.ctl[eng.POS].fill_(P)
            ms = []
            for i in range(8):
                eng.ctl[eng.POS].fill_(P)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                barrier()
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    ms.append(e0.elapsed_time(e1))
            verify[f"ms_n{n_rows}"] = statistics.median(ms)
        verify["verify_cost_vs_plain_step"] = verify["ms_n5"] / verify["ms_n1"]

    # ---- long cache: 32,768 pre-filled positions (seeded N(0,1) K/V), then the same decode ---------
    longctx = {}
    if a.context > 0:
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        n_long = min(n_new, 256)
        kw = dict(max_len=a.context + P + n_long + 64, device=dev)
        if world > 1:
            kw["tp"] = tp.TPGroup(transport=a.transport)
        eng = Engine(cfg, W, **kw)
        eng.set_context(a.context)
        eng.generate(prompt, n_long)
        barrier()
        gen_l, _, d = eng.generate(prompt, n_long, timing=True)
        td = torch.tensor([d], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(td, op=dist.ReduceOp.MAX)
        longctx = {"context": a.context, "tokens": n_long, "plain_tok_s": (n_long - 1) / float(td.item()),
                   "plain_ms_per_token": float(td.item()) * 1e3 / (n_long - 1),
                   "kv_bytes_per_token": 2 * cfg.hkv * 2 * cfg.head_dim * a.context *
                                         sum(t == "full_attention" for t in cfg.layer_types)}
        if not a.no_mtp:
            truth_l = prompt + gen_l + [0] * 64
            for label, fa in (("a0", 0), ("a4", 4)):
                eng.generate_spec(prompt, n_long, 4, force_accept=fa, truth=truth_l)
                barrier()
                out, _, d, st = eng.generate_spec(prompt, n_long, 4, timing=True, force_accept=fa, truth=truth_l)
                td = torch.tensor([d], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(td, op=dist.ReduceOp.MAX)
                d = float(td.item())
                longctx[f"mtp_k4_{label}"] = {"tok_s": (n_long - 1) / d, "ms_per_cycle": d * 1e3 / max(1, st["cycles"]),
                                              "identical_to_plain": out == gen_l}

    line = {}
    if rank == 0:
        peak, peak_kind = measured_peak()
        B_tok, pb = bytes_per_token(eng, P + n_new / 2)
        ms_tok = dec_total / (a.steps * (n_new - 1)) * 1e3
        # dominant kernel alone, in situ
        seq_ms, seq_launches, seq_bytes = w4_sequence_timing(eng, 1)
        seq5_ms, _, _ = w4_sequence_timing(eng, 5)
        pair1_us, pair1_gbs = mlp_pair_timing(eng, 1)
        pair5_us, pair5_gbs = mlp_pair_timing(eng, 5)
        achieved = seq_bytes / (seq_ms * 1e-3) / 1e9
        ratio = ncu_traffic_ratio()
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": ratio * seq_bytes / seq_launches if ratio else None,
                    "traffic_note": "dram bytes per launch = algorithmic bytes x the ratio of the kept ncu capture "
                                    "(profiles/w4_chain_kernel_27b_shapes.md)" if ratio else "no ncu capture kept",
                    "peak_kind": f"of {peak_kind}",
                    "per_launch": {"algorithmic_bytes": seq_bytes / seq_launches,
                                   "avg_us": seq_ms * 1e3 / seq_launches},
                    "kernel": "w4_chain_kernel",
                    "how": f"{seq_launches} launches (every W4 matrix of one token, in order) as one graph, "
                           f"median of 10 CUDA-event timings; bytes = packed weights + scales + x + out"}
        cpu = None
        if world == 1 and not a.no_cpu:
            tok_s, cores, kind, desc, _ = cpu_reference_tokens(a.cpu_tokens, 1, layers=a.layers)
            cpu = {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": kind, "sample": desc}
        line = {
            "metric": "batch-1 decode tok/s (plain)", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": dec_total / a.steps * 1e3,
            "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD.format(layers=cfg.layers, prompt=P, tokens=n_new),
                       "parallelism": "single GPU" if world == 1 else
                       f"tp{world}: one sequence, every matrix sharded; {2 * cfg.layers + 2} exchanges of fp32 partial "
                       f"rows per token, transport {a.transport}",
                       "l2": "inputs larger than L2 (13 GB of weights streamed per token)",
                       "timing": "CUDA events around the decode graph replays, max over ranks"},
            "ms_per_token": ms_tok,
            "hbm_roofline": {"bytes_per_token": B_tok, "tok_s_at_measured_peak": peak * 1e9 / B_tok,
                             "frac_of_measured": value / (peak * 1e9 / B_tok),
                             "tok_s_at_8TBs": 8e12 / B_tok, "frac_of_8TBs": value / (8e12 / B_tok),
                             "note": "bytes one rank streams per token"},
            "roofline": roofline,
            "w4_sequence": {"ms_n1": seq_ms, "ms_n5": seq5_ms, "bytes": seq_bytes, "launches": seq_launches},
            "w4_mlp_pair": {"us_m1": pair1_us, "gbs_m1": pair1_gbs, "us_m5": pair5_us, "gbs_m5": pair5_gbs},
            "mtp_k4": mtp,
            "verify_pass": verify,
            "long_context": longctx,
            "prefill": prefill,
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": (P // 8) * 36 + 8,
                    "d2h_bytes_per_step": n_new * 4},
            "gpu_launches": launches,
            "kernels_per_token": kernels_per_token,
            "clocks": clocks,
            "cpu_baseline": cpu,
        }
        if parity is not None:
            line["tp_parity"] = parity
        if exchange_us is not None:
            line["tp_exchange"] = {"us_per_exchange": exchange_us, "per_token": 2 * cfg.layers + 2,
                                   "transport": a.transport, "error": eng.tp.error(),
                                   "what": "one fp32 row [hidden] from every rank to every rank + the residual norm "
                                           "over the parts, back to back in one graph"}
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs that hold collectives go first; a teardown that still stalls must not hold the GPUs
        eng.graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        threading.Timer(30.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--layers", type=int, default=64, help="model depth (64 = the 27B shape)")
    ap.add_argument("--tokens", type=int, default=N_NEW, help="generated tokens per step")
    ap.add_argument("--prompt", type=int, default=PROMPT_LEN, help="prompt length (profiling runs use a short one)")
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"],
                    help="tensor-parallel exchange: own peer-memory kernels, or NCCL all-gather + norm")
    ap.add_argument("--context", type=int, default=32768,
                    help="pre-filled cache length of the long-context block (0 = skip it)")
    ap.add_argument("--draft-vocab", type=int, default=49152,
                    help="also time the MTP cycle with the draft head pruned to this many ids (0 = skip)")
    ap.add_argument("--prefill-tokens", type=int, default=1024,
                    help="prompt length of the prefill comparison (8-row vs 64-row passes; 0 = skip)")
    ap.add_argument("--no-mtp", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-tokens", type=int, default=8, help="whole tokens timed for cpu_baseline (N = 1 only)")
    ap.add_argument("--ref-vocab", type=int, default=0, help="reference arm: cut the vocabulary (tests only)")
    ap.add_argument("--no-tp-parity", action="store_true")
    a = ap.parse_args()
    if a.impl == "reference":
        run_reference_arm(a)
    elif a.impl == "reference-gpu":
        run_reference_gpu(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
