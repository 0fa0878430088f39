"""Python op surface `_w4`: same functions, keyword arguments, defaults and error behaviour as the
reference module `qengine._w4` (csrc/gemv_w4_bind.cpp:24-120), bound to qe_w4_gemv of
libqengine_b200.so through ctypes.

    gemv(x, qw, scales, out, M, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1,
         blocks_per_sm=0, min_units=4)
    gemv_swiglu(x, qw, scales, out, I, ...same...)
    auto_ksplit(Mp, Kp, N, warps=8)

Additions without a counterpart in the reference: `gemv_partial` (fp32 partial sums of a matrix
split along K over tensor-parallel ranks), `gemv_fused` (the GEMV with the residual add + RMSNorm
that produces its input fused into the launch), `gemv_chain` (several dependent GEMVs as one
cooperative launch) and `gemv_static` (no allocation).

Workspace: like the reference binding (gemv_w4_bind.cpp:12-22, 71-79) a per-device, grow-only
pair of buffers is kept here -- fp32 partial-sum slots (contents irrelevant) and int32 arrival
counters that the kernel leaves zeroed. They grow only outside CUDA-graph capture (the first,
eager call of a shape allocates); replaced buffers stay alive because a captured graph may still
point at them.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import W4Cfg, W4Norm, W4Params, W4Plan, check, launches, lib

EPI_NONE, EPI_SWIGLU = 0, 1
_MIN_WS_FLOATS, _MIN_COUNTERS = 1 << 18, 1 << 14


class _Workspace:
    def __init__(self):
        self.keep, self.ws, self.counters, self.gbar = [], None, None, None


_per_device: dict[int, _Workspace] = {}


def _req(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _workspace(dev: torch.device, ws_floats: int, counters: int) -> _Workspace:
    W = _per_device.setdefault(dev.index if dev.index is not None else torch.cuda.current_device(),
                               _Workspace())
    if W.ws is None or W.ws.numel() < ws_floats:
        _req(not torch.cuda.is_current_stream_capturing(),
             "W4 workspace would have to grow during graph capture: run the shape once eagerly first")
        if W.ws is not None:
            W.keep.append(W.ws)
        W.ws = torch.zeros(max(ws_floats, _MIN_WS_FLOATS), dtype=torch.float32, device=dev)
    if W.counters is None or W.counters.numel() < counters:
        _req(not torch.cuda.is_current_stream_capturing(),
             "W4 counters would have to grow during graph capture: run the shape once eagerly first")
        if W.counters is not None:
            W.keep.append(W.counters)
        W.counters = torch.zeros(max(counters, _MIN_COUNTERS), dtype=torch.int32, device=dev)
    return W


def reset_workspaces():
    """Zero the arrival counters and partial-sum slots of every device's workspace. Only needed
    after a launch that reported a ring error (`ring_error() != 0`): such a launch may leave them
    non-zero."""
    for W in _per_device.values():
        if W.counters is not None:
            W.counters.zero_()
        if W.ws is not None:
            W.ws.zero_()


def _packed(qw, scales):
    _req(qw.dtype == torch.int32 and qw.dim() == 4 and qw.size(2) == 32 and qw.size(3) == 4,
         "qw must be int32 [Mp/16, Kp/64, 32, 4] from quant.quantize_w4")
    _req(scales.dtype == torch.float16 and scales.dim() == 3 and scales.size(2) == 16,
         "scales must be fp16 [Mp/16, Kp/128, 16]")
    _req(qw.is_contiguous() and scales.is_contiguous(), "packed tensors must be contiguous")
    Mp, Kp = qw.size(0) * 16, qw.size(1) * 64
    _req(Kp % 128 == 0 and scales.size(0) == qw.size(0) and scales.size(1) == Kp // 128,
         "qw / scales shapes disagree")
    _req(qw.data_ptr() % 16 == 0 and scales.data_ptr() % 16 == 0, "packed tensors must be 16-byte aligned")
    return Mp, Kp


def _cfg(warps, unroll, ksplit, pdl, variant, mode, bps, min_units):
    _req(warps in (0, 4, 8, 16), "warps in {0 (auto),4,8,16}")
    _req(unroll in (0, 1, 2, 4), "unroll in {0 (auto),1,2,4}")
    _req(mode in (-1, 0, 2, 3, 4), "mode in {-1 (auto), 0, 2, 3, 4}")
    return W4Cfg(int(warps), int(unroll), int(ksplit), int(bool(pdl)), int(variant), int(mode), int(bps),
                 int(min_units))


class Job:
    """One GEMV of a chain: the C structs plus the tensors they point into (kept alive)."""
    __slots__ = ("p", "nrm", "dev", "keep")

    def __init__(self, p, nrm, dev, keep):
        self.p, self.nrm, self.dev, self.keep = p, nrm, dev, keep


def _launch(jobs, cfg, what):
    """Launch 1..4 jobs as one kernel (qe_w4_gemv_chain); scratch sized for the largest plan."""
    dev = jobs[0].dev
    ws_floats = counters = 0
    for j in jobs:
        plan = W4Plan()
        check(lib.qe_w4_plan_gemv(C.byref(j.p), C.byref(cfg), C.byref(plan)), f"{what} plan", kernels=0)
        ws_floats, counters = max(ws_floats, plan.ws_floats), max(counters, plan.counters)
    W = _workspace(dev, ws_floats, counters)
    for j in jobs:
        j.p.ws, j.p.counters = W.ws.data_ptr(), W.counters.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    n = len(jobs)
    if n == 1 and jobs[0].nrm is None:
        code = lib.qe_w4_gemv(C.byref(jobs[0].p), C.byref(cfg), stream)
    elif n == 1:
        code = lib.qe_w4_gemv_ex(C.byref(jobs[0].p), C.byref(jobs[0].nrm), C.byref(cfg), stream)
    else:
        if W.gbar is None:
            _req(not torch.cuda.is_current_stream_capturing(), "run the chain once eagerly before capturing it")
            W.gbar = torch.zeros(2, dtype=torch.int32, device=dev)
        ps = (C.POINTER(W4Params) * n)(*[C.pointer(j.p) for j in jobs])
        ns = (C.POINTER(W4Norm) * n)(*[C.pointer(j.nrm) if j.nrm is not None else C.POINTER(W4Norm)() for j in jobs])
        code = lib.qe_w4_gemv_chain(ps, ns, n, C.byref(cfg), W.gbar.data_ptr(), stream)
    _req(code != -22, f"{what}: argument combination not supported by the kernel")
    _req(code == 0, f"{what} launch failed: CUDA error {code}")
    launches[0] += 1


def job(x, qw, scales, out, M, swiglu=False, allow_f32_out=False, allow_f16_x=False) -> Job:
    """Describe out = x @ W~^T (or the SwiGLU of a gate/up pack) without launching it.
    allow_f16_x: x may be fp16 (rows written by `norm_rows(xn16_out=...)`, see qe_w4_params::x_f16);
    the reference's surface (`gemv`, `gemv_swiglu`) takes bf16 only."""
    for t in (x, qw, scales, out):
        _req(isinstance(t, torch.Tensor) and t.is_cuda, "CUDA tensors")
    epilogue = EPI_SWIGLU if swiglu else EPI_NONE
    out_f32 = allow_f32_out and out.dtype == torch.float32 and epilogue == EPI_NONE
    x_f16 = allow_f16_x and x.dtype == torch.float16
    _req(x.dtype == torch.bfloat16 or x_f16, "x must be bf16 (W4A16 kernel)")
    _req(out.dtype == torch.bfloat16 or out_f32, "out must be bf16")
    Mp, Kp = _packed(qw, scales)
    _req(x.dim() == 2 and out.dim() == 2, "x [N,K], out [N,M]")
    _req(x.stride(1) == 1 and out.stride(1) == 1, "x and out need unit stride along K / M")
    N, K = x.size(0), x.size(1)
    M = int(M)
    _req(1 <= N <= 8, "N must be 1..8")
    _req(out.size(0) == N and out.size(1) == M, "out shape must be [N, M]")
    _req(Kp - 128 < K <= Kp, f"x has K={K} but the packed weight has Kp={Kp}")
    if epilogue == EPI_SWIGLU:
        _req(Mp // 2 - 8 < M <= Mp // 2, "SwiGLU: out width I must match packed rows/2")
    else:
        _req(Mp - 16 < M <= Mp, "out width M must match packed rows")
    _req(x.data_ptr() != out.data_ptr(), "in-place not supported")
    if x_f16:
        _req(K == Kp and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "fp16 x: K == Kp, aligned rows")
    p = W4Params(qw.data_ptr(), scales.data_ptr(), x.data_ptr(), out.data_ptr(), None, None,
                 M, K, Mp, Kp, N, x.stride(0), out.stride(0), epilogue, int(out_f32), int(x_f16))
    return Job(p, None, x.device, (x, qw, scales, out))


def job_fused(h_in, delta, norm_w, eps, qw, scales, out, M, h_out=None, xn_out=None, tok=None,
              swiglu=False, f16=False) -> Job:
    """Describe out = gemv(RMSNorm1p(h_in + delta) * (1 + norm_w)) without launching it (see
    `gemv_fused` for the arguments). f16: keep the normalised rows as fp16 and run the fp16
    flavour of the GEMV (qe_w4_norm::f16; the caller vouches for sqrt(K) * |1 + norm_w| < 65504)."""
    for t in (h_in, norm_w, qw, scales, out):
        _req(isinstance(t, torch.Tensor) and t.is_cuda, "CUDA tensors")
    Mp, Kp = _packed(qw, scales)
    bf = torch.bfloat16
    _req(h_in.dtype == bf and norm_w.dtype == bf and out.dtype == bf, "h_in, norm_w and out must be bf16")
    _req(out.dim() == 2 and out.stride(1) == 1, "out [N, M] rows")
    N, M = out.size(0), int(M)
    _req(1 <= N <= 8 and out.size(1) == M, "N in 1..8 and out [N, M]")
    _req(h_in.dim() == 2 and h_in.stride(1) == 1 and h_in.size(1) == Kp and norm_w.numel() == Kp and
         norm_w.is_contiguous(), "h_in [*, K] with K == Kp, norm_w [K]")
    _req((Mp // 2 - 8 < M <= Mp // 2) if swiglu else (Mp - 16 < M <= Mp), "out width must match packed rows")
    nrm = W4Norm()
    nrm.h_in, nrm.ldh, nrm.norm_w, nrm.eps = h_in.data_ptr(), h_in.stride(0), norm_w.data_ptr(), float(eps)
    if tok is not None:
        _req(tok.dtype == torch.int32 and tok.is_contiguous() and tok.numel() >= N and h_in.is_contiguous(),
             "tok int32 [>= N], contiguous table")
        nrm.tok, nrm.vocab = tok.data_ptr(), h_in.size(0)
    else:
        _req(h_in.size(0) == N, "h_in must have N rows")
    for name, t in (("delta", delta), ("h_out", h_out), ("xn_out", xn_out)):
        if t is None:
            continue
        _req(t.is_cuda and t.dtype == bf and t.dim() == 2 and t.stride(1) == 1 and t.size(0) == N and
             t.size(1) == Kp, f"{name} must be bf16 [N, K]")
    if delta is not None:
        nrm.delta, nrm.ldd = delta.data_ptr(), delta.stride(0)
    if h_out is not None:
        _req(h_out.data_ptr() != h_in.data_ptr(), "h_out must not alias h_in")
        nrm.h_out, nrm.ldho = h_out.data_ptr(), h_out.stride(0)
    if xn_out is not None:
        nrm.xn_out, nrm.ldxo = xn_out.data_ptr(), xn_out.stride(0)
    nrm.f16 = int(bool(f16))
    p = W4Params(qw.data_ptr(), scales.data_ptr(), None, out.data_ptr(), None, None, M, Kp, Mp, Kp, N,
                 0, out.stride(0), EPI_SWIGLU if swiglu else EPI_NONE, 0, 0)
    return Job(p, nrm, out.device, (h_in, delta, norm_w, qw, scales, out, h_out, xn_out, tok))


def gemv_chain(jobs, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1, blocks_per_sm=0, min_units=4):
    """Not in the reference: run 1..4 jobs (`job`, `job_fused`) that depend on each other only
    through their tensors as ONE launch, with a grid-wide barrier between consecutive jobs. The
    results are bit-identical to launching them one by one with the same options; what is saved
    is the start-up of a kernel per matrix (the weight stream of job j + 1 is requested while job
    j finishes)."""
    jobs = list(jobs)
    _req(1 <= len(jobs) <= 4, "a chain holds 1..4 jobs")
    _req(all(j.dev == jobs[0].dev for j in jobs), "all jobs of a chain live on one device")
    _launch(jobs, _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units), "gemv_w4 chain")


def gemv(x, qw, scales, out, M, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1,
         blocks_per_sm=0, min_units=4):
    """out[N, M] = x[N, K] @ W~^T (W packed by quant.quantize_w4)."""
    _launch([job(x, qw, scales, out, M)],
            _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units), "gemv_w4")


def gemv_swiglu(x, qw, scales, out, I, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1,
                blocks_per_sm=0, min_units=4):
    """out[N, I] = silu(x @ Wg^T) * (x @ Wu^T) (packed by quant.quantize_w4_gate_up)."""
    _launch([job(x, qw, scales, out, I, swiglu=True)],
            _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units), "gemv_w4")


def gemv_partial(x, qw, scales, out32, M, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1,
                 blocks_per_sm=0, min_units=4):
    """Not in the reference: `out32` is fp32 [N, M] and receives the unrounded sums -- one rank's
    partial result of a matrix split along K over tensor-parallel ranks."""
    _req(out32.dtype == torch.float32, "out32 must be fp32")
    _launch([job(x, qw, scales, out32, M, allow_f32_out=True)],
            _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units), "gemv_w4")


def gemv_fused(h_in, delta, norm_w, eps, qw, scales, out, M, *, h_out=None, xn_out=None, tok=None,
               swiglu=False, f16=False, warps=0, unroll=0, ksplit=0, pdl=True, variant=0, mode=-1,
               blocks_per_sm=0, min_units=4):
    """Not in the reference: out = gemv(RMSNorm1p(h_in + delta) * (1 + norm_w)) in one launch.

    h_in bf16 [N, K]; delta bf16 [N, K] or None; h_out (optional, must not alias h_in) receives
    bf16(h_in + delta) and xn_out (optional) the normed rows. With `tok` (int32 [>= N]) h_in is an
    embedding table [V, K] and row r is table[tok[r]]. Same arithmetic as `_C.rmsnorm1p` followed
    by `gemv`."""
    _launch([job_fused(h_in, delta, norm_w, eps, qw, scales, out, M, h_out=h_out, xn_out=xn_out, tok=tok,
                       swiglu=swiglu, f16=f16)],
            _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units), "gemv_w4 fused")


def norm_rows(h_in, delta, norm_w, eps, xn_out, h_out=None, tok=None, xn16_out=None, warps=0, unroll=0, ksplit=0,
              pdl=True, variant=0, mode=-1, blocks_per_sm=0, min_units=4):
    """Not in the reference: the prologue of `gemv_fused` as a launch of its own (one block per row),
    bit-identical to it for the same launch options: xn_out = RMSNorm1p(h_in + delta) * (1 + w),
    h_out = bf16(h_in + delta) (may alias h_in). `norm_rows` + `gemv` == `gemv_fused`.
    xn16_out (fp16 [N, K], optional) receives the same rows as fp16: the input of a GEMV job with
    fp16 activations, which equals `gemv_fused(f16=True)`."""
    bf = torch.bfloat16
    _req(xn_out.is_cuda and xn_out.dtype == bf and xn_out.dim() == 2 and xn_out.stride(1) == 1, "xn_out bf16 [N, K]")
    N, K = xn_out.shape
    _req(1 <= N <= MAX_GEMM_ROWS and K % 8 == 0 and norm_w.dtype == bf and norm_w.numel() == K and
         norm_w.is_contiguous(), "N in 1..64, K % 8 == 0, norm_w [K]")
    _req(h_in.is_cuda and h_in.dtype == bf and h_in.dim() == 2 and h_in.stride(1) == 1 and h_in.size(1) == K, "h_in [*, K]")
    nrm = W4Norm()
    nrm.h_in, nrm.ldh, nrm.norm_w, nrm.eps = h_in.data_ptr(), h_in.stride(0), norm_w.data_ptr(), float(eps)
    nrm.xn_out, nrm.ldxo = xn_out.data_ptr(), xn_out.stride(0)
    if tok is not None:
        _req(tok.dtype == torch.int32 and tok.is_contiguous() and tok.numel() >= N and h_in.is_contiguous(), "tok int32 [>= N]")
        nrm.tok, nrm.vocab = tok.data_ptr(), h_in.size(0)
    else:
        _req(h_in.size(0) == N, "h_in must have N rows")
    for name, t in (("delta", delta), ("h_out", h_out)):
        if t is not None:
            _req(t.is_cuda and t.dtype == bf and t.dim() == 2 and t.stride(1) == 1 and t.shape == (N, K), f"{name} bf16 [N, K]")
    if delta is not None:
        nrm.delta, nrm.ldd = delta.data_ptr(), delta.stride(0)
    if h_out is not None:
        nrm.h_out, nrm.ldho = h_out.data_ptr(), h_out.stride(0)
    if xn16_out is not None:
        _req(xn16_out.is_cuda and xn16_out.dtype == torch.float16 and xn16_out.shape == (N, K) and
             xn16_out.stride(1) == 1, "xn16_out fp16 [N, K]")
        nrm.xn16_out, nrm.ldx16 = xn16_out.data_ptr(), xn16_out.stride(0)
    cfg = _cfg(warps, unroll, ksplit, pdl, variant, mode, blocks_per_sm, min_units)
    check(lib.qe_w4_norm_rows(C.byref(nrm), N, K, C.byref(cfg), torch.cuda.current_stream().cuda_stream), "norm_rows")


MAX_GEMM_ROWS = 64
_gemm_scratch: dict[int, tuple] = {}


def gemm(x, qw, scales, out, M, swiglu=False, pdl=True, variant=0):
    """Not in the reference (which prefills in passes of at most 8 rows through `gemv`): the same
    product for N = 1..64 rows with the matrix read from HBM once for all of them
    (qe_w4_gemm). out may be bf16 or, without SwiGLU, fp32 (unrounded sums). Needs K == Kp and
    16-byte aligned rows of x. A row agrees with `gemv` to fp32 rounding, not bit for bit (the
    groups of a tile are added in another order); results do not depend on N. variant 0: tcgen05
    with the accumulator in tensor memory; variant 1: the mma.sync kernel (needs Kp / 128 even)."""
    for t in (x, qw, scales, out):
        _req(isinstance(t, torch.Tensor) and t.is_cuda, "CUDA tensors")
    out_f32 = out.dtype == torch.float32 and not swiglu
    _req(x.dtype == torch.bfloat16 and (out.dtype == torch.bfloat16 or out_f32), "x bf16, out bf16 (or fp32 sums)")
    Mp, Kp = _packed(qw, scales)
    _req(x.dim() == 2 and out.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1, "x [N,K], out [N,M] rows")
    N, K, M = x.size(0), x.size(1), int(M)
    _req(1 <= N <= MAX_GEMM_ROWS and out.size(0) == N and out.size(1) == M, "N in 1..64 and out [N, M]")
    _req(K == Kp, "gemm needs K == Kp")
    _req(variant in (0, 1) and (variant == 0 or (Kp // 128) % 2 == 0), "variant 1 needs an even number of 128-k groups")
    _req(x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "gemm needs 16-byte aligned rows of x")
    _req((Mp // 2 - 8 < M <= Mp // 2) if swiglu else (Mp - 16 < M <= Mp), "out width must match packed rows")
    _req(x.data_ptr() != out.data_ptr(), "in-place not supported")
    p = W4Params(qw.data_ptr(), scales.data_ptr(), x.data_ptr(), out.data_ptr(), None, None, M, K, Mp, Kp, N,
                 x.stride(0), out.stride(0), EPI_SWIGLU if swiglu else EPI_NONE, int(out_f32), 0)
    cfg = W4Cfg(0, 0, 0, int(bool(pdl)), int(variant), -1, 0, 4)
    plan = W4Plan()
    check(lib.qe_w4_plan_gemm(C.byref(p), C.byref(cfg), C.byref(plan)), "gemm plan", kernels=0)
    if plan.ws_floats:  # a matrix of few rows is split along K: scratch of its own (the GEMV's must stay zero)
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        W = _gemm_scratch.get(dev)
        if W is None or W[0].numel() < plan.ws_floats or W[1].numel() < plan.counters:
            _req(not torch.cuda.is_current_stream_capturing(),
                 "gemm scratch would have to grow during graph capture: run the shape once eagerly first")
            W = (torch.empty(max(plan.ws_floats, 1 << 20), dtype=torch.float32, device=x.device),
                 torch.zeros(max(plan.counters, 1 << 10), dtype=torch.int32, device=x.device), W)  # old ones stay alive
            _gemm_scratch[dev] = W
        p.ws, p.counters = W[0].data_ptr(), W[1].data_ptr()
    code = lib.qe_w4_gemm(C.byref(p), C.byref(cfg), torch.cuda.current_stream().cuda_stream)
    _req(code != -22, "gemm: argument combination not supported by the kernel")
    _req(code == 0, f"gemm launch failed: CUDA error {code}")
    launches[0] += 1


def auto_ksplit(Mp, Kp, N, warps=8):
    return int(lib.qe_w4_auto_ksplit(int(Mp), int(Kp), int(N), int(warps)))


def ring_error():
    """Sticky error word of the weight rings' bounded barrier waits (0 = none); synchronises."""
    return int(lib.qe_w4_ring_error())


def clear_error():
    lib.qe_w4_clear_error()


def gemv_static(x, qw, scales, out, M, swiglu=False, warps=0, unroll=0, ksplit=0, variant=0, mode=-1,
                blocks_per_sm=0, min_units=4):
    """The W4 GEMV for callers that must not allocate (no counterpart in the reference).

    `gemv` keeps its partial-sum scratch in torch tensors that may have to grow, i.e. it can reach
    the CUDA allocator. A host that runs where allocation is off limits -- inside another runtime's
    callback, between the capture and the replay of a graph, under a memory pool it does not own --
    calls this instead: the scratch is a fixed array inside the library (about 4.1 MiB per GPU),
    nothing is allocated, and a shape whose launch plan needs more than that array raises
    RuntimeError. The first call on a device resolves the array's address and should come before
    any stream capture. All calls share the array, so calls that overlap on the GPU race: keep
    them on one stream. Same validation and results as `gemv` / `gemv_swiglu`."""
    for t in (x, qw, scales, out):
        _req(isinstance(t, torch.Tensor) and t.is_cuda, "CUDA tensors")
    _req(x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "x and out must be bf16")
    Mp, Kp = _packed(qw, scales)
    _req(x.dim() == 2 and out.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1, "x [N,K], out [N,M] rows")
    N, K, M = x.size(0), x.size(1), int(M)
    _req(1 <= N <= 8 and out.size(0) == N and out.size(1) == M, "N in 1..8 and out [N, M]")
    _req(Kp - 128 < K <= Kp, "shapes disagree")
    _req((Mp // 2 - 8 < M <= Mp // 2) if swiglu else (Mp - 16 < M <= Mp), "out width must match packed rows")
    p = W4Params(qw.data_ptr(), scales.data_ptr(), x.data_ptr(), out.data_ptr(), None, None, M, K, Mp, Kp, N,
                 x.stride(0), out.stride(0), EPI_SWIGLU if swiglu else EPI_NONE, 0, 0)
    cfg = W4Cfg(int(warps), int(unroll), int(ksplit), 0, int(variant), int(mode), int(blocks_per_sm), int(min_units))
    code = lib.qe_w4_gemv_static(C.byref(p), C.byref(cfg), torch.cuda.current_stream().cuda_stream)
    _req(code != -28, "gemv_static: this shape needs more scratch than the library's fixed array "
                      "(1 Mi partial-sum floats, 16 Ki tile counters); use gemv with caller scratch")
    _req(code == 0, f"gemv_static failed: error {code}")
    launches[0] += 1
