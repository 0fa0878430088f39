"""ctypes loader for libqengine_b200.so (the C ABI declared in include/qengine_b200.h).

There is no fallback of any kind: if the shared library is missing or lacks a symbol the import
fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libqengine_b200.so"

c_int, c_long, c_float, c_void_p, c_size_t = C.c_int, C.c_long, C.c_float, C.c_void_p, C.c_size_t
P = c_void_p


class W4Params(C.Structure):
    """struct qe_w4_params"""
    _fields_ = [("qw", P), ("scales", P), ("x", P), ("out", P), ("ws", P), ("counters", P),
                ("M", c_int), ("K", c_int), ("Mp", c_int), ("Kp", c_int), ("N", c_int),
                ("ldx", c_long), ("ldo", c_long), ("epilogue", c_int), ("out_f32", c_int), ("x_f16", c_int)]


class W4Cfg(C.Structure):
    """struct qe_w4_cfg"""
    _fields_ = [("warps", c_int), ("unroll", c_int), ("ksplit", c_int), ("pdl", c_int),
                ("variant", c_int), ("mode", c_int), ("blocks_per_sm", c_int), ("min_units", c_int)]


class W4Norm(C.Structure):
    """struct qe_w4_norm"""
    _fields_ = [("h_in", P), ("tok", P), ("vocab", c_int), ("delta", P), ("norm_w", P), ("h_out", P),
                ("xn_out", P), ("ldh", c_long), ("ldd", c_long), ("ldho", c_long), ("ldxo", c_long),
                ("eps", c_float), ("f16", c_int), ("xn16_out", P), ("ldx16", c_long)]


class W4Plan(C.Structure):
    """struct qe_w4_plan"""
    _fields_ = [("mode", c_int), ("grid_x", c_int), ("grid_y", c_int), ("threads", c_int),
                ("ws_floats", c_long), ("counters", c_long)]


# name -> (restype, argtypes); must list every symbol of include/qengine_b200.h
SIGNATURES = {
    "qe_abi_version": (c_int, []),
    "qe_sm_count": (c_int, []),
    "qe_embed": (c_int, [P, P, P, c_int, c_int, c_int, c_long, P]),
    "qe_rmsnorm1p": (c_int, [P, P, P, P, c_int, c_int, c_long, c_long, c_long, c_float, P]),
    "qe_gemv_bf16": (c_int, [P, P, P, c_int, c_int, c_int, c_long, c_long, P]),
    "qe_swiglu": (c_int, [P, P, c_int, c_int, c_long, c_long, P]),
    "qe_argmax": (c_int, [P, c_int, c_int, c_long, P, P, c_int, P, P, P]),
    "qe_rmsnorm1p_parts": (c_int, [P, P, c_int, P, P, c_int, c_int, c_long, c_long, c_float, P]),
    "qe_argmax_v": (c_int, [P, c_int, c_int, c_long, P, P, c_int, P, P, P, c_int, P]),
    "qe_argmax_merge": (c_int, [P, P, c_int, c_int, P, P]),
    "qe_tp_block_bytes": (c_long, [c_int, c_int]),
    "qe_tp_alloc": (c_int, [c_long, P]),
    "qe_tp_free": (c_int, [P]),
    "qe_tp_export": (c_int, [P, P]),
    "qe_tp_import": (c_int, [P, P]),
    "qe_tp_unmap": (c_int, [P]),
    "qe_tp_comm_create": (c_int, [P, c_int, c_int, c_int, P]),
    "qe_tp_comm_destroy": (c_int, [P]),
    "qe_tp_set_timeout_ms": (c_int, [P, c_long]),
    "qe_tp_exchange_norm": (c_int, [P, P, P, P, P, P, c_int, c_long, c_long, c_long, c_long, c_float, P]),
    "qe_tp_exchange_argmax": (c_int, [P, P, P, c_int, P, P]),
    "qe_tp_error": (c_int, [P, P]),
    "qe_tp_clear_error": (c_int, [P]),
    "qe_accept": (c_int, [P, P, c_int, P, P, P, c_int, P]),
    "qe_commit": (c_int, [P, P, P, P, c_int, P]),
    "qe_accept_commit": (c_int, [P, P, c_int, P, P, P, c_int, P, c_int, P]),
    "qe_chain_draft": (c_int, [P, P, P, P, c_int, P]),
    "qe_mtp_select": (c_int, [P, P, c_int, P, c_long, P, c_int, P, P, P]),
    "qe_force_drafts": (c_int, [P, P, P, c_int, c_int, c_int, c_int, P]),
    "qe_gdn_step_n": (c_int, [P, P, P, P, c_long, P, P, P, P, P, P, P, P, P, P, P, c_long, c_int,
                              c_int, c_int, c_int, c_float, c_int, P]),
    "qe_attn_prep": (c_int, [P, P, P, c_long, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_float, P]),
    "qe_attn_decode": (c_int, [P, P, P, P, P, c_long, P, P, P, c_long, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_float, P]),
    "qe_attn_error": (c_int, []),
    "qe_set_pdl_trigger": (None, [c_int]),
    "qe_set_pdl_launch": (None, [c_int]),
    "qe_set_gdn_early": (None, [c_int]),
    "qe_set_gdn_phases": (None, [c_int]),
    "qe_l2_persist_limit": (c_int, [c_size_t]),
    "qe_stream_access_window": (c_int, [C.c_uint64, c_size_t, c_float, P]),
    "qe_w4_cfg_default": (None, [C.POINTER(W4Cfg)]),
    "qe_w4_plan_gemv": (c_int, [C.POINTER(W4Params), C.POINTER(W4Cfg), C.POINTER(W4Plan)]),
    "qe_w4_auto_ksplit": (c_int, [c_int, c_int, c_int, c_int]),
    "qe_w4_gemv": (c_int, [C.POINTER(W4Params), C.POINTER(W4Cfg), P]),
    "qe_w4_gemv_ex": (c_int, [C.POINTER(W4Params), C.POINTER(W4Norm), C.POINTER(W4Cfg), P]),
    "qe_w4_norm_rows": (c_int, [C.POINTER(W4Norm), c_int, c_int, C.POINTER(W4Cfg), P]),
    "qe_w4_gemv_chain": (c_int, [C.POINTER(C.POINTER(W4Params)), C.POINTER(C.POINTER(W4Norm)), c_int,
                                 C.POINTER(W4Cfg), P, P]),
    "qe_w4_ring_error": (c_int, []),
    "qe_w4_clear_error": (c_int, []),
    "qe_w4_gemv_static": (c_int, [C.POINTER(W4Params), C.POINTER(W4Cfg), P]),
    "qe_w4_gemm": (c_int, [C.POINTER(W4Params), C.POINTER(W4Cfg), P]),
    "qe_w4_plan_gemm": (c_int, [C.POINTER(W4Params), C.POINTER(W4Cfg), C.POINTER(W4Plan)]),
}


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m qengine_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


# Number of kernels this process has enqueued through the wrappers (eagerly or into a graph being
# captured). The engine reads it around a capture to know how many kernel nodes a graph holds.
launches = [0]


def check(code: int, what: str, kernels: int = 1) -> None:
    """Turn a launcher's return code into RuntimeError (the reference throws via TORCH_CHECK)."""
    if code == 0:
        launches[0] += kernels
        return
    if code == -22:
        raise RuntimeError(f"{what}: argument not supported by the kernels")
    raise RuntimeError(f"{what}: CUDA error {code}")
