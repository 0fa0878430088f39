"""The C ABI: the shared library loads and exports every symbol include/qengine_b200.h declares,
and the ctypes signature table covers exactly those symbols. No compute calls (CPU only)."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "qengine_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from qengine_b200 import _lib
    names = _declared()
    assert len(names) >= 24
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_struct_layouts_match_header():
    """Field order of the ctypes mirrors follows the header's struct definitions."""
    from qengine_b200 import _lib
    text = (ROOT / "include" / "qengine_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)

    def fields(name):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, flags=re.S).group(1)
        out = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            out += [re.sub(r"[\s\*]", "", v) for v in decl.split(",")][0:1] and \
                   [re.sub(r"^.*[\s\*]", "", v.strip()) for v in decl.split(",")]
        return out

    assert fields("qe_w4_params") == [f[0] for f in _lib.W4Params._fields_]
    assert fields("qe_w4_cfg") == [f[0] for f in _lib.W4Cfg._fields_]
    assert fields("qe_w4_plan") == [f[0] for f in _lib.W4Plan._fields_]


def test_abi_version_and_plan_without_gpu():
    from qengine_b200 import _lib
    assert _lib.lib.qe_abi_version() == 3
    assert _lib.lib.qe_w4_auto_ksplit(5120, 17408, 1, 8) == 1


def test_fp16_activation_preconditions_are_checked_at_the_boundary():
    """qe_w4_gemv with x_f16 = 1 must refuse what its vector path cannot serve (unpadded K,
    misaligned rows, odd strides) with QE_ERR_ARG (-22) before anything is launched."""
    import ctypes as C
    from qengine_b200 import _lib
    buf = (C.c_char * 4096)()
    base = (C.addressof(buf) + 255) & ~255
    cfg = _lib.W4Cfg()
    _lib.lib.qe_w4_cfg_default(C.byref(cfg))

    def call(K, Kp, x, ldx):
        p = _lib.W4Params(base, base, x, base, base, base, 16, K, 16, Kp, 1, ldx, 16, 0, 0, 1)
        return _lib.lib.qe_w4_gemv(C.byref(p), C.byref(cfg), None)

    assert call(200, 256, base, 256) == -22      # K != Kp
    assert call(256, 256, base + 2, 256) == -22  # row start not 16-byte aligned
    assert call(256, 256, base, 260) == -22      # stride not a multiple of 8 elements


def test_gemm_plan_and_argument_checks_without_gpu():
    """qe_w4_plan_gemm is shape arithmetic (148 SMs assumed without a device): matrices with fewer
    128-row super-tiles than half the SMs are split along K and need scratch, the others do not.
    qe_w4_gemm refuses what its kernels cannot serve with QE_ERR_ARG (-22) before any launch."""
    import ctypes as C
    from qengine_b200 import _lib
    cfg = _lib.W4Cfg()
    _lib.lib.qe_w4_cfg_default(C.byref(cfg))

    def plan(M, K, epilogue=0, variant=0):
        p = _lib.W4Params(None, None, None, None, None, None, M, K, -(-M // 16) * 16, K, 64, K, M, epilogue, 0, 0)
        c = _lib.W4Cfg(0, 0, 0, 1, variant, -1, 0, 4)
        out = _lib.W4Plan()
        assert _lib.lib.qe_w4_plan_gemm(C.byref(p), C.byref(c), C.byref(out)) == 0
        return out

    down = plan(5120, 17408)          # 40 super-tiles -> 3 parts of K
    assert (down.grid_x, down.ws_floats, down.counters, down.threads) == (120, 40 * 3 * 64 * 128, 40, 17 * 32)
    big = plan(2 * 17408, 5120, epilogue=1)  # gate/up: 272 super-tiles, never split
    assert (big.grid_x, big.ws_floats, big.counters) == (148, 0, 0)
    assert plan(16480, 5120).ws_floats == 0 and plan(16480, 5120).grid_x == 129
    assert plan(5120, 17408, variant=1).ws_floats == 0  # the mma.sync kernel never splits

    buf = (C.c_char * 4096)()
    base = (C.addressof(buf) + 255) & ~255

    def call(N, K, Kp, x, ldx, x_f16=0):
        p = _lib.W4Params(base, base, x, base, None, None, 16, K, 16, Kp, N, ldx, 16, 0, 0, x_f16)
        return _lib.lib.qe_w4_gemm(C.byref(p), C.byref(cfg), None)

    assert call(65, 256, 256, base, 256) == -22      # more than 64 rows
    assert call(8, 200, 256, base, 256) == -22       # K != Kp
    assert call(8, 256, 256, base + 2, 256) == -22   # rows not 16-byte aligned
    assert call(8, 256, 256, base, 260) == -22       # stride not a multiple of 8 elements
    assert call(8, 256, 256, base, 256, x_f16=1) == -22
