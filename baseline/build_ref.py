"""Recipe: the unmodified reference, built for sm_100a, under baseline/_ref/ (git-ignored).

    python baseline/build_ref.py [--reference DIR] [--no-native]

It produces two trees, each laid out like the reference checkout (`python/qengine`, `tests`), so
that the reference's own `tests/conftest.py` finds the package next to it:

  baseline/_ref/native/   the reference as it is: its Python package plus its two extensions
                          (`qengine._C` from bindings.cpp + basic.cu + gdn.cu + attn.cu and
                          `qengine._w4` from gemv_w4.cu + gemv_w4_bind.cpp) compiled for sm_100a
                          with the flags of its scripts/build_w4.sh and python/build_c.py. It is
                          the same-box GPU comparator: `bench.py --impl reference-gpu` runs the
                          reference engine on it.
  baseline/_ref/shim/     the reference's Python package with `_C` and `_w4` replaced by the
                          two files of baseline/shim/, which re-export qengine_b200. Its copy of
                          tests/test_gemv_w4.py and tests/test_kernels.py therefore exercises this
                          repository's library, unmodified (tests/test_reference_suites_gpu.py).

Sources are compiled from where they lie in the reference checkout; only Python files and the two
test files are copied. Nothing under baseline/_ref/ is committed.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
sys.path.insert(0, str(HERE.parent))

PY_FILES = ["__init__.py", "quant.py", "reference.py", "engine.py", "draft_vocab.py"]
TEST_FILES = ["conftest.py", "test_gemv_w4.py", "test_kernels.py"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _copy_tree_skeleton(ref: Path, root: Path):
    (root / "python" / "qengine").mkdir(parents=True, exist_ok=True)
    (root / "tests").mkdir(parents=True, exist_ok=True)
    for f in PY_FILES:
        shutil.copyfile(ref / "python" / "qengine" / f, root / "python" / "qengine" / f)
    for f in TEST_FILES:
        shutil.copyfile(ref / "tests" / f, root / "tests" / f)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout[-3000:] + r.stderr[-6000:])
        raise SystemExit(f"build step failed ({r.returncode})")


def build_native(ref: Path, root: Path):
    import torch
    from torch.utils.cpp_extension import CUDA_HOME
    cuda = Path(CUDA_HOME or "/usr/local/cuda")
    nvcc = str(cuda / "bin" / "nvcc")
    tdir = Path(torch.__file__).parent
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    csrc = ref / "csrc"
    obj = root / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
           f"-I{sysconfig.get_paths()['include']}", f"-I{cuda / 'include'}", f"-I{csrc}"]
    link = [f"-L{tdir / 'lib'}", f"-L{cuda / 'lib64'}", f"-Wl,-rpath,{tdir / 'lib'}",
            f"-Wl,-rpath,{cuda / 'lib64'}", "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
            "-ltorch_python", "-lcudart"]

    def cu(name):
        o = obj / (name + ".o")
        _run([nvcc, "-O3", "-std=c++20", *ARCH, "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              f"-I{csrc}", "-c", str(csrc / name), "-o", str(o)])
        return str(o)

    def cpp(name, module):
        o = obj / (name + ".o")
        _run(["g++", "-O2", "-std=c++20", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              f"-DTORCH_EXTENSION_NAME={module}", "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", str(csrc / name),
              "-o", str(o)])
        return str(o)

    pkg = root / "python" / "qengine"
    objs = [cu("gemv_w4.cu"), cpp("gemv_w4_bind.cpp", "_w4")]
    _run(["g++", "-shared", "-o", str(pkg / ("_w4" + ext)), *objs, *link])
    objs = [cu("basic.cu"), cu("gdn.cu"), cu("attn.cu"), cpp("bindings.cpp", "_C")]
    _run(["g++", "-shared", "-o", str(pkg / ("_C" + ext)), *objs, *link])
    shutil.rmtree(obj)


def build(reference: str | None = None, native: bool = True) -> Path | None:
    """Returns baseline/_ref/ or None when no reference checkout is at hand (prebuilt trees, if
    any, are left alone)."""
    from oracle.build_ref import find_reference
    ref = Path(reference) if reference else find_reference()
    if ref is None or not (ref / "csrc" / "gemv_w4.cu").exists():
        return None
    _copy_tree_skeleton(ref, OUT / "shim")
    for f in ("_C.py", "_w4.py"):
        shutil.copyfile(HERE / "shim" / f, OUT / "shim" / "python" / "qengine" / f)
    if native:
        _copy_tree_skeleton(ref, OUT / "native")
        stamp = OUT / "native" / "BUILT"
        srcs = sorted((ref / "csrc").iterdir())
        newest = max(p.stat().st_mtime for p in srcs)
        if not stamp.exists() or stamp.stat().st_mtime < newest:
            build_native(ref, OUT / "native")
            stamp.write_text("sm_100a\n")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("QENGINE_REFERENCE_DIR"))
    ap.add_argument("--no-native", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, native=not a.no_native)
    print(out if out else "no reference checkout found; nothing built")
