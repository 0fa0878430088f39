"""Build libqengine_b200.so (hand-written sm_100a CUDA behind a C ABI) in-tree with nvcc.

    python -m qengine_b200.build [--force] [--verbose]

Each `csrc/*.cu` is compiled to an object (in parallel) and linked into
`qengine_b200/libqengine_b200.so`. Objects are rebuilt when a source or header is newer.
No torch headers are involved: the library depends on the CUDA runtime only.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ = PKG / "build"
LIB = PKG / "libqengine_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]


def nvcc() -> str:
    exe = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found (set NVCC)")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    cmd = [nvcc(), *ARCH_FLAGS, *COMMON, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    (OBJ / (src.stem + ".ptxas.log")).write_text(r.stderr)
    if verbose:
        print(r.stderr)
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    hdr = _newest_header()
    todo, objs = [], []
    for s in sources():
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr):
            todo.append(s)
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose), todo))
    if todo or not LIB.exists():
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
