"""Recipe for oracle/_ref/: the reference's own torch model, made importable next to the oracle.

The reference's CPU path for the decode step is plain Python (python/qengine/reference.py and
python/qengine/quant.py of manaspros/qengine), so "building" it means placing those two modules,
unmodified, in a package of their own under oracle/_ref/ (git-ignored: reference sources never
enter this repository's history; the directory travels with the built artefacts). The package's
__init__ is written here because the reference's own __init__ pulls in its CUDA extension.

    python -m oracle.build_ref [--reference DIR]

DIR defaults to $QENGINE_REFERENCE_DIR, else a checkout named `reference` beside this repository.
With oracle/_ref in place, tests and the CPU arm of bench.py can time and compare against the
reference's functions (`load()`); without it they use the oracle's restatement.
"""
from __future__ import annotations

import argparse
import importlib
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
FILES = ("reference.py", "quant.py")


def find_reference() -> Path | None:
    cands = [os.environ.get("QENGINE_REFERENCE_DIR"), HERE.parents[1] / "reference"]
    for c in cands:
        if c and (Path(c) / "python" / "qengine" / "reference.py").exists():
            return Path(c)
    return None


def build(reference: Path | None = None) -> bool:
    """Copy the two modules when a checkout is available; True if oracle/_ref is usable."""
    ref = Path(reference) if reference else find_reference()
    if ref is not None:
        pkg = DEST / "qengine_ref"
        pkg.mkdir(parents=True, exist_ok=True)
        for f in FILES:
            shutil.copyfile(ref / "python" / "qengine" / f, pkg / f)
        (pkg / "__init__.py").write_text("# the reference's torch model and quantiser, unmodified copies\n")
    return all((DEST / "qengine_ref" / f).exists() for f in FILES)


def load():
    """(reference module, quant module) from oracle/_ref, or None when it has not been built."""
    if not all((DEST / "qengine_ref" / f).exists() for f in FILES):
        return None
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    return importlib.import_module("qengine_ref.reference"), importlib.import_module("qengine_ref.quant")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    print("oracle/_ref ready:", build(ap.parse_args().reference))
