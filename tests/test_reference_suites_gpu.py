"""The reference's own acceptance suites for the two extensions, run unmodified against this
library: baseline/build_ref.py lays out a `qengine` package whose `_C` and `_w4` modules re-export
qengine_b200 (baseline/shim/) beside unmodified copies of tests/test_gemv_w4.py and
tests/test_kernels.py of the reference. Skipped when that tree has not been built."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
SHIM = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "shim"


def _run(test_file: str, timeout: int, deselect=()):
    if not (SHIM / "tests" / test_file).exists():
        pytest.skip("baseline/_ref/shim is not built (python baseline/build_ref.py)")
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    skip = [f"--deselect={test_file}::{name}" for name in deselect]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", *skip, test_file],
                       cwd=SHIM / "tests", env=env, capture_output=True, text=True, timeout=timeout)
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "skipped" not in r.stdout.splitlines()[-1], tail


def test_reference_w4_gemv_suite_passes_on_this_library():
    _run("test_gemv_w4.py", 1500)


def test_reference_kernel_suite_passes_on_this_library():
    # test_rope_matches_hf_mrope compares the reference's torch model with Hugging Face's rotary
    # embedding built from a checkpoint directory on disk; it calls no kernel and needs files
    # that are not available offline.
    _run("test_kernels.py", 900, deselect=["test_rope_matches_hf_mrope"])
