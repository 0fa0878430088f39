"""The reference arm of bench.py (whole tokens on the host cores through the reference's torch path,
or the oracle's restatement when oracle/_ref has not been built) runs without a GPU: one JSON line
with the contract's keys; ranks other than 0 print nothing and exit 0."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _run(env_extra, *args):
    env = dict(os.environ, **env_extra)
    # a cut-down shape (4 layers, 4,096-row head) keeps the CPU suite short; the arm itself is the same
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1", "--layers", "4", "--ref-vocab", "4096", *args],
                          capture_output=True, text=True, env=env, timeout=600)


def test_reference_arm_line():
    r = _run({})
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["value"] > 0
    assert line["higher_is_better"] is True and line["gpu_launches"] == 0
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert "workload" in line["config"] and line["ms_per_step"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_nothing():
    r = _run({"RANK": "1", "WORLD_SIZE": "2"}, "--gpus", "2")
    assert r.returncode == 0 and r.stdout.strip() == ""
