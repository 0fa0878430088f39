"""The prepared-weights cache directory (reference layout) and the GPTQ-grid repack, on CPU."""
import pickle
import pickletools

import pytest
import torch

from qengine_b200 import cache, quant
from qengine_b200.synth import build_model, tiny_config


def _same(a, b):
    if isinstance(a, quant.W4Packed):
        return (isinstance(b, quant.W4Packed) and torch.equal(a.qw, b.qw) and torch.equal(a.scales, b.scales)
                and (a.M, a.K, a.gate_up) == (b.M, b.K, b.gate_up))
    if isinstance(a, torch.Tensor):
        return a.dtype == b.dtype and torch.equal(a, b)
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, list):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    return a == b


def test_round_trip_in_the_reference_layout(tmp_path):
    cfg = tiny_config()
    W = build_model(cfg, seed=3)
    d = cache.save_cache(cache.cache_path(tmp_path, "tiny"), W)
    assert d.name == "tiny-w4-rtn-g128-v1"
    names = sorted(p.name for p in d.iterdir())
    assert names == sorted(["COMPLETE", "top.pt", "lm_head.pt", "mtp.pt"]
                           + [f"layer{i:02d}.pt" for i in range(cfg.layers)])
    back = cache.load_cache(d, cfg)
    for k in ("embed", "final_norm", "lm_head", "layers", "mtp"):
        assert _same(W[k], back[k]), k
    # the files name the reference's class, so its engine can unpickle them
    import zipfile
    with zipfile.ZipFile(d / "lm_head.pt") as z:
        pkl = z.read([n for n in z.namelist() if n.endswith("data.pkl")][0])
    ops = [(op.name, arg) for op, arg, _ in pickletools.genops(pkl)]
    text = " ".join(str(a) for _, a in ops if isinstance(a, str))
    assert "qengine.quant" in text and "W4Packed" in text and "qengine_b200" not in text
    # and the alias used for writing is gone again
    import sys
    assert "qengine.quant" not in sys.modules
    assert quant.W4Packed.__module__ == "qengine_b200.quant"
    assert pickle.loads(pickle.dumps(quant.W4Packed(torch.zeros(1), torch.zeros(1), 1, 1))).M == 1


def test_partial_directories_are_refused(tmp_path):
    cfg = tiny_config()
    W = build_model(cfg, seed=4)
    d = cache.save_cache(tmp_path / "m", W)
    (d / "COMPLETE").unlink()
    with pytest.raises(FileNotFoundError):
        cache.load_cache(d, cfg)
    (d / "COMPLETE").write_text("x\n")
    (d / "layer01.pt").unlink()
    with pytest.raises(FileNotFoundError):
        cache.load_cache(d, cfg)


def test_config_json_round_trip(tmp_path):
    cfg = tiny_config()
    cache.write_config(tmp_path, cfg)
    assert cache.config_from_dir(tmp_path) == cfg


def test_grid_repack_is_exact_on_grid_matrices():
    g = torch.Generator().manual_seed(11)
    M, K = 40, 384
    W = torch.randn(M, K, generator=g) * 0.02
    W[3, 128:256] = 0          # an all-zero group
    p0 = quant.quantize_w4(W)
    on_grid = quant.dequantize_w4(p0)                    # fp32 values code * scale
    stored = on_grid.to(torch.bfloat16)                  # how a checkpoint holds them
    p1, stats = cache.pack_from_grid(stored)
    # the packed matrix multiplies with values that round to the stored ones
    again = quant.dequantize_w4(p1)
    assert torch.equal(again.to(torch.bfloat16), stored)
    assert stats["exact_frac"] == 1.0
    # a group that never uses code -8 or 7 still comes back exactly (no re-quantisation drift)
    codes = torch.randint(5, 12, (16, 128), generator=g)
    s = torch.full((16, 1), 0.0123).to(torch.float16)
    Wg = ((codes - 8).float() * s.float()).to(torch.bfloat16)
    p2, st2 = cache.pack_from_grid(Wg)
    assert torch.equal(quant.dequantize_w4(p2).to(torch.bfloat16), Wg) and st2["exact_frac"] == 1.0
    with pytest.raises(ValueError):
        cache.pack_from_grid(torch.zeros(16, 100))


def test_grid_repack_against_the_reference():
    """tests/golden/grid_repack.pt holds the reference's prepare_from_grid on a GPTQ-style grid.
    Same codes everywhere; the same scales wherever the reference reproduced the stored values
    (its scale search is narrower and misses a few groups, which this one recovers exactly)."""
    from pathlib import Path
    g = torch.load(Path(__file__).resolve().parent / "golden" / "grid_repack.pt")
    p, st = cache.pack_from_grid(g["grid"])
    assert torch.equal(p.qw, g["qw"])
    M, G = g["exact_groups"].shape
    mine = p.scales.permute(0, 2, 1).reshape(M, G)
    ref = g["scales"].permute(0, 2, 1).reshape(M, G)
    ok = g["exact_groups"]
    assert torch.equal(mine[ok], ref[ok])
    assert 0.5 < float(ok.float().mean()) < 1.0 and st["exact_frac"] == 1.0
    assert torch.equal(quant.dequantize_w4(p).to(torch.bfloat16), g["grid"])


def test_files_pickled_with_the_reference_class_load_here(tmp_path):
    """The other direction of the interchange: layer files whose matrices are instances of the
    reference's own `qengine.quant.W4Packed` (as its engine writes them, python/qengine/engine.py:
    224-229) load into this package's class. Needs the unmodified copy of the reference package
    that baseline/build_ref.py lays out (its quant module has no CUDA dependency)."""
    import subprocess
    import sys
    from pathlib import Path
    ref_pkg = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "shim" / "python"
    if not (ref_pkg / "qengine" / "quant.py").exists():
        pytest.skip("baseline/_ref is not built")
    cfg = tiny_config()
    W = build_model(cfg, seed=9)
    d = cache.save_cache(tmp_path / "ours", W)
    # re-save every file from a separate interpreter in which qengine.quant is the reference's module
    script = f"""
import sys, torch
sys.path.insert(0, {str(ref_pkg)!r})
import importlib.util, types
pkg = types.ModuleType("qengine"); pkg.__path__ = [{str(ref_pkg / 'qengine')!r}]; sys.modules["qengine"] = pkg
spec = importlib.util.spec_from_file_location("qengine.quant", {str(ref_pkg / 'qengine' / 'quant.py')!r})
m = importlib.util.module_from_spec(spec); sys.modules["qengine.quant"] = m; spec.loader.exec_module(m)
from pathlib import Path
src, dst = Path({str(d)!r}), Path({str(tmp_path / 'theirs')!r}); dst.mkdir()
n = 0
for f in sorted(src.glob("*.pt")):
    obj = torch.load(f, weights_only=False)
    def count(o):
        global n
        if isinstance(o, m.W4Packed): n += 1
        elif isinstance(o, dict): [count(v) for v in o.values()]
    count(obj)
    torch.save(obj, dst / f.name)
(dst / "COMPLETE").write_text("w4-rtn-g128-v1\\n")
print(n)
"""
    r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert int(r.stdout.strip()) == 1 + 4 * cfg.layers + 5   # lm_head, 4 per layer, 5 in the MTP layer
    back = cache.load_cache(tmp_path / "theirs", cfg)
    for k in ("embed", "final_norm", "lm_head", "layers", "mtp"):
        assert _same(W[k], back[k]), k
