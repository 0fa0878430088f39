"""Golden vectors for the GPTQ-grid repack: outputs of the reference's own
W4Linear.prepare_from_grid (python/qengine/engine.py:117-180), which lives in the module that
imports the reference's CUDA extension. Run after `python baseline/build_ref.py` (that recipe
compiles the extension next to an unmodified copy of the package); everything runs on the CPU.

    python tests/golden/make_grid_golden.py

Writes tests/golden/grid_repack.pt: a seeded matrix on the int4 grid stored as bf16 (every group
reaches code 7 or -8, as a GPTQ-quantised group does), the reference's packed result and, per
group, whether the reference reproduced the stored values bit for bit (its scale search covers two
fp16 steps around absmax / 7 and absmax / 8, which does not always contain the scale)."""
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
NATIVE = HERE.parents[1] / "baseline" / "_ref" / "native" / "python"


def main():
    if not (NATIVE / "qengine" / "engine.py").exists():
        raise SystemExit("build the reference first: python baseline/build_ref.py")
    sys.path.insert(0, str(NATIVE))
    from qengine import quant as RQ
    from qengine.engine import W4Linear
    g = torch.Generator().manual_seed(7)
    M, K = 64, 512
    s = (torch.rand(M, K // 128, generator=g) * 0.02 + 0.002).to(torch.float16)
    q = torch.randint(-8, 8, (M, K // 128, 128), generator=g)
    q[:, :, 0] = 7
    q[::3, :, 1] = -8
    grid = (q.float() * s.float().unsqueeze(-1)).reshape(M, K).to(torch.bfloat16)
    packed, stats = W4Linear().prepare_from_grid(grid)
    back = RQ.dequantize_w4(packed).to(torch.bfloat16)
    exact = (back == grid).view(M, K // 128, 128).all(-1)
    torch.save({"grid": grid, "qw": packed.qw, "scales": packed.scales, "exact_groups": exact,
                "exact_frac": stats["exact_frac"]}, HERE / "grid_repack.pt")
    print(f"wrote grid_repack.pt: reference exact on {int(exact.sum())} of {exact.numel()} groups")


if __name__ == "__main__":
    main()
