"""Index arithmetic of the prefill GEMM (qengine_b200/csrc/w4_gemm.cu), restated in Python and
checked exhaustively on the CPU: every 1 KB unit of a matrix is multiplied exactly once, by the
warp that also requested it from HBM in that order, for both kernels and for the shapes that
exercise their corner cases. A change of the device-side split has to keep these invariants.
"""
from __future__ import annotations

import pytest

SMS = 148
SHAPES = [(1, 2), (2, 4), (3, 8), (5, 40), (16, 48), (147, 4), (148, 2), (149, 136), (320, 48), (320, 136),
          (896, 40), (1030, 40), (2176, 40), (2368, 2), (2369, 4), (5000, 2), (15520, 40), (63, 16), (13, 24)]


def share_begin(total, parts, i):
    per, rem = divmod(total, parts)
    return i * per + min(i, rem)


@pytest.mark.parametrize("tiles,G", SHAPES)
@pytest.mark.parametrize("NW,GS,STAGES", [(16, 4, 2), (16, 2, 4)])
def test_mma_sync_kernel_covers_every_unit_once(tiles, G, NW, GS, STAGES):
    """w4_gemm_kernel: tiles per CTA, 1 / 2 / 4 warps per tile, rounds of NW / wpt tiles, slabs of GS
    groups; a warp's weight stages are the first my_it slabs of the CTA's walk."""
    if G % GS:
        pytest.skip("this geometry needs K / 128 to be a multiple of its slab")
    nctas = min(SMS, tiles)
    seen = set()
    for cta in range(nctas):
        T0 = share_begin(tiles, nctas, cta)
        nt = share_begin(tiles, nctas, cta + 1) - T0
        assert nt >= 1
        wpt = 1
        while wpt * 2 <= GS and nt * wpt * 2 <= NW:
            wpt *= 2
        RS, SPT = NW // wpt, G // GS
        n_it = -(-nt // RS) * SPT
        for warp in range(NW):
            tl, sub = divmod(warp, wpt)
            upw, j0 = GS // wpt, sub * (GS // wpt)
            my_it = (-(-(nt - tl) // RS) if tl < nt else 0) * SPT
            assert my_it <= n_it
            for q in range(my_it):
                rnd, s = divmod(q, SPT)
                assert rnd * RS + tl < nt
                u = (T0 + rnd * RS + tl) * G + s * GS + j0
                for i in range(upw):
                    assert u + i not in seen and (u + i) // G == T0 + rnd * RS + tl
                    seen.add(u + i)
    assert len(seen) == tiles * G


def kparts(tiles, G, swiglu=False):
    ST = (tiles + 7) // 8
    if swiglu or ST * 2 > SMS:
        return 1
    return max(1, min(SMS // ST, G // 8, 16))


@pytest.mark.parametrize("tiles,G", SHAPES)
def test_tensor_memory_kernel_steps_and_rings(tiles, G):
    """w4_gemm_tc_kernel: jobs (super-tile, part of K) round-robin over the CTAs; the steps of a CTA
    in order; warps 0..7 prepare the even steps, 8..15 the odd ones, tile = warp % 8; a warp
    requests its units from HBM in exactly the order in which it consumes them; with K split
    every CTA has one job at most, so a super-tile without all its tiles is always a last job."""
    KP = kparts(tiles, G)
    ST = (tiles + 7) // 8
    J = ST * KP
    nctas = min(SMS, J)
    assert KP == 1 or J <= SMS
    seen = set()
    for cta in range(nctas):
        nj = (J - cta + nctas - 1) // nctas if cta < J else 0
        steps = []  # (job index, tile0, g)
        for j in range(nj):
            jidx = cta + j * nctas
            st, part = divmod(jidx, KP)
            for g in range(share_begin(G, KP, part), share_begin(G, KP, part + 1)):
                steps.append((j, st * 8, g))
        assert all(b[0] - a[0] in (0, 1) for a, b in zip(steps, steps[1:]))
        for warp in range(16):
            par, ti = warp >> 3, warp & 7
            own = [s for z, s in enumerate(steps) if (z & 1) == par]
            valid = [s[1] + ti < tiles for s in own]
            # validity is monotone: once a tile is missing, the rest of the warp's stream is too
            assert valid == sorted(valid, reverse=True)
            for (j, tile0, g), ok in zip(own, valid):
                if ok:
                    u = (tile0 + ti) * G + g
                    assert u not in seen
                    seen.add(u)
    assert len(seen) == tiles * G


def test_kparts_of_the_27b_matrices():
    assert kparts(320, 48) == 3 and kparts(320, 136) == 3     # out / down projections: 40 super-tiles
    assert kparts(1030, 40) == 1 and kparts(896, 40) == 1     # in_proj
    assert kparts(2176, 40, swiglu=True) == 1                 # gate/up
    assert kparts(320, 80) == 3                               # the draft layer's fc
    assert kparts(4, 4) == 1                                  # too few groups to split
