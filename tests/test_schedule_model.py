"""The closed-form task assignment of the kernel's scheduler, restated in Python and checked for its invariants.

`build_schedule` (csrc/mm_kernel.cuh) gives SM g of G, per phase with NT = M * n weight tiles of k units each:
the whole tiles r + g, r + g + G, ... (r = NT mod G) and at most one partial task: remainder tile t = floor(g r / G),
shared by the SMs [ceil(t G / r), ceil((t + 1) G / r)), each with one contiguous range of the tile's k units.
The properties below are what the epilogue's reduction relies on: every unit of every tile is covered exactly once,
the contributors of a split tile are consecutive SMs starting at the recorded first one, and the recorded part count
is the number of SMs with a non-empty range.
"""
import itertools

import pytest


def sm_tasks(g, G, M, n, k):
    """Tasks of SM g in one phase: list of (tile, first unit, end unit, parts, first contributing SM)."""
    NT = M * n
    r = NT % G
    tasks = []
    if r > 0:
        t = (g * r) // G
        gs, ge = (t * G + r - 1) // r, ((t + 1) * G + r - 1) // r
        S, li = ge - gs, g - gs
        assert 0 <= li < S
        base, extra = k // S, k % S
        ub = li * base + min(li, extra)
        ue = ub + base + (1 if li < extra else 0)
        if ue > ub:
            tasks.append((t, ub, ue, min(S, k), gs))
    t = r + g
    while t < NT:
        tasks.append((t, 0, k, 1, 0))
        t += G
    return tasks


@pytest.mark.parametrize('G', [1, 8, 132, 148])
@pytest.mark.parametrize('n,k', [(20, 12), (24, 5), (1, 1), (64, 16), (7, 3)])
def test_every_unit_of_every_tile_is_covered_exactly_once(G, n, k):
    for M in list(range(0, 12)) + [16, 31, 100, 320]:
        NT = M * n
        cover = {}
        parts = {}
        for g in range(G):
            tasks = sm_tasks(g, G, M, n, k)
            assert sum(1 for t in tasks if t[3] > 1 or (t[1], t[2]) != (0, k)) <= 1      # one partial task at most
            for (t, ub, ue, np_, first) in tasks:
                assert 0 <= t < NT and 0 <= ub < ue <= k
                for u in range(ub, ue):
                    assert (t, u) not in cover
                    cover[(t, u)] = g
                parts.setdefault(t, []).append((g, np_, first))
        assert len(cover) == NT * k
        for t, plist in parts.items():
            sms = sorted(g for g, _, _ in plist)
            np_, first = plist[0][1], plist[0][2]
            assert all(p[1] == np_ for p in plist)
            assert len(sms) == np_
            if np_ > 1:
                assert all(p[2] == first for p in plist)
                assert sms == list(range(first, first + np_))                             # consecutive contributors


def test_unit_load_is_balanced():
    """Whole tiles are dealt evenly (NT - r is a multiple of G); a partial share is at most ceil(k / floor(G / r))."""
    G, n, k = 148, 20, 12
    for M in (1, 8, 13, 64):
        r = (M * n) % G
        loads = [sum(ue - ub for (_, ub, ue, _, _) in sm_tasks(g, G, M, n, k)) for g in range(G)]
        bound = 0 if r == 0 else -(-k // (G // r))
        assert max(loads) - min(loads) <= bound


def test_small_division_helper_model():
    """`udiv_small`: one approximate float division and a +-1 correction is exact for dividends below 2^24 and
    quotients below 2^21 (the kernel's uses: tile, unit, SM, token and chunk indices, all far below that)."""
    import numpy as np
    rng = np.random.default_rng(0)
    a = rng.integers(0, 1 << 24, size=200000, dtype=np.int64)
    b = rng.integers(8, 1 << 16, size=200000, dtype=np.int64)             # quotients < 2^21
    for err in (-2e-7, 0.0, 2e-7):                                                       # a relative error of ~2 ulp
        q = np.floor((a.astype(np.float32) / b.astype(np.float32)).astype(np.float64) * (1.0 + err)).astype(np.int64)
        rem = a - q * b
        q = np.where(rem < 0, q - 1, np.where(rem >= b, q + 1, q))
        assert np.array_equal(q, a // b)
