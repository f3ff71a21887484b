"""Host-side check of the streaming qmm's work partition (no GPU needed).

Re-plays, in Python, the control flow every thread block of the kernel follows (which slab, which
span of units, where each row-tile segment ends, which workspace slot a partial tile goes to, how many
partial tiles each row tile expects) on the partition the C library computes, and asserts that every
(unit) is processed exactly once, slots never collide and ticket counts agree."""
import ctypes

import pytest

from dflash_mlx_b200 import _lib


def _plan(M, K, N, G):
    out = (ctypes.c_int * 400)()
    n = _lib.lib().dflash_verify_qmm_plan(M, K, N, G, out, 400)
    assert n > 0, _lib.lib().dflash_last_error_string()
    v = list(out[:n])
    NT, S, maxp, grid = v[:4]
    return NT, S, maxp, grid, v[4:4 + S + 1], v[4 + S + 1:4 + 2 * (S + 1)]


def _cta_of(u, units, ctas):
    return ((u + 1) * ctas - 1) // units


def _simulate(M, K, N, G):
    NT, S, maxp, grid, chunk0, cta0 = _plan(M, K, N, G)
    C = K // (8 * G)
    assert chunk0[0] == 0 and chunk0[-1] == C and cta0[0] == 0 and cta0[-1] == grid
    geom = []
    for s in range(S):
        cs = chunk0[s + 1] - chunk0[s]
        assert 1 <= cs <= 2048 // (8 * G)
        units = NT * cs
        ctas = min(cta0[s + 1] - cta0[s], units)
        assert ctas >= 1
        geom.append((cs, units, ctas))

    def pieces(s, nt):
        cs, units, ctas = geom[s]
        a = _cta_of(nt * cs, units, ctas)
        b = _cta_of((nt + 1) * cs - 1, units, ctas)
        return a, b - a + 1

    covered = set()
    slots = set()
    arrivals = [0] * NT
    direct = [0] * NT
    for b in range(grid):
        s = 0
        while s + 1 < S and b >= cta0[s + 1]:
            s += 1
        cs, units, ctas = geom[s]
        bl = b - cta0[s]
        if bl >= ctas:
            continue
        u0, u1 = bl * units // ctas, (bl + 1) * units // ctas
        assert u1 > u0
        nt, kc = divmod(u0, cs)
        for u in range(u0, u1):
            key = (s, nt, kc)
            assert key not in covered
            covered.add(key)
            if kc == cs - 1 or u == u1 - 1:
                total = sum(pieces(s2, nt)[1] for s2 in range(S))
                first, _ = pieces(s, nt)
                if total > 1:
                    pidx = bl - first
                    assert 0 <= pidx < maxp, (pidx, maxp)
                    slot = (s, pidx, nt)
                    assert slot not in slots
                    slots.add(slot)
                    arrivals[nt] += 1
                else:
                    direct[nt] += 1
            kc += 1
            if kc == cs:
                kc = 0
                nt += 1
    assert len(covered) == NT * C
    for nt in range(NT):
        total = sum(pieces(s2, nt)[1] for s2 in range(S))
        if total > 1:
            assert arrivals[nt] == total and direct[nt] == 0
            # the reducer enumerates slots (s2, p) for p < pieces(s2, nt): all must have been written
            for s2 in range(S):
                for p in range(pieces(s2, nt)[1]):
                    assert (s2, p, nt) in slots
        else:
            assert direct[nt] == 1 and arrivals[nt] == 0
    return NT, S, maxp, grid


SHAPES = [(16, 4096, 12288, 64), (16, 5120, 17408, 64), (16, 17408, 5120, 64), (16, 5120, 1024, 64),
          (16, 6144, 5120, 64), (16, 512, 2048, 64), (16, 2048, 512, 64), (16, 512, 64, 64), (3, 1024, 40, 64),
          (16, 1024, 8192, 32), (16, 256, 96, 32), (16, 4096, 4096, 128), (16, 1024, 64, 128), (16, 5120, 151936, 64)]


@pytest.mark.parametrize("M,K,N,G", SHAPES)
@pytest.mark.parametrize("max_blocks", [0, 1, 2, 3, 7, 40, 148, 296])
def test_partition_is_exact(M, K, N, G, max_blocks):
    lib = _lib.lib()
    lib.dflash_verify_qmm_set_max_blocks(max_blocks)
    try:
        NT, S, maxp, grid = _simulate(M, K, N, G)
        need = lib.dflash_verify_qmm_workspace_bytes(M, K, N, G)
        assert need >= S * maxp * NT * 4096
    finally:
        lib.dflash_verify_qmm_set_max_blocks(0)
