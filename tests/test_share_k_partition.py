"""The arithmetic with which the few-row int8 engine shares K among the SMs
(nnops_b200/csrc/gemm_i8_skinny.cu: range_begin, cta_of_unit, SegmentList and the slot rule),
restated in Python and checked exhaustively on small cases: every K block of every tile is
worked exactly once, the parts of a tile are exactly the CTAs the finisher will look for, and no
two parts that are alive together share a slot."""
import itertools

import pytest


def range_begin(c, grid, tiles, num_kb):
    return c * (tiles * num_kb) // grid


def cta_of_unit(u, grid, total):
    return ((u + 1) * grid - 1) // total


def segments(u_begin, u_end, num_kb):
    """Pieces of a CTA's range in working order: head part, tail part, whole tiles."""
    first_full = (u_begin + num_kb - 1) // num_kb * num_kb
    last_full_end = u_end // num_kb * num_kb
    out = []
    head_end = min(first_full, u_end)
    if head_end > u_begin:
        t = u_begin // num_kb
        out.append((t, u_begin - t * num_kb, u_begin - t * num_kb + head_end - u_begin))
    if last_full_end >= first_full and last_full_end < u_end:
        out.append((last_full_end // num_kb, 0, u_end - last_full_end))
    if last_full_end > first_full:
        out += [(t, 0, num_kb) for t in range(first_full // num_kb, last_full_end // num_kb)]
    return out


@pytest.mark.parametrize("tiles,num_kb,grid", [(t, k, g) for t, k, g in itertools.product(
    (1, 2, 3, 7, 10, 32, 86), (1, 2, 5, 8, 32, 33), (1, 2, 3, 8, 37, 148)) if t * k >= g])
def test_every_unit_once_and_parts_consistent(tiles, num_kb, grid):
    total = tiles * num_kb
    covered = [0] * total
    parts = {}      # tile -> list of (cta, kb0, kb1)
    for c in range(grid):
        u0, u1 = range_begin(c, grid, tiles, num_kb), range_begin(c + 1, grid, tiles, num_kb)
        segs = segments(u0, u1, num_kb)
        assert sum(kb1 - kb0 for _, kb0, kb1 in segs) == u1 - u0
        slots = set()
        for tile, kb0, kb1 in segs:
            assert 0 <= kb0 < kb1 <= num_kb
            for kb in range(kb0, kb1):
                covered[tile * num_kb + kb] += 1
            if kb0 != 0 or kb1 != num_kb:
                slot = 2 * c + (1 if kb0 == 0 else 0)
                assert slot not in slots          # a CTA's two parts use different slots
                slots.add(slot)
                parts.setdefault(tile, []).append((c, kb0, kb1))
        # parts come first, whole tiles last
        kinds = [(kb0 != 0 or kb1 != num_kb) for _, kb0, kb1 in segs]
        assert kinds == sorted(kinds, reverse=True)
    assert covered == [1] * total
    for tile, plist in parts.items():
        first = cta_of_unit(tile * num_kb, grid, total)
        last = cta_of_unit((tile + 1) * num_kb - 1, grid, total)
        assert [c for c, _, _ in plist] == list(range(first, last + 1))      # whom the finisher looks for
        assert len(plist) >= 2                                                # a lone part would be a whole tile
        for c, kb0, _ in plist:
            # the slot the finisher reads for CTA c is the slot CTA c wrote
            assert (1 if c == first else 0) == (1 if kb0 == 0 else 0)
        assert sum(kb1 - kb0 for _, kb0, kb1 in plist) == num_kb
