"""The tile walk of the int8 tensor-core GEMM (nnops_b200/csrc/gemm_i8_umma.cu: FastDiv, TileWalk),
restated in Python: the multiply-and-shift division equals `//` for every dividend below 2^31, and
the walk visits every (m block, n block) exactly once in the grouped order its comment describes
(m-fastest inside groups of `group_m` m-blocks, a shorter last group).  No GPU.
"""
import random


def fastdiv_init(d: int):
    shift = (d - 1).bit_length() if d > 1 else 0          # 32 - clz(d - 1)
    mul = ((1 << 32) * ((1 << shift) - d)) // d + 1
    assert 0 < mul < (1 << 32)
    return mul, shift


def fastdiv(n: int, mul: int, shift: int) -> int:
    return ((((n * mul) >> 32) + n) & 0xFFFFFFFF) >> shift  # __umulhi(n, mul) + n in 32 bits, then the shift


def test_fastdiv_equals_floor_division():
    rng = random.Random(1)
    divisors = list(range(1, 2050)) + [rng.randrange(1, 1 << 30) for _ in range(2000)] + [(1 << 31) - 1, 1 << 30]
    for d in divisors:
        mul, shift = fastdiv_init(d)
        probes = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, (1 << 31) - 1, (1 << 31) - 2]
        probes += [rng.randrange(0, 1 << 31) for _ in range(40)]
        for n in probes:
            if 0 <= n < (1 << 31):
                assert fastdiv(n, mul, shift) == n // d, (n, d)


def walk(tile: int, num_m: int, num_n: int, group_m: int):
    """TileWalk::operator() with the same intermediate values."""
    group_m = group_m if group_m < num_m else max(num_m, 1)
    group_size = group_m * num_n
    groups = (num_m + group_m - 1) // group_m
    last_gm = max(num_m - (groups - 1) * group_m, 1)
    by_group, by_gm, by_last = fastdiv_init(max(group_size, 1)), fastdiv_init(group_m), fastdiv_init(last_gm)
    group = fastdiv(tile, *by_group)
    first_m = group * group_m
    in_group = tile - group * group_size
    last = num_m - first_m < group_m
    gm = last_gm if last else group_m
    n_blk = fastdiv(in_group, *(by_last if last else by_gm))
    return first_m + in_group - n_blk * gm, n_blk


def reference_walk(tile: int, num_m: int, num_n: int, group_m: int):
    group_size = group_m * num_n
    group = tile // group_size
    first_m = group * group_m
    gm = min(num_m - first_m, group_m)
    in_group = tile - group * group_size
    return first_m + in_group % gm, in_group // gm


def test_walk_covers_every_tile_once_in_grouped_order():
    rng = random.Random(2)
    shapes = [(1, 1, 4), (16, 112, 32), (32, 16, 4), (7, 5, 3), (33, 9, 8), (784, 4, 4), (3, 200, 2), (100, 1, 16)]
    shapes += [(rng.randrange(1, 80), rng.randrange(1, 80), rng.randrange(1, 40)) for _ in range(60)]
    for num_m, num_n, group_m in shapes:
        seen = set()
        for tile in range(num_m * num_n):
            got = walk(tile, num_m, num_n, group_m)
            assert got == reference_walk(tile, num_m, num_n, group_m), (tile, num_m, num_n, group_m)
            assert 0 <= got[0] < num_m and 0 <= got[1] < num_n
            seen.add(got)
        assert len(seen) == num_m * num_n
