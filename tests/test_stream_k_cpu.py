"""The stream-K work partition of the bf16 pair kernel, checked on the host through the iterator the kernel itself runs
(`symplex_b200_stream_k_items`): every k-block of every tile belongs to exactly one CTA pair, a pair leaves at most one
set of partial sums (so one workspace slot per pair is enough) and does that first, a tile that is split has exactly
one owner - the pair with its last k-block - which comes last in that pair's list, and the owner's contributors are
exactly the lower-numbered pairs that hold the tile's other pieces (so an owner only ever waits for pairs placed
before it)."""
import ctypes
import random

import pytest

FULL, PARTIAL, OWNER = 0, 1, 2
GRAIN = 4  # range boundaries are multiples of four k-blocks


def _items(lib, pair, pairs, tiles, nkb):
    cap = tiles + 4
    items = (ctypes.c_int32 * (4 * cap))()
    contrib = (ctypes.c_int32 * cap)()
    n = lib.symplex_b200_stream_k_items(pair, pairs, tiles, nkb, items, cap, contrib)
    assert 0 <= n <= cap
    return [(items[4 * i], items[4 * i + 1], items[4 * i + 2], items[4 * i + 3], contrib[i]) for i in range(n)]


def _check(lib, pairs, tiles, nkb):
    cover = [[0] * nkb for _ in range(tiles)]
    partial_by_tile, owner_of, owner_contrib = {}, {}, {}
    for p in range(pairs):
        its = _items(lib, p, pairs, tiles, nkb)
        assert its, f"pair {p} of {pairs} has no work ({tiles} tiles x {nkb} k-blocks)"
        kinds = [k for *_, k, _c in its]
        assert kinds.count(PARTIAL) <= 1 and kinds.count(OWNER) <= 1
        if PARTIAL in kinds:
            assert kinds[0] == PARTIAL, "the contribution to another pair's tile comes first"
        if OWNER in kinds:
            assert kinds[-1] == OWNER, "the tile that needs other pairs' sums comes last"
        for t, k0, k1, kind, nc in its:
            assert 0 <= t < tiles and 0 <= k0 < k1 <= nkb
            for k in range(k0, k1):
                cover[t][k] += 1
            if kind == FULL:
                assert (k0, k1) == (0, nkb) and nc == 0
            elif kind == PARTIAL:
                assert k1 < nkb and nc == 0
                partial_by_tile.setdefault(t, []).append(p)
            else:
                assert kind == OWNER and k0 > 0 and k1 == nkb and nc >= 1
                owner_of[t] = p
                owner_contrib[t] = nc
    assert all(c == 1 for row in cover for c in row), "every k-block of every tile exactly once"
    assert set(partial_by_tile) == set(owner_of), "a tile has partial sums if and only if it has an owner waiting for them"
    for t, ps in partial_by_tile.items():
        o, nc = owner_of[t], owner_contrib[t]
        assert sorted(ps) == list(range(o - nc, o)), (t, ps, o, nc)


def test_invalid_arguments(lib):
    assert lib.symplex_b200_stream_k_items(0, 0, 1, 1, None, 0, None) == -1
    assert lib.symplex_b200_stream_k_items(5, 4, 1, 1, None, 0, None) == -1
    assert lib.symplex_b200_stream_k_items(0, 4, 0, 8, None, 0, None) == -1


@pytest.mark.parametrize("pairs,tiles,nkb", [(74, 128, 64), (74, 162, 64), (74, 304, 128), (74, 8, 150), (74, 12, 151),
                                              (74, 74, 64), (74, 75, 16), (66, 1, 1056), (2, 3, 8), (74, 1024, 64)])
def test_partition_of_the_shapes_the_gpu_tests_run(lib, pairs, tiles, nkb):
    _check(lib, pairs, tiles, nkb)


def test_partition_of_random_shapes(lib):
    rng = random.Random(7)
    done = 0
    while done < 300:
        pairs = rng.choice([74, 66, 10, 4, 1])
        tiles = rng.randint(1, 300)
        nkb = rng.randint(1, 260)
        if tiles * nkb < pairs * 2 * GRAIN:  # the launcher refuses shorter ranges: a pair could be left without work
            continue
        _check(lib, pairs, tiles, nkb)
        done += 1
