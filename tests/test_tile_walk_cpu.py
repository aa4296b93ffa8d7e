"""The tile order of the persistent kernel, computed on the host by the very
function the kernel uses (``torch.ops.flashoverlap_op.tile_walk``): every tile
exactly once for every raster group, taper, rotation and owner cycling; raster
groups complete tile row by tile row; the cost model's group sizes are the
kernel's."""
import itertools

import pytest
import torch

import flashoverlap_b200  # noqa: F401  (loads the native library)
from flashoverlap_b200.tune.model import raster_group_sizes


def walk(TM, TN, G, taper=True, owner_stride=0, ws=1, me=0, rot=0):
    return list(torch.ops.flashoverlap_op.tile_walk(TM, TN, G, taper, owner_stride, ws, me, rot))


@pytest.mark.parametrize("TM,TN", [(1, 1), (1, 7), (5, 3), (16, 32), (32, 5), (33, 2)])
def test_every_tile_exactly_once(TM, TN):
    for G, taper in itertools.product((1, 2, 3, 4, 8, 16, 64), (True, False)):
        for rot in sorted({0, TM // 2, TM - 1}):
            assert sorted(walk(TM, TN, G, taper, rot=rot)) == list(range(TM * TN)), (G, taper, rot)


def test_owner_cycling_visits_every_tile_and_all_owners_early():
    TM, TN, ws = 32, 4, 8
    stride = TM // ws
    for me in range(ws):
        for G in (1, 2, 8):
            w = walk(TM, TN, G, True, stride, ws, me)
            assert sorted(w) == list(range(TM * TN))
            # the first ws tile rows of the walk belong to ws different owners, starting with this rank's
            rows = []
            for t in w:
                if t // TN not in rows:
                    rows.append(t // TN)
            owners = [r // stride for r in rows[:ws]]
            assert sorted(owners) == list(range(ws)) and owners[0] == me


def test_groups_are_column_major_and_match_the_model():
    TM, TN = 16, 6
    for G, taper in itertools.product((1, 2, 4, 8), (True, False)):
        w = walk(TM, TN, G, taper)
        sizes = raster_group_sizes(TM, G, taper)
        assert sum(sizes) == TM
        pos, first_row = 0, 0
        for size in sizes:
            tiles = w[pos:pos + size * TN]
            # exactly the next `size` tile rows, all their columns
            assert sorted(tiles) == [r * TN + c for r in range(first_row, first_row + size) for c in range(TN)]
            # column-major inside the group: the tile rows of a column are consecutive in the walk
            for c in range(TN):
                assert [t // TN for t in tiles[c * size:(c + 1) * size]] == list(range(first_row, first_row + size))
                assert all(t % TN == c for t in tiles[c * size:(c + 1) * size])
            pos += size * TN
            first_row += size
        if taper and TM > 1:
            assert sizes[-1] == 1          # little is left to communicate after the last tile


def test_rotation_starts_at_the_given_tile_row():
    w = walk(8, 3, 2, False, rot=5)
    assert w[0] // 3 == 5 and sorted(w) == list(range(24))


def test_arguments_are_checked():
    with pytest.raises(RuntimeError):
        walk(0, 4, 1)
    with pytest.raises(RuntimeError):
        walk(8, 4, 2, True, 3, 4, 0)      # owner_stride * ws != TM
    with pytest.raises(RuntimeError):
        walk(8, 4, 2, True, 0, 2, 2)      # rank outside the group
