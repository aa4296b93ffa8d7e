"""Index helpers against brute-force restatements of their definitions."""
import pytest
import torch

from flashoverlap_b200.utils.reorder import (
    from_tile_order,
    generate_row_mapping,
    reorder_indices,
    reorder_rows_by_world_size,
    to_tile_order,
)


def brute_reorder(S, hint):
    new = [-1] * S
    for i, e in enumerate(hint):
        new[e] = i
    rest = [x for x in range(S) if x not in hint]
    for i, e in enumerate(rest, start=len(hint)):
        new[e] = i
    return new


@pytest.mark.parametrize("S,hint", [(8, []), (8, [3, 1]), (16, list(reversed(range(16)))), (5, [4, 0, 2])])
def test_reorder_indices_matches_definition(S, hint):
    assert reorder_indices(S, hint, device="cpu").tolist() == brute_reorder(S, hint)


def test_reorder_indices_rejects_bad_hints():
    with pytest.raises(ValueError):
        reorder_indices(4, [0, 0], device="cpu")
    with pytest.raises(ValueError):
        reorder_indices(4, [4], device="cpu")
    with pytest.raises(ValueError):
        reorder_indices(2, [0, 1, 1], device="cpu")


def test_row_mapping_groups_rows_by_rank_inside_each_segment():
    M, N, BM, BN, ws = 8, 8, 4, 4, 2
    segs = [1, 3]
    re = generate_row_mapping(M, N, BM, BN, segs, ws, device="cpu").tolist()
    rows = M * N // BN
    assert sorted(re) == list(range(rows))
    start = 0
    for s in segs:
        n = s * BM
        ids = list(range(start, start + n))
        expect = sorted(ids, key=lambda r: r % ws)  # python's sort is stable
        for new_pos, old in enumerate(expect):
            assert re[old] == start + new_pos
        start += n
    with pytest.raises(ValueError):
        generate_row_mapping(M, N, BM, BN, [1, 1], ws, device="cpu")


def test_reorder_rows_by_world_size():
    x = torch.arange(12).reshape(6, 2)
    y = reorder_rows_by_world_size(x, 3)
    assert y[:, 0].tolist() == [0, 6, 2, 8, 4, 10]


@pytest.mark.parametrize("rldn", [1, 2, 4])
def test_tile_order_roundtrip_and_definition(rldn):
    M, N, BM, BN = 8, 16, 2, 4
    tm, tn = M // BM, N // BN
    x = torch.arange(M * N, dtype=torch.float32).reshape(M, N)
    RA = reorder_indices(tm * tn, [5, 2, 7], device="cpu").reshape(tm, tn)
    y = to_tile_order(x, BM, BN, RA, rldn)
    assert torch.equal(from_tile_order(y, BM, BN, RA, rldn), x)
    flat = y.reshape(-1)
    w = rldn * BN
    for r in range(M):
        for c in range(N):
            s = int(RA[r // BM, c // BN])
            off = ((s // rldn) * BM + r % BM) * w + (s % rldn) * BN + c % BN
            assert flat[off] == x[r, c]
