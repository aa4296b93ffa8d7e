"""Tile-order and row-order index arrays.

These restate, vectorised, the index conventions of the reference's helpers
(reference: example/utils.py:6-65) so that tuned configs and scripts written
for it keep their meaning:

* ``hint[i]`` is the tile (row-major id ``m * TN + n``) stored in output slot
  ``i``; ``RA[tile] = slot`` is its inverse, completed with the unlisted tiles
  in ascending order.
* the reduce-scatter row map sends row ``r`` of every segment to the block of
  rank ``r % world_size`` inside that segment, keeping the order of rows.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch


def div_up(x: int, y: int) -> int:
    return (x + y - 1) // y


def _default_device(device):
    if device is not None:
        return torch.device(device)
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


def reorder_indices(num_tiles: int, hint: Sequence[int], device=None) -> torch.Tensor:
    """Slot of every tile: ``RA[hint[i]] = i``; tiles not in ``hint`` follow in
    ascending order.  O(num_tiles) (the reference's list search is quadratic,
    reference: example/utils.py:6-22).  Raises on duplicates or out-of-range ids.
    """
    hint_t = torch.as_tensor(list(hint), dtype=torch.long)
    if hint_t.numel() > num_tiles:
        raise ValueError(f"hint has {hint_t.numel()} entries for {num_tiles} tiles")
    if hint_t.numel() and (int(hint_t.min()) < 0 or int(hint_t.max()) >= num_tiles):
        raise ValueError("hint contains a tile id outside [0, num_tiles)")
    listed = torch.zeros(num_tiles, dtype=torch.bool)
    listed[hint_t] = True
    if int(listed.sum()) != hint_t.numel():
        raise ValueError("hint lists a tile more than once")
    order = torch.empty(num_tiles, dtype=torch.long)
    order[hint_t] = torch.arange(hint_t.numel())
    rest = (~listed).nonzero(as_tuple=True)[0]
    order[rest] = torch.arange(hint_t.numel(), num_tiles)
    return order.to(dtype=torch.int32, device=_default_device(device))


def generate_row_mapping(M: int, N: int, BM: int, BN: int, S_list: Iterable[int], world_size: int,
                         device=None) -> torch.Tensor:
    """Row map ``RE`` of the reference's scatter epilogue (reference:
    example/utils.py:24-52): the reordered buffer is viewed as ``M*N/BN`` rows of
    ``BN`` values; inside each segment of ``S * BM`` rows the rows are stably
    sorted by ``row % world_size``; ``RE[old_row] = new_row``.
    """
    S = [int(s) for s in S_list]
    total_tiles = (M * N) // (BM * BN)
    if sum(S) != total_tiles:
        raise ValueError(f"sum(S_list) = {sum(S)} must equal the number of tiles {total_tiles}")
    rows = M * N // BN
    remap = torch.empty(rows, dtype=torch.long)
    start = 0
    for s in S:
        n = s * BM
        ids = torch.arange(start, start + n)
        order = torch.sort(ids % world_size, stable=True).indices
        remap[ids[order]] = torch.arange(start, start + n)
        start += n
    return remap.to(dtype=torch.int32, device=_default_device(device))


def reorder_rows_by_world_size(tensor: torch.Tensor, world_size: int) -> torch.Tensor:
    """Rows grouped by ``row % world_size`` (stable), i.e. the order in which a
    contiguous-block reduce-scatter hands out the reference's interleaved rows
    (reference: example/utils.py:54-65)."""
    rows = torch.arange(tensor.shape[0], device=tensor.device)
    order = torch.argsort(rows % world_size, stable=True)
    return tensor[order]


def to_tile_order(x: torch.Tensor, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1) -> torch.Tensor:
    """Reference layout of a natural-order matrix: tile ``t`` goes to slot
    ``RA[t]``.  Pure PyTorch; the oracle for the kernels' reordered stores."""
    M, N = x.shape
    tm, tn = M // BM, N // BN
    ra = RA.reshape(-1).to(torch.long).cpu()
    tiles = x.reshape(tm, BM, tn, BN).permute(0, 2, 1, 3).reshape(tm * tn, BM, BN)
    slots = torch.empty_like(tiles)
    slots[ra.to(x.device)] = tiles
    # slot s sits at block row s // rldn, block column s % rldn of a matrix of width rldn * BN
    out = slots.reshape(tm * tn // rldn, rldn, BM, BN).permute(0, 2, 1, 3).reshape(-1, rldn * BN)
    return out.reshape(M, N) if rldn * BN == N else out.reshape(-1).reshape(M, N)


def from_tile_order(x: torch.Tensor, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1) -> torch.Tensor:
    """Inverse of :func:`to_tile_order`."""
    M, N = x.shape
    tm, tn = M // BM, N // BN
    ra = RA.reshape(-1).to(torch.long).to(x.device)
    slots = x.reshape(-1).reshape(tm * tn // rldn, BM, rldn, BN).permute(0, 2, 1, 3).reshape(tm * tn, BM, BN)
    tiles = slots[ra]
    return tiles.reshape(tm, tn, BM, BN).permute(0, 2, 1, 3).reshape(M, N)
