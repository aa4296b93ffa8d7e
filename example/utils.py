"""Index helpers under the reference's module name (reference: example/utils.py),
and, run as a script, a walk through what they compute on a small case:

    python example/utils.py

prints the slot order of a 2 x 4 tile grid for a completion-order hint, moves a
matrix into that tile order and back, and shows the row map of a
reduce-scatter whose wave groups are split over two ranks.  Needs no GPU.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from flashoverlap_b200.utils.reorder import (  # noqa: F401,E402
    div_up,
    from_tile_order,
    generate_row_mapping,
    reorder_indices,
    reorder_rows_by_world_size,
    to_tile_order,
)


def main():
    M, N, BM, BN = 256, 512, 128, 128
    tm, tn = div_up(M, BM), div_up(N, BN)
    hint = [3, 1, 7, 5, 0, 2, 4, 6]                      # tile ids in the order the GEMM completes them
    RA = reorder_indices(tm * tn, hint, device="cpu").reshape(tm, tn)
    print(f"{tm} x {tn} tiles; completion order {hint}\nslot of every tile (RA):\n{RA}")
    x = torch.arange(M * N, dtype=torch.float32).reshape(M, N)
    tiled = to_tile_order(x, BM, BN, RA.reshape(-1))
    back = from_tile_order(tiled, BM, BN, RA.reshape(-1))
    print("tile order and back is the identity:", bool(torch.equal(back, x)))
    print("first element of every slot (tile-ordered buffer):", [int(tiled.reshape(-1)[s * BM * BN]) for s in range(tm * tn)])
    RE = generate_row_mapping(M, N, BM, BN, [4, 4], 2, device="cpu")
    print(f"reduce-scatter row map for wave groups [4, 4] over 2 ranks: {RE.numel()} rows, first 8: {RE[:8].tolist()}")
    rows = reorder_rows_by_world_size(torch.arange(8).reshape(8, 1), 2).reshape(-1).tolist()
    print("rows regrouped by owner (row % 2):", rows)


if __name__ == "__main__":
    main()
