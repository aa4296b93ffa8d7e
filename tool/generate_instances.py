"""Writes ``configs/AlgoDict.pt``, the map from tile shape to Algo index
(reference: tool/generate_instances.py:5-63, which also generates the C++
instantiation lists; here the tile table is part of csrc/kernels/gemm_launch.h
and this tool checks that the Python copy agrees with the built library)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import flashoverlap_b200  # noqa: E402,F401
from flashoverlap_b200.utils import config as cfg  # noqa: E402


def main():
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    n = impl.num_algos()
    native = [tuple(impl.algo_tile(i)) for i in range(n)]
    if native != [tuple(t) for t in cfg.ALGO_TILES]:
        raise SystemExit(f"tile table mismatch: library {native} vs python {cfg.ALGO_TILES}")
    f = cfg.save_algo_dict()
    for tile, idx in cfg.algo_dict().items():
        print(f"Algo {idx}: TileM {tile[0]} TileN {tile[1]} TileK {tile[2]}")
    print(f"saved {f}")


if __name__ == "__main__":
    main()
