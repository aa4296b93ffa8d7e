"""Stage 1 of tuning: time every GEMM tile configuration on one GPU and keep the
ten fastest (reference: tune/profile_config.py).

    python tune/profile_config.py --m 4096 --n 8192 --k 1024 [--dtype float16]
"""
import argparse

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES  # noqa: E402

from flashoverlap_b200.tune.runtime import RASTER_CHOICES, profile_gemm
from flashoverlap_b200.utils import config as cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--path", default=None, help="config directory (default: configs/)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    cfg.save_algo_dict(args.path)
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.cutlass_init()
    BM, BN, dur, algo, by_raster = profile_gemm(impl, args.m, args.n, args.k, DTYPES[args.dtype],
                                                rasters=RASTER_CHOICES, with_raster_table=True)
    impl.check_status()
    f = cfg.save_stage1(args.m, args.n, args.k, BM, BN, dur, algo, args.path, dur_raster=by_raster)
    for row in zip(algo, BM, BN, dur):
        print("Algo %d  %dx%d  %.4f ms" % row)
    print(f"saved {f}")


if __name__ == "__main__":
    main()
