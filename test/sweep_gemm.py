"""GEMM sweep (reference: test/sweep_gemm.py:24-141): this library's GEMM (best
tile configuration per shape) against the vendor GEMM over an M x N x K grid.

    python test/sweep_gemm.py --m 1024 4096 8192 --n 4096 8192 --k 1024 4096 [--dtype bfloat16]
"""
import argparse
import json

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES  # noqa: E402

from flashoverlap_b200.tune.runtime import make_inputs, mean_time_ms, usable_algos
from flashoverlap_b200.utils import config as cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--n", type=int, nargs="+", default=[4096, 8192])
    ap.add_argument("--k", type=int, nargs="+", default=[1024, 4096, 8192])
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--rasters", type=int, nargs="+", default=[0],
                    help="raster groups (tile rows walked together) to try per tile; 0 = the library's default")
    ap.add_argument("--jsonl", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.cutlass_init()
    base = torch.classes.flashoverlap_class.BaselineImpl()
    base.cublas_init()
    print(f"{'M':>6} {'N':>6} {'K':>6} | {'vendor ms':>10} {'own ms':>10} {'ratio':>6} {'TFLOP/s':>8}  best tile")
    for M in args.m:
        for N in args.n:
            for K in args.k:
                A, B, C = make_inputs(M, N, K, DTYPES[args.dtype])
                t_vendor = mean_time_ms(lambda: base.cublas_gemm(A, B, C), 10, args.reps)
                timed = []
                for rg in args.rasters:
                    impl.set_raster_group(rg)
                    timed += [(mean_time_ms(lambda a=a: impl.cutlass_gemm(A, B, C, a), 10, args.reps), a, rg)
                              for a in usable_algos(M, N)]
                impl.set_raster_group(0)
                best = min(timed)
                tf = 2.0 * M * N * K / (best[0] * 1e-3) / 1e12
                tile = cfg.ALGO_TILES[best[1]]
                print(f"{M:>6} {N:>6} {K:>6} | {t_vendor:>10.4f} {best[0]:>10.4f} {best[0] / t_vendor:>6.2f} {tf:>8.0f}"
                      f"  {tile[0]}x{tile[1]}x{tile[2]}" + (f" raster {best[2]}" if best[2] else ""))
                if args.jsonl:
                    with open(args.jsonl, "a") as fh:
                        fh.write(json.dumps({"M": M, "N": N, "K": K, "dtype": args.dtype, "vendor_ms": t_vendor,
                                             "own_ms": best[0], "algo": best[1], "raster_group": best[2],
                                             "tflops": tf}) + "\n")
    impl.check_status()


if __name__ == "__main__":
    main()
