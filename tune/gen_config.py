"""Stage 1 from an external profiler's CSV (reference: tune/gen_config.py:17-137,
which reads ``m{M}n{N}k{K}.gemm.csv`` of the CUTLASS profiler).  Rows are sorted
by runtime, rows with split-K > 1 are rejected, tile shapes are mapped to Algo
indices through AlgoDict and the surviving configurations are re-timed with this
library's kernel.

    python tune/gen_config.py --m 4096 --n 8192 --k 1024 --path /dir/with/csv
"""
import argparse
import os

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES  # noqa: E402

from flashoverlap_b200.tune.runtime import make_inputs, mean_time_ms
from flashoverlap_b200.utils import config as cfg


def rows_from_csv(path, algo_dict, keep: int = 10):
    """Algo indices of the fastest rows of a profiler CSV, fastest first.

    The file needs the columns ``cta_m``, ``cta_n``, ``cta_k`` and ``Runtime``
    (any case); ``split_k_slices``, if present, must be 1 in every row that is
    used (reference: tune/gen_config.py:45-47 asserts the same).  Rows whose tile
    shape this build does not have are skipped."""
    import csv

    with open(path, newline="") as fh:
        reader = csv.DictReader(fh)
        if reader.fieldnames is None:
            raise ValueError(f"{path} is empty")
        cols = {c.strip().lower(): c for c in reader.fieldnames}
        for c in ("cta_m", "cta_n", "cta_k", "runtime"):
            if c not in cols:
                raise ValueError(f"{path} lacks the column {c!r}")
        rows = list(reader)
    rows.sort(key=lambda r: float(r[cols["runtime"]]))
    picked = []
    for r in rows:
        key = (int(float(r[cols["cta_m"]])), int(float(r[cols["cta_n"]])), int(float(r[cols["cta_k"]])))
        if key not in algo_dict:
            continue
        if "split_k_slices" in cols and int(float(r[cols["split_k_slices"]])) != 1:
            raise AssertionError("split-K configurations are not supported")
        if algo_dict[key] not in picked:
            picked.append(algo_dict[key])
        if len(picked) == keep:
            break
    return picked


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--path", default=".", help="directory holding m{M}n{N}k{K}.gemm.csv")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--config-dir", default=None)
    args = ap.parse_args()
    algo_dict = cfg.load_algo_dict(args.config_dir)
    csv = os.path.join(args.path, f"m{args.m}n{args.n}k{args.k}.gemm.csv")
    algos = rows_from_csv(csv, algo_dict)
    if not algos:
        raise SystemExit("no row of the CSV names a tile shape this build has; rebuild with that shape or profile "
                         "with tune/profile_config.py")
    torch.cuda.set_device(0)
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.cutlass_init()
    A, B, C = make_inputs(args.m, args.n, args.k, DTYPES[args.dtype])
    timed = sorted((mean_time_ms(lambda a=a: impl.cutlass_gemm(A, B, C, a), 10, 100), a) for a in algos
                   if args.m % cfg.ALGO_TILES[a][0] == 0 and args.n % cfg.ALGO_TILES[a][1] == 0)
    f = cfg.save_stage1(args.m, args.n, args.k, [cfg.ALGO_TILES[a][0] for _, a in timed],
                        [cfg.ALGO_TILES[a][1] for _, a in timed], [t for t, _ in timed], [a for _, a in timed],
                        args.config_dir)
    print(f"saved {f}")


if __name__ == "__main__":
    main()
