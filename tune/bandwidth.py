"""Bandwidth curve of a collective on the GPUs of this job (reference:
tune/bandwidth.py; with torchrun across nodes it plays the role of
tune/bandwidth_multinode.py and writes the ``_ws{N}`` file).

    torchrun --nproc_per_node=8 tune/bandwidth.py --comm_op all_reduce
    torchrun --nproc_per_node=8 tune/bandwidth.py --comm_op p2p_push
"""
import argparse
import os

from _common import DTYPES, finish, make_overlap_impl, start

from flashoverlap_b200.tune.bandwidth import measure_curve, plot_curve
from flashoverlap_b200.utils import config as cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter", "p2p_push"])
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--points", type=int, default=36)
    ap.add_argument("--max_elements", type=int, default=None)
    ap.add_argument("--multinode", action="store_true", help="name the file ..._ws{N}.pt")
    ap.add_argument("--path", default=None)
    args = ap.parse_args()
    rank, world = start()
    multinode = args.multinode or int(os.environ.get("GROUP_WORLD_SIZE", "1")) > 1
    impl = make_overlap_impl()
    max_el = args.max_elements
    if args.comm_op == "p2p_push" and max_el is None:
        max_el = 64 << 20
    curve = measure_curve(impl, args.comm_op, DTYPES[args.dtype], args.points, max_elements=max_el)
    impl.check_status()
    if rank == 0:
        f = cfg.save_bandwidth(curve, args.comm_op, world, multinode, args.path)
        png = str(f)[:-3] + ".png"
        plotted = plot_curve(curve, f"{args.comm_op} x{world}", png)
        for n, bw in curve.tolist():
            print(f"{int(n):>12d} elements  {bw:8.1f} GB/s")
        print(f"saved {f}" + (f" and {png}" if plotted else ""))
    finish()


if __name__ == "__main__":
    main()
