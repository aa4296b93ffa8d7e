"""Bandwidth curve of a collective or of one of the library's own transports on
the GPUs of this job (reference: tune/bandwidth.py:56-158).

    torchrun --nproc_per_node=8 tune/bandwidth.py --comm_op all_reduce
    torchrun --nproc_per_node=8 tune/bandwidth.py --comm_op p2p_push
    torchrun --nproc_per_node=8 tune/bandwidth.py --comm_op multimem_allreduce --table profiles/x.txt

Writes ``configs/bandwidth_{op}_tp{N}.pt`` (``[elements, GB/s]``), a PNG when
matplotlib is present, and with ``--table`` the same curve as text.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flashoverlap_b200.cli import DTYPES, finish, make_overlap_impl, start  # noqa: E402
from flashoverlap_b200.tune.bandwidth import COMM_OPS, NCCL_OPS, curve_table, measure_curve, plot_curve  # noqa: E402
from flashoverlap_b200.utils import config as cfg  # noqa: E402


def build_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm_op", default="all_reduce", choices=list(COMM_OPS))
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--points", type=int, default=36)
    ap.add_argument("--max_elements", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--reps", type=int, default=200)
    ap.add_argument("--chunk_bytes", type=int, default=8192, help="p2p_push_bulk: bytes per bulk copy")
    ap.add_argument("--ctas", type=int, default=0, help="own transports: CTAs to launch (0 = all SMs)")
    ap.add_argument("--multinode", action="store_true", help="name the file ..._ws{N}.pt")
    ap.add_argument("--path", default=None)
    ap.add_argument("--table", default=None, help="also write the curve as a text table to this file")
    return ap


def run(args, rank, world, gather_ranks=False):
    multinode = args.multinode or int(os.environ.get("GROUP_WORLD_SIZE", "1")) > 1
    own = args.comm_op not in NCCL_OPS
    max_el = args.max_elements
    if own and max_el is None:
        max_el = 64 << 20  # the symmetric workspace holds 128 MiB per buffer
    need = (max_el or 2 ** 29) if own else 8192 * 8192
    impl = make_overlap_impl(nvls=True if args.comm_op.startswith("multimem") else None, max_m=8192,
                             max_n=max(8192, need // 8192))
    if args.comm_op.startswith("multimem") and not impl.nvls_available():
        if rank == 0:
            print("no multicast mapping on this machine: the multimem curves cannot be measured")
        return None, None
    res = measure_curve(impl, args.comm_op, DTYPES[args.dtype], args.points, args.warmup, args.reps, max_el,
                        args.chunk_bytes, args.ctas, gather_ranks=gather_ranks)
    curve, per_rank = (res if gather_ranks else (res, None))
    impl.check_status()
    if rank == 0:
        f = cfg.save_bandwidth(curve, args.comm_op, world, multinode, args.path)
        png = str(f)[:-3] + ".png"
        plotted = plot_curve(curve, f"{args.comm_op} x{world}", png)
        text = curve_table(curve, args.comm_op, world)
        print(text, end="")
        if args.table:
            with open(args.table, "w") as fh:
                fh.write(text)
        print(f"saved {f}" + (f" and {png}" if plotted else ""))
    return curve, per_rank


def main():
    args = build_parser().parse_args()
    rank, world = start()
    run(args, rank, world)
    finish()


if __name__ == "__main__":
    main()
