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
    ap.add_argument("--comm_op", default=["all_reduce"], choices=list(COMM_OPS), nargs="+",
                    help="one or more curves to measure in this run")
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
    """Measures every curve named in args.comm_op with one implementation object;
    returns {comm_op: (curve, per-rank times or None)}."""
    multinode = args.multinode or int(os.environ.get("GROUP_WORLD_SIZE", "1")) > 1
    ops = list(args.comm_op) if isinstance(args.comm_op, (list, tuple)) else [args.comm_op]
    any_own = any(op not in NCCL_OPS for op in ops)
    any_mm = any(op.startswith("multimem") for op in ops)
    max_own = args.max_elements if args.max_elements is not None else 64 << 20  # the workspace holds 128 MiB per buffer
    impl = make_overlap_impl(nvls=True if any_mm else None, max_m=8192, max_n=max(8192, max_own // 8192 if any_own else 0))
    out = {}
    tables = []
    for op in ops:
        if op.startswith("multimem") and not impl.nvls_available():
            if rank == 0:
                print(f"{op}: no multicast mapping on this machine, cannot be measured")
            continue
        max_el = args.max_elements if op in NCCL_OPS else max_own
        res = measure_curve(impl, op, DTYPES[args.dtype], args.points, args.warmup, args.reps, max_el,
                            args.chunk_bytes, args.ctas, gather_ranks=gather_ranks)
        curve, per_rank = (res if gather_ranks else (res, None))
        impl.check_status()
        out[op] = (curve, per_rank)
        if rank == 0:
            f = cfg.save_bandwidth(curve, op, world, multinode, args.path)
            png = str(f)[:-3] + ".png"
            plotted = plot_curve(curve, f"{op} x{world}", png)
            text = curve_table(curve, op, world)
            tables.append(text)
            print(text, end="")
            print(f"saved {f}" + (f" and {png}" if plotted else ""))
    if rank == 0 and args.table and tables:
        with open(args.table, "w") as fh:
            fh.write("\n".join(tables))
    return out


def main():
    args = build_parser().parse_args()
    rank, world = start()
    run(args, rank, world)
    finish()


if __name__ == "__main__":
    main()
