"""Stage 2 of tuning: tile-order hint, wave grouping and kernel knobs (reference:
tune/search.py:599-618).

    torchrun --nproc_per_node=8 tune/search.py --m_dim 4096 --n_dim 8192 --k_dim 1024 \
        --comm_op all_reduce [--predictive_search]

Exhaustive: every fused candidate and every composition of the wave count is
timed.  Predictive (flag, or M*N above the reference's threshold): candidates
are ranked on the measured bandwidth curves of ``tune/bandwidth.py`` (the NCCL
curve of the collective for the wave grouping, the curve of the library's own
transport for the fused kernel) and only the best are timed.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flashoverlap_b200.cli import DTYPES, finish, make_overlap_impl, start  # noqa: E402
from flashoverlap_b200.tune import search  # noqa: E402
from flashoverlap_b200.utils import config as cfg  # noqa: E402


def build_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m_dim", "--m", type=int, default=4096)
    ap.add_argument("--k_dim", "--k", type=int, default=8192)
    ap.add_argument("--n_dim", "--n", type=int, default=8192)
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter"])
    ap.add_argument("--predictive_search", action="store_true")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--multinode", action="store_true")
    ap.add_argument("--path", default=None)
    return ap


def run(args, rank, world):
    impl = make_overlap_impl()
    M, N, K = args.m_dim, args.n_dim, args.k_dim
    multinode = args.multinode or int(os.environ.get("GROUP_WORLD_SIZE", "1")) > 1
    if args.predictive_search or M * N > search.PREDICTIVE_THRESHOLD:
        curve = cfg.load_bandwidth(args.comm_op, world, multinode, args.path)
        nvls = args.comm_op == "all_reduce" and world > 1 and impl.allreduce_uses_nvls()
        link, kind = search.link_bandwidth_from_curves(world, multinode, args.path, nvls=nvls)
        if link is None and world > 1 and impl.transport() == "p2p":
            raise SystemExit("no curve of the library's own transport found: run tune/bandwidth.py --comm_op p2p_push "
                             "(and multimem_allreduce where NVLink SHARP is available) first")
        if rank == 0:
            print(f"Bandwidth curve captured ({kind or 'NCCL only'}: {link} GB/s).\nStart predictive searching.")
        return search.predictive_search(impl, M, N, K, args.comm_op, curve, link, DTYPES[args.dtype], args.path,
                                        link_kind="nvls" if kind.startswith("multimem") else "p2p")
    if rank == 0:
        print("Start exhaustive searching.")
    return search.exhaustive_search(impl, M, N, K, args.comm_op, DTYPES[args.dtype], args.path)


def main():
    args = build_parser().parse_args()
    rank, world = start()
    run(args, rank, world)
    finish()


if __name__ == "__main__":
    main()
