"""Stage 2 of tuning: tile-order hint, wave grouping and kernel knobs (reference:
tune/search.py; under a multi-node torchrun it replaces tune/search_multinode.py).

    torchrun --nproc_per_node=8 tune/search.py --m_dim 4096 --n_dim 8192 --k_dim 1024 \
        --comm_op all_reduce [--predictive_search]
"""
import argparse
import os

from _common import DTYPES, finish, make_overlap_impl, start

from flashoverlap_b200.tune import search
from flashoverlap_b200.utils import config as cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m_dim", "--m", type=int, default=4096)
    ap.add_argument("--k_dim", "--k", type=int, default=8192)
    ap.add_argument("--n_dim", "--n", type=int, default=8192)
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter"])
    ap.add_argument("--predictive_search", action="store_true")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--multinode", action="store_true")
    ap.add_argument("--path", default=None)
    args = ap.parse_args()
    rank, world = start()
    impl = make_overlap_impl()
    M, N, K = args.m_dim, args.n_dim, args.k_dim
    if args.predictive_search or M * N > search.PREDICTIVE_THRESHOLD:
        multinode = args.multinode or int(os.environ.get("GROUP_WORLD_SIZE", "1")) > 1
        curve = cfg.load_bandwidth(args.comm_op, world, multinode, args.path)
        p2p = None
        try:
            p2p = float(cfg.load_bandwidth("p2p_push", world, multinode, args.path)[:, 1].max())
        except FileNotFoundError:
            pass
        if rank == 0:
            print("Bandwidth curve captured.\nStart predictive searching.")
        search.predictive_search(impl, M, N, K, args.comm_op, curve, p2p, DTYPES[args.dtype], args.path)
    else:
        if rank == 0:
            print("Start exhaustive searching.")
        search.exhaustive_search(impl, M, N, K, args.comm_op, DTYPES[args.dtype], args.path)
    finish()


if __name__ == "__main__":
    main()
