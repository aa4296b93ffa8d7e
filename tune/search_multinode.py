"""Stage 2 of tuning across nodes (reference: tune/search_multinode.py).

    torchrun --nnodes=2 --nproc_per_node=8 --rdzv_backend=c10d --rdzv_endpoint=HOST:PORT \
        tune/search_multinode.py --m_dim 4096 --n_dim 8192 --k_dim 512 --comm_op all_reduce

What differs from tune/search.py, as in the reference: the rendezvous is
retried; the bandwidth curve is the ``_ws{N}`` file of
tune/bandwidth_multinode.py; and the tile-order hint uses the stricter
sampling rule of the reference's multi-node search: 10 samples, and a tile
counts for a wave only if it finished in that wave in at least 9 of them
(reference: tune/search_multinode.py:165-182).  Ranks on different hosts run
on the NCCL transport (two-stream overlap), so the wave grouping found here is
what decides the speed.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import search as single  # noqa: E402

from flashoverlap_b200.cli import finish, start  # noqa: E402
from flashoverlap_b200.tune import search  # noqa: E402


def main():
    ap = single.build_parser()
    ap.add_argument("--rendezvous_retries", type=int, default=5)
    args = ap.parse_args()
    args.multinode = True
    rank, world = start(retries=args.rendezvous_retries)
    search.HINT_RULE.update(samples=10, min_agree=9)
    sol = single.run(args, rank, world)
    if rank == 0:
        print(f"world {world}: Algo {sol['Algo']}, cSeg {sol['cSeg']}, two-stream {sol.get('two_stream_dur')} ms")
    finish()


if __name__ == "__main__":
    main()
