"""Bandwidth curve across nodes (reference: tune/bandwidth_multinode.py).

    torchrun --nnodes=2 --nproc_per_node=8 --rdzv_backend=c10d --rdzv_endpoint=HOST:PORT \
        tune/bandwidth_multinode.py --comm_op all_reduce

Differences from the single-node tool, as in the reference: the rendezvous is
retried (nodes rarely start in the same second; reference :27-39), the file is
named ``bandwidth_{op}_ws{N}.pt`` so that single-node curves are not
overwritten, and the per-rank times of every size are gathered so that a slow
node shows (reference :100-101): rank 0 prints min / mean / max over the ranks
and names the slowest rank.  Ranks on different hosts cannot map one another's
memory, so only the NCCL collectives can be measured across nodes; the
library's own transports are refused with a message.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import bandwidth  # noqa: E402

from flashoverlap_b200.cli import finish, start  # noqa: E402
from flashoverlap_b200.tune.bandwidth import NCCL_OPS  # noqa: E402


def main():
    ap = bandwidth.build_parser()
    ap.add_argument("--rendezvous_retries", type=int, default=5)
    args = ap.parse_args()
    args.multinode = True
    rank, world = start(retries=args.rendezvous_retries)
    nodes = int(os.environ.get("GROUP_WORLD_SIZE", os.environ.get("NNODES", "1")))
    own = [op for op in args.comm_op if op not in NCCL_OPS]
    if own and nodes > 1:
        if rank == 0:
            print(f"{own} need peer-mapped memory: measure them inside one node with tune/bandwidth.py")
        finish()
        return 2
    results = bandwidth.run(args, rank, world, gather_ranks=True)
    for op, (curve, per_rank) in results.items():
        if rank == 0 and per_rank is not None and per_rank.numel() > 0:
            print(f"# {op}: per-size times over the ranks (ms): min mean max slowest-rank")
            for (n, _), row in zip(curve.tolist(), per_rank.tolist()):
                worst = max(range(len(row)), key=lambda i: row[i])
                print(f"{int(n):>12d} {min(row):9.4f} {sum(row) / len(row):9.4f} {max(row):9.4f} {worst:4d}")
    finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
