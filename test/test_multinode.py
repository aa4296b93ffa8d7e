"""Speed test across nodes (reference: test/test_multinode.py).

    torchrun --nnodes=2 --nproc_per_node=8 --rdzv_backend=c10d --rdzv_endpoint=HOST:PORT \
        test/test_multinode.py --m_dim 4096 --n_dim 8192 --k_dim 512 --comm_op all_reduce

Same table as test/test.py.  What differs, as in the reference: the rendezvous
comes from the environment and is retried, the tuned config and the bandwidth
curves are looked up in a directory every node can read (``--path``; default
``configs/``, which must then be shared), and before measuring every node
reports its host name and ranks so that a mis-wired launch shows.  Ranks on
different hosts run on the NCCL transport: "overlap dur" is then the two-stream
design with the tuned wave grouping.
"""
import os
import socket
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import test as speed_test  # noqa: E402  (test/test.py)


def main():
    import torch.distributed as dist

    from flashoverlap_b200.cli import start

    retries = int(os.environ.get("FLASHOVERLAP_RENDEZVOUS_RETRIES", "5"))
    rank, world = start(retries=retries)
    hosts = [None] * world
    dist.all_gather_object(hosts, (socket.gethostname(), rank, int(os.environ.get("LOCAL_RANK", "0"))))
    if rank == 0:
        by_host = {}
        for h, r, lr in hosts:
            by_host.setdefault(h, []).append(r)
        for h, ranks in sorted(by_host.items()):
            print(f"node {h}: ranks {sorted(ranks)}")
        if len(by_host) > 1:
            print("ranks on several hosts: the NCCL transport is used (two-stream overlap)")
    speed_test.main(rendezvous_retries=retries)  # the process group exists already; start() is a no-op there


if __name__ == "__main__":
    main()
