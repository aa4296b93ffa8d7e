"""Two ranks.  Rank 0 runs the fused all-reduce with a 300 ms deadline; rank 1
sleeps on the host for 1.5 s before launching (no kernel or collective of it is
in flight meanwhile).  Rank 0's wait for rank 1's partial tiles runs out: its
kernel returns, the status word says which wait gave up.  After a collective
reset the same call succeeds on both ranks."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import flashoverlap_b200  # noqa: F401
from flashoverlap_b200.parallel import init_distributed, make_overlap_impl


def main():
    rank, world, _ = init_distributed()
    impl = make_overlap_impl(timeout_ms=300 if rank == 0 else 3000, nvls=False)
    M, N, K = 512, 1024, 256
    g = torch.Generator().manual_seed(rank)
    A = torch.randn(M, K, generator=g).cuda().half()
    B = (torch.randn(N, K, generator=g) / K ** 0.5).cuda().half()
    ref = A.float() @ B.float().t()
    dist.all_reduce(ref)
    out = impl.gemm_allreduce_fused(A, B, None, 0.0, 0)  # a healthy call first (also sizes the workspace)
    torch.cuda.synchronize()
    impl.check_status()
    assert (out.float() - ref).abs().max().item() < 0.05
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 1:
        time.sleep(1.5)
    impl.gemm_allreduce_fused(A, B, None, 0.0, 0)
    torch.cuda.synchronize()
    st = impl.status()
    if rank == 0:
        ok = st[0] in (2, 3)
        print(f"rank 0 {'timed out as expected' if ok else 'did NOT time out'}: {impl.status_string()}", flush=True)
        if not ok:
            return 1
    else:
        print(f"rank 1 status after late launch: {impl.status_string()}", flush=True)
    impl.reset()  # collective: drain, zero the counters, clear the status
    impl.set_timeout_ms(10000)
    out = impl.gemm_allreduce_fused(A, B, None, 0.0, 0)
    torch.cuda.synchronize()
    impl.check_status()
    err = (out.float() - ref).abs().max().item()
    print(f"rank {rank} recovered: max err {err:.4f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if err < 0.05 else 1


if __name__ == "__main__":
    sys.exit(main())
