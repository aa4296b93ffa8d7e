"""CPU worker for the gloo tests: world_size ranks, fp32, the plumbing config
(M=256, N=512, K=256 per rank, A ~ N(0,1), B ~ N(0,1)/sqrt(K), seeded by rank;
RMSNorm eps=1e-6, gamma ~ 1 + 0.1 N(0,1))."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from flashoverlap_b200.models import RMSNorm, RowParallelLayer
from flashoverlap_b200.ops import emulate
from flashoverlap_b200.parallel import broadcast_nccl_id, init_distributed, max_over_ranks
from flashoverlap_b200.utils.reorder import from_tile_order, reorder_indices


def main():
    mode = sys.argv[1]
    rank, world, _ = init_distributed(backend="gloo", timeout_s=float(os.environ.get("FO_TEST_TIMEOUT", "60")))
    if mode == "never_joins" and rank == world - 1:
        # a rank that skips the collective: the others must fail with an error, not hang
        return 0
    M, N, K, eps = 256, 512, 256, 1e-6
    g = torch.Generator().manual_seed(rank)
    A = torch.randn(M, K, generator=g)
    B = torch.randn(N, K, generator=g) / K ** 0.5
    gw = torch.Generator().manual_seed(1234)
    gamma = 1 + 0.1 * torch.randn(N, generator=gw)

    if mode == "never_joins":
        try:
            emulate.gemm_allreduce(A, B)
        except Exception as exc:
            print(f"rank {rank}: collective failed as expected: {type(exc).__name__}", flush=True)
            return 0
        print(f"rank {rank}: collective unexpectedly succeeded", flush=True)
        return 1

    # golden: torch semantics
    full = A @ B.t()
    dist.all_reduce(full)
    xf = full
    gold_ar = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma
    ok = True

    def check(name, got, want, tol=1e-4):
        nonlocal ok
        err = (got - want).abs().max().item()
        good = err <= tol * max(1.0, want.abs().max().item())
        ok = ok and good
        print(f"rank {rank} {'PASS' if good else 'FAIL'} {name}: {err:.3g}", flush=True)

    check("emulated fused AR", emulate.gemm_allreduce(A, B), full)
    check("emulated fused AR+RMSNorm", emulate.gemm_allreduce(A, B, gamma, eps), gold_ar)
    rows = M // world
    blk = slice(rank * rows, (rank + 1) * rows)
    check("emulated fused RS (contiguous)", emulate.gemm_reducescatter(A, B), full[blk])
    check("emulated fused RS+RMSNorm (contiguous)", emulate.gemm_reducescatter(A, B, gamma, eps), gold_ar[blk])
    check("emulated fused RS (interleaved)", emulate.gemm_reducescatter(A, B, interleave=True), full[rank::world])
    # reference-compatible layouts
    BM, BN = 128, 256
    tm, tn = M // BM, N // BN
    RA = reorder_indices(tm * tn, [3, 0], device="cpu").reshape(tm, tn)
    C = emulate.gemm_allreduce_overlap(A, B, BM, BN, RA)
    check("compat AR layout", from_tile_order(C, BM, BN, RA), full)
    D = emulate.gemm_reducescatter_overlap(A, B, BM, BN, RA)
    check("compat RS layout", from_tile_order(D, BM // world, BN, RA), full[rank::world])
    # the golden modules themselves (matmul + collective + RMSNorm) on gloo
    layer = RowParallelLayer(K, N, "all_reduce", None, dtype=torch.float32, device="cpu")
    norm = RMSNorm(N, eps=eps, dtype=torch.float32, device="cpu")
    with torch.no_grad():
        layer.weight.copy_(B)
        norm.weight.copy_(gamma)
        check("RowParallelLayer(all_reduce) + RMSNorm", norm(layer(A)), gold_ar)
        layer_rs = RowParallelLayer(K, N, "reduce_scatter", None, dtype=torch.float32, device="cpu")
        layer_rs.weight.copy_(B)
        check("RowParallelLayer(reduce_scatter)", layer_rs(A), full[blk])
    # two-level groups for jobs on several nodes: the ranks cut into pretend nodes
    from flashoverlap_b200.parallel import build_hierarchy

    os.environ["FLASHOVERLAP_FAKE_NODES"] = str(world)  # every rank its own node
    h = build_hierarchy()
    assert (h.nodes, h.local_size, h.node, h.local_rank) == (world, 1, rank, 0) and h.intra is None
    if world > 1:
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, group=h.inter)
        assert float(t) == world * (world + 1) / 2
    os.environ["FLASHOVERLAP_FAKE_NODES"] = "1"  # one node holding every rank
    h = build_hierarchy()
    assert (h.nodes, h.local_size, h.node, h.local_rank) == (1, world, 0, rank) and h.inter is None
    del os.environ["FLASHOVERLAP_FAKE_NODES"]
    # control-plane helpers
    assert max_over_ranks(float(rank)) == float(world - 1)
    ids = broadcast_nccl_id() if world == 1 else None  # NCCL ids need the native library + GPU; world 1 path only
    assert ids is None or len(ids) == 16
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
