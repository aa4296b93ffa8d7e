"""GEMM + AllReduce + RMSNorm: the overlapped layer followed by the reorder-aware
RMSNorm against matmul + dist.all_reduce + a PyTorch RMSNorm (reference:
example/correctness_ar.py:99-127; tolerance 1e-2), plus the natively fused layer.

    torchrun --nproc_per_node=2 example/correctness_ar.py --m_dim 4096 --n_dim 8192 --k_dim 4096
(under torchrun spell the options --m_dim/--n_dim/--k_dim: torchrun itself claims the prefix --m)
"""
import argparse

import torch.distributed as dist
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import finish, make_overlap_impl, start  # noqa: E402

from flashoverlap_b200.models import FusedRowParallelLinear, OverlapRowParallelLayer, ReorderRMSNorm, RMSNorm, \
    RowParallelLayer
from flashoverlap_b200.parallel import broadcast_nccl_id
from flashoverlap_b200.utils import config as cfg


def default_config(M, N):
    algo = 3 if M % 256 == 0 and N % 256 == 0 else 1
    BM, BN, _ = cfg.ALGO_TILES[algo]
    tiles = (M // BM) * (N // BN)
    return {"BM": BM, "BN": BN, "Algo": algo, "hint": list(range(tiles)),
            "cSeg": [tiles // 2, tiles - tiles // 2] if tiles > 1 else [1]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", "--m_dim", dest="m", type=int, default=4096)
    ap.add_argument("--n", "--n_dim", dest="n", type=int, default=8192)
    ap.add_argument("--k", "--k_dim", dest="k", type=int, default=4096)
    ap.add_argument("--path", default=None)
    args = ap.parse_args()
    rank, ws = start()
    M, N, K = args.m, args.n, args.k
    try:
        config = cfg.load_config(M, N, K, args.path)
        cfg.validate_stage2(config, M, N)
    except (FileNotFoundError, ValueError):
        config = default_config(M, N)
    torch.manual_seed(100 + rank)
    x = torch.ones((M, K), dtype=torch.float16, device="cuda")
    golden = RowParallelLayer(K, N, "all_reduce", None)
    with torch.no_grad():
        golden.weight.normal_(0.0, 0.5 / K ** 0.5)
    layer = OverlapRowParallelLayer(rank, ws, K, N, M, config, "all_reduce", broadcast_nccl_id())
    layer.weight = golden.weight
    norm_ref = RMSNorm(N)
    dist.broadcast(norm_ref.weight.data, src=0)
    norm = ReorderRMSNorm(N, M, config["BM"], config["BN"], config["hint"], eps=norm_ref.eps)
    norm.weight = norm_ref.weight
    with torch.no_grad():
        y1 = norm_ref(golden(x))
        y2 = norm(layer(x))
        fused = FusedRowParallelLinear(make_overlap_impl(), K, N, "all_reduce", norm=True, eps=norm_ref.eps,
                                       algo=config["Algo"])
        fused.weight, fused.norm_weight = golden.weight, norm_ref.weight
        y3 = fused(x)
    torch.cuda.synchronize()
    layer.overlap_class.check_status()
    ok2 = torch.allclose(y1, y2, atol=1e-2, rtol=1e-2)
    ok3 = torch.allclose(y1, y3, atol=1e-2, rtol=1e-2)
    flag = torch.tensor([int(ok2 and ok3)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN) if ws > 1 else None
    if rank == 0:
        print(f"overlap + ReorderRMSNorm all close: {ok2}; fused kernel all close: {ok3}; "
              f"max diff {float((y1.float() - y2.float()).abs().max()):.4g} / "
              f"{float((y1.float() - y3.float()).abs().max()):.4g}")
        print("PASS" if flag.item() == 1 else "FAIL")
    finish()
    raise SystemExit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
