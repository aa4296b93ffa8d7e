"""GEMM + ReduceScatter + RMSNorm against PyTorch (reference:
example/correctness_rs.py:100-142; tolerance 5e-2, prints the worst element).
The overlapped layer keeps the rows ``r, r + size, ...`` on rank r, so the golden
path feeds the same rows grouped by ``row % size`` to reduce_scatter_tensor.

    torchrun --nproc_per_node=2 example/correctness_rs.py --m_dim 4096 --n_dim 8192 --k_dim 4096
(under torchrun spell the options --m_dim/--n_dim/--k_dim: torchrun itself claims the prefix --m)
"""
import argparse

import torch.distributed as dist
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import finish, make_overlap_impl, start  # noqa: E402
from correctness_ar import default_config

from flashoverlap_b200.models import FusedRowParallelLinear, OverlapRowParallelLayer, ReorderRMSNorm, RMSNorm, \
    RowParallelLayer
from flashoverlap_b200.parallel import broadcast_nccl_id
from flashoverlap_b200.utils import config as cfg
from flashoverlap_b200.utils.reorder import reorder_rows_by_world_size


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
    torch.manual_seed(200 + rank)
    x = torch.empty((M, K), dtype=torch.float16, device="cuda").normal_(0.0, 0.5)
    golden = RowParallelLayer(K, N, "reduce_scatter", None)
    with torch.no_grad():
        golden.weight.normal_(0.0, 0.5 / K ** 0.5)
    layer = OverlapRowParallelLayer(rank, ws, K, N, M, config, "reduce_scatter", broadcast_nccl_id())
    layer.weight = golden.weight
    norm_ref = RMSNorm(N)
    dist.broadcast(norm_ref.weight.data, src=0)
    norm = ReorderRMSNorm(N, M // ws, config["BM"] // ws, config["BN"], config["hint"], eps=norm_ref.eps)
    norm.weight = norm_ref.weight
    with torch.no_grad():
        y1 = norm_ref(golden(reorder_rows_by_world_size(x, ws)))
        y2 = norm(layer(x))
        fused = FusedRowParallelLinear(make_overlap_impl(), K, N, "reduce_scatter", norm=True, eps=norm_ref.eps,
                                       algo=config["Algo"], interleave=True)
        fused.weight, fused.norm_weight = golden.weight, norm_ref.weight
        y3 = fused(x)
    torch.cuda.synchronize()
    layer.overlap_class.check_status()
    diff = (y1.float() - y2.float()).abs()
    idx = int(diff.argmax())
    ok2 = torch.allclose(y1, y2, atol=5e-2, rtol=5e-2)
    ok3 = torch.allclose(y1, y3, atol=5e-2, rtol=5e-2)
    flag = torch.tensor([int(ok2 and ok3)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN) if ws > 1 else None
    if rank == 0:
        r, c = divmod(idx, N)
        print(f"worst element ({r}, {c}): golden {float(y1[r, c]):.4f} overlap {float(y2[r, c]):.4f} "
              f"diff {float(diff.max()):.4g}")
        print(f"overlap + ReorderRMSNorm all close: {ok2}; fused kernel all close: {ok3}")
        print("PASS" if flag.item() == 1 else "FAIL")
    finish()
    raise SystemExit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
