"""Row-parallel layers under the reference's module name (reference:
example/RowParallelLinear.py), and, run as a script, the layers side by side
on the ranks of the job (one process per GPU, or a single process):

    torchrun --nproc_per_node=4 example/RowParallelLinear.py [--tokens 4096 --hidden 8192 --in_features 8192]

``RowParallelLayer`` (``torch.matmul`` + one NCCL collective: the non-overlapped
path), ``FusedRowParallelLinear`` (one fused kernel, all-reduce and
reduce-scatter form, with and without the fused RMSNorm) and
``OverlapRowParallelLayer`` (the reference-compatible overlap call, whose
tile-reordered output is put back in order here) are run on the same input;
the script prints the largest difference to the PyTorch path and the time per
call.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from flashoverlap_b200.models.row_parallel import (  # noqa: F401,E402
    FusedRowParallelLinear,
    HierarchicalRowParallelLinear,
    OverlapRowParallelLayer,
    RowParallelLayer,
)


def main():
    import torch.distributed as dist

    from flashoverlap_b200.cli import DTYPES, finish, make_overlap_impl, start
    from flashoverlap_b200.parallel import broadcast_nccl_id, max_over_ranks
    from flashoverlap_b200.utils.reorder import from_tile_order
    from flashoverlap_b200.utils.timing import time_steps

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=8192, help="output features")
    ap.add_argument("--in_features", type=int, default=8192, help="input features before the split over the ranks")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--algo", type=int, default=8)
    args = ap.parse_args()
    rank, ws = start()
    dt = DTYPES[args.dtype]
    M, N, K = args.tokens, args.hidden, args.in_features // ws
    impl = make_overlap_impl(max_m=M, max_n=N)
    torch.manual_seed(11 + rank)
    x = (torch.randn(M, K, device="cuda") / (K * ws) ** 0.5).to(dt)
    w = torch.randn(N, K, device="cuda").to(dt)
    gamma = (1 + 0.1 * torch.randn(N, generator=torch.Generator().manual_seed(5))).to("cuda", dt)  # same on every rank
    rows = M // ws

    def med(fn):
        return max_over_ranks(sorted(time_steps(fn, 10, 3))[5]) * 1e3

    def report(name, got, want, us, base_us):
        err = (got.float() - want.float()).abs().max().item() / max(1.0, want.float().abs().max().item())
        flag = torch.tensor([err], device="cuda")
        if ws > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"{name:<46} max rel. diff {flag.item():.2e}   {us:8.1f} us   ({base_us / us:.2f}x of matmul + NCCL)")
        return flag.item() <= 2e-2

    ok = True
    for comm_op in ("all_reduce", "reduce_scatter"):
        plain = RowParallelLayer(K, N, comm_op, dtype=dt)
        fused = FusedRowParallelLinear(impl, K, N, comm_op=comm_op, norm=False, algo=args.algo, dtype=dt)
        fused_norm = FusedRowParallelLinear(impl, K, N, comm_op=comm_op, norm=True, algo=args.algo, dtype=dt)
        with torch.no_grad():
            for layer in (plain, fused, fused_norm):
                layer.weight.copy_(w)
            fused_norm.norm_weight.copy_(gamma)
            want = plain(x)
            base_us = med(lambda: plain(x))
            ok &= report(f"FusedRowParallelLinear {comm_op}", fused(x).clone(), want, med(lambda: fused(x)), base_us)
            wf = want.float()
            want_norm = wf * torch.rsqrt(wf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()

            def plain_norm():
                y = plain(x).float()
                return (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).to(dt)

            ok &= report(f"FusedRowParallelLinear {comm_op} + RMSNorm", fused_norm(x).clone(), want_norm,
                         med(lambda: fused_norm(x)), med(plain_norm))
    # the reference-compatible layer: one wave group, completion order = tile order
    bm, bn = impl.algo_tile(args.algo)[0], impl.algo_tile(args.algo)[1]
    tiles = (M // bm) * (N // bn)
    config = {"BM": bm, "BN": bn, "Algo": args.algo, "hint": [], "cSeg": [tiles]}
    compat = OverlapRowParallelLayer(rank, ws, K, N, M, config, "all_reduce", broadcast_nccl_id(), dtype=dt)
    with torch.no_grad():
        compat.weight.copy_(w)
        plain = RowParallelLayer(K, N, "all_reduce", dtype=dt)
        plain.weight.copy_(w)
        want = plain(x)
        got = from_tile_order(compat(x), bm, bn, compat.reorder_array.reshape(-1))
        ok &= report("OverlapRowParallelLayer all_reduce (reordered)", got, want, med(lambda: compat(x)),
                     med(lambda: plain(x)))
    impl.check_status()
    compat.overlap_class.check_status()
    if rank == 0:
        print("PASS" if ok else "FAIL")
    finish()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
