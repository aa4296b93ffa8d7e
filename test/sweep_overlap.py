"""Shape sweep of the fused operations against the non-overlapped baseline
(cuBLAS GEMM, one NCCL collective, RMSNorm kernel) at the tensor-parallel size
of this job: M in {1024..16384}, N in {4096, 8192}, K in {4096, 8192, 14336}
split over the ranks, fp16 by default.  Steps of both sides alternate, the L2
is flushed before every step, times are the MAX over ranks.

    torchrun --nproc_per_node=8 test/sweep_overlap.py [--m_list 1024 4096] [--jsonl sweep.jsonl]
"""
import argparse
import json

from _common import DTYPES, finish, make_baseline_impl, make_overlap_impl, start, torch

from flashoverlap_b200.parallel import max_over_ranks
from flashoverlap_b200.utils.timing import time_pairs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m_list", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--n_list", type=int, nargs="+", default=[4096, 8192])
    ap.add_argument("--k_list", type=int, nargs="+", default=[4096, 8192, 14336], help="K before the split")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--jsonl", default=None)
    args = ap.parse_args()
    rank, ws = start()
    dt = DTYPES[args.dtype]
    impl = make_overlap_impl(max_m=max(args.m_list), max_n=max(args.n_list))
    base = make_baseline_impl()
    if rank == 0:
        print(f"TP={ws} {args.dtype}\n{'M':>6} {'N':>6} {'K/rank':>7} | {'AR fused':>9} {'AR base':>9} {'x':>5} | "
              f"{'RS fused':>9} {'RS base':>9} {'x':>5}   (ms, with RMSNorm)")
    for M in args.m_list:
        if M % ws or (M // ws) % 128:
            continue
        algo = 3 if M % 256 == 0 else 0
        for N in args.n_list:
            for Kt in args.k_list:
                K = Kt // ws // 8 * 8
                A = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dt)
                B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
                W = torch.ones(N, device="cuda", dtype=dt)
                C = torch.empty(M, N, device="cuda", dtype=dt)
                O = torch.empty_like(C)
                D = torch.empty(M // ws, N, device="cuda", dtype=dt)
                DO = torch.empty_like(D)

                def b_ar():
                    base.gemm_allreduce(A, B, C)
                    torch.ops.flashoverlap_op.rmsnorm(C, O, W, 1e-5)

                def b_rs():
                    base.gemm_reducescatter(A, B, C, D)
                    torch.ops.flashoverlap_op.rmsnorm(D, DO, W, 1e-5)

                f1, b1 = time_pairs(lambda: impl.gemm_allreduce_fused(A, B, W, 1e-5, algo), b_ar, args.steps, 3)
                f2, b2 = time_pairs(lambda: impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, algo, False), b_rs,
                                    args.steps, 3)
                t = [max_over_ranks(sum(x)) / args.steps for x in (f1, b1, f2, b2)]
                impl.check_status()
                if rank == 0:
                    print(f"{M:>6} {N:>6} {K:>7} | {t[0]:>9.4f} {t[1]:>9.4f} {t[1] / t[0]:>5.2f} | {t[2]:>9.4f} "
                          f"{t[3]:>9.4f} {t[3] / t[2]:>5.2f}", flush=True)
                    if args.jsonl:
                        with open(args.jsonl, "a") as fh:
                            fh.write(json.dumps({"tp": ws, "dtype": args.dtype, "M": M, "N": N, "K_per_rank": K,
                                                 "ar_fused_ms": t[0], "ar_baseline_ms": t[1], "rs_fused_ms": t[2],
                                                 "rs_baseline_ms": t[3]}) + "\n")
                del A, B, C, O, D, DO
    finish()


if __name__ == "__main__":
    main()
