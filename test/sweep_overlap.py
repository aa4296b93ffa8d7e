"""Shape sweep of the fused operations at the tensor-parallel size of this job,
with the exhaustive and the predictive search run side by side on every shape:
M in {1024..16384}, N in {4096, 8192}, K in {4096, 8192, 14336} split over the
ranks, fp16 by default (the sweep the reference's predictive search is meant
for; reference: tune/search.py:529-618).

For every shape and both collectives the script

1. times this library's GEMM for the candidate tile configurations (stage 1),
2. exhaustive: times the fused kernel for every (tile configuration, raster
   group) candidate and keeps the best,
3. predictive: ranks the same candidates with the cost model on the GEMM times
   of step 1 and the link bandwidth MEASURED at the start of the run (the
   library's own transport, 64 MiB messages) and the time one row costs a row
   group (measured with a GEMM of negligible K), and times only the model's first
   ``--top_k`` picks (3, as ``tune.search.predictive_search`` does, against 8 to
   12 candidates for the exhaustive arm); when the two arms' picks differ both are
   timed again in alternation and the gap is the ratio of those times,
4. times the non-overlapped baseline (cuBLAS GEMM, one NCCL collective, RMSNorm
   kernel) in alternation with the best fused configuration.

Times are the MAX over ranks, L2 flushed before every timed step.

    torchrun --nproc_per_node=8 test/sweep_overlap.py [--m_list 1024 4096] [--jsonl sweep.jsonl] [--md sweep.md]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES, finish, make_baseline_impl, make_overlap_impl, start  # noqa: E402
from flashoverlap_b200.parallel import max_over_ranks  # noqa: E402
from flashoverlap_b200.tune.model import predict_fused_ms  # noqa: E402
from flashoverlap_b200.tune.runtime import mean_time_ms, measure_row_us  # noqa: E402
from flashoverlap_b200.tune.search import knob_candidates  # noqa: E402
from flashoverlap_b200.utils.config import ALGO_TILES  # noqa: E402
from flashoverlap_b200.utils.timing import time_pairs  # noqa: E402


def measure_link(impl, ws, reps=10):
    """(GB/s per NVLink direction per GPU, "nvls" | "p2p") of the transport the fused kernels use."""
    if ws == 1:
        return 1.0, "p2p"
    total = 64 << 20
    if impl.allreduce_uses_nvls():
        ms = mean_time_ms(lambda: impl.multimem_bench("allreduce", total, 0, False), 3, reps)
        return total * (1 + 1 / ws) / (ms * 1e-3) / 1e9, "nvls"
    per_peer = total // (ws - 1) // 16 * 16
    ms = mean_time_ms(lambda: impl.p2p_push(per_peer, 0), 3, reps)
    return per_peer * (ws - 1) / (ms * 1e-3) / 1e9, "p2p"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m_list", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--n_list", type=int, nargs="+", default=[4096, 8192])
    ap.add_argument("--k_list", type=int, nargs="+", default=[4096, 8192, 14336], help="K before the split")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--search_reps", type=int, default=5)
    ap.add_argument("--algos", type=int, nargs="+", default=[0, 3, 8], help="tile configurations to consider")
    ap.add_argument("--top_k", type=int, default=3,
                    help="how many of the model's best candidates the predictive arm times (the library's "
                         "predictive_search times 3)")
    ap.add_argument("--jsonl", default=None)
    ap.add_argument("--md", default=None, help="write a markdown table here (rank 0)")
    args = ap.parse_args()
    rank, ws = start()
    dt = DTYPES[args.dtype]
    impl = make_overlap_impl(max_m=max(args.m_list), max_n=max(args.n_list))
    base = make_baseline_impl()
    link_gbs, link_kind = measure_link(impl, ws)
    # what one row of N values costs a row group in the reduce phase (measured once per N and collective)
    row_us = {(op, N): measure_row_us(impl, N, op, dt, algo=args.algos[0]) for op in ("all_reduce", "reduce_scatter")
              for N in args.n_list}
    rows_md = []
    if rank == 0:
        print(f"TP={ws} {args.dtype}; measured link {link_gbs:.0f} GB/s per direction ({link_kind}); row time "
              + ", ".join(f"{op} N={n}: {v:.1f} us" for (op, n), v in row_us.items()))
        print(f"{'op':>3} {'M':>6} {'N':>6} {'K/rank':>7} | {'exh ms':>8} {'pick':>10} | {'pred ms':>8} {'pick':>10} "
              f"{'gap':>6} | {'base ms':>8} {'x':>5}")
    agree = total = 0
    for M in args.m_list:
        if M % ws or (M // ws) % 128:
            continue
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
                algos = [a for a in args.algos if M % ALGO_TILES[a][0] == 0 and N % ALGO_TILES[a][1] == 0
                         and (M // ws) % ALGO_TILES[a][0] == 0]
                def gemm_time(a, rg):  # stage 1: the GEMM alone for every (tile configuration, raster group)
                    impl.set_raster_group(rg)
                    try:
                        return mean_time_ms(lambda: impl.cutlass_gemm(A, B, C, a), 3, args.search_reps, flush=True)
                    finally:
                        impl.set_raster_group(0)

                gemm_ms = {(a, rg): gemm_time(a, rg) for a in algos for rg in knob_candidates(M, ALGO_TILES[a][0])}
                for op in ("all_reduce", "reduce_scatter"):
                    def fused(a):
                        if op == "all_reduce":
                            impl.gemm_allreduce_fused(A, B, W, 1e-5, a)
                        else:
                            impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, a, False)

                    def timed(a, rg):
                        impl.set_raster_group(rg)
                        try:
                            return mean_time_ms(lambda: fused(a), 3, args.search_reps, flush=True)
                        finally:
                            impl.set_raster_group(0)

                    cands = [(a, rg) for a in algos for rg in knob_candidates(M, ALGO_TILES[a][0])]
                    times = {c: timed(*c) for c in cands}                       # exhaustive: everything is timed
                    ex = min(times, key=times.get)
                    kind = link_kind if op == "all_reduce" else "p2p"
                    pred = {c: predict_fused_ms(M, N, gemm_ms[c], ws, op, link_gbs, transport=kind,
                                                tile_m=ALGO_TILES[c[0]][0], raster_group=c[1], row_us=row_us[(op, N)])
                            for c in cands}
                    ranked = sorted(pred, key=pred.get)[:args.top_k]            # predictive: the model's first few
                    pr_times = {c: timed(*c) for c in ranked}                   # picks are timed, the fastest kept
                    pr = min(pr_times, key=pr_times.get)
                    pr_ms = pr_times[pr]
                    if pr == ex:
                        gap = 0.0
                    else:
                        # both picks again, in alternation, so that clock and power drift do not decide the comparison
                        def run_pick(c):
                            impl.set_raster_group(c[1])
                            fused(c[0])

                        tp_, te_ = time_pairs(lambda: run_pick(pr), lambda: run_pick(ex), args.steps, 2)
                        impl.set_raster_group(0)
                        gap = max_over_ranks(sum(tp_)) / max_over_ranks(sum(te_)) - 1.0

                    def b_step():
                        if op == "all_reduce":
                            base.gemm_allreduce(A, B, C)
                            torch.ops.flashoverlap_op.rmsnorm(C, O, W, 1e-5)
                        else:
                            base.gemm_reducescatter(A, B, C, D)
                            torch.ops.flashoverlap_op.rmsnorm(D, DO, W, 1e-5)

                    impl.set_raster_group(ex[1])
                    f, b = time_pairs(lambda: fused(ex[0]), b_step, args.steps, 3)
                    impl.set_raster_group(0)
                    f_ms, b_ms = max_over_ranks(sum(f)) / args.steps, max_over_ranks(sum(b)) / args.steps
                    impl.check_status()
                    total += 1
                    agree += int(gap <= 0.05)
                    rec = {"tp": ws, "dtype": args.dtype, "op": op, "M": M, "N": N, "K_per_rank": K,
                           "exhaustive": {"algo": ex[0], "raster": ex[1], "ms": times[ex], "timed": len(cands)},
                           "predictive": {"algo": pr[0], "raster": pr[1], "ms": pr_ms, "predicted_ms": pred[pr],
                                          "timed": len(ranked)}, "gap": gap, "fused_ms": f_ms, "baseline_ms": b_ms,
                           "speedup": b_ms / f_ms, "link_gbs": link_gbs, "link_kind": kind}
                    if rank == 0:
                        tag = "AR" if op == "all_reduce" else "RS"
                        print(f"{tag:>3} {M:>6} {N:>6} {K:>7} | {times[ex]:>8.4f} {str(ex):>10} | {pr_ms:>8.4f} "
                              f"{str(pr):>10} {100 * gap:>5.1f}% | {b_ms:>8.4f} {b_ms / f_ms:>5.2f}", flush=True)
                        rows_md.append(f"| {tag} | {M} | {N} | {K} | {times[ex]:.4f} | Algo {ex[0]} raster {ex[1]} | "
                                       f"{pr_ms:.4f} | Algo {pr[0]} raster {pr[1]} | {100 * gap:.1f} % | {f_ms:.4f} | "
                                       f"{b_ms:.4f} | {b_ms / f_ms:.2f} |")
                        if args.jsonl:
                            with open(args.jsonl, "a") as fh:
                                fh.write(json.dumps(rec) + "\n")
                del A, B, C, O, D, DO
    if rank == 0:
        summary = (f"predictive pick within 5 % of the exhaustive best on {agree} of {total} cases "
                   f"({100.0 * agree / max(total, 1):.0f} %)")
        print(summary)
        if args.md:
            with open(args.md, "w") as fh:
                fh.write(f"TP = {ws}, {args.dtype}, link {link_gbs:.0f} GB/s per direction ({link_kind}, measured at "
                         f"the start of the run); times in ms, MAX over ranks, RMSNorm included.\n\n")
                fh.write("| op | M | N | K/rank | exhaustive ms | pick | predictive ms | pick | gap | fused | "
                         "cuBLAS+NCCL+RMSNorm | speed-up |\n|---|---|---|---|---|---|---|---|---|---|---|---|\n")
                fh.write("\n".join(rows_md) + "\n\n" + summary + "\n")
    finish()


if __name__ == "__main__":
    main()
