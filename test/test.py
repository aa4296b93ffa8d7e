"""Speed test (reference: test/test.py:120-391): GEMM, vendor GEMM, collective,
non-overlapped baseline (vendor GEMM then NCCL) and the fused operation, each as
the mean of 200 event-timed repetitions after 20 warm-ups, MAX over ranks, and
``speedup = baseline / overlap``.  Also prints the roofline fraction of the fused
time and writes one JSON line per run (``--jsonl``).

    torchrun --nproc_per_node=8 test/test.py --m_dim 4096 --n_dim 8192 --k_dim 1024 --comm_op all_reduce
    ... --single_seg     (no overlap: own GEMM, then one NCCL collective)
    ... --rmsnorm        (include RMSNorm on both sides)
"""
import argparse
import json

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import (DTYPES, finish, make_baseline_impl, make_overlap_impl, measured_link_gbs,  # noqa: E402
                                   measured_peaks, start)
from flashoverlap_b200.tune.model import div_up  # noqa: E402
from flashoverlap_b200.tune.runtime import make_inputs, mean_time_ms, search_two_stream  # noqa: E402
from flashoverlap_b200.utils import config as cfg  # noqa: E402
from flashoverlap_b200.utils.reorder import generate_row_mapping, reorder_indices  # noqa: E402


def build_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m_dim", "--m", type=int, default=4096)
    ap.add_argument("--k_dim", "--k", type=int, default=8192)
    ap.add_argument("--n_dim", "--n", type=int, default=8192)
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter"])
    ap.add_argument("--single_seg", action="store_true")
    ap.add_argument("--rmsnorm", action="store_true")
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    ap.add_argument("--reps", type=int, default=200)
    ap.add_argument("--path", default=None)
    ap.add_argument("--jsonl", default=None)
    ap.add_argument("--peaks", default=None, help="JSON file with the measured peaks (default: MEASURED_PEAKS.json)")
    return ap


def main(argv=None, rendezvous_retries=0):
    args = build_parser().parse_args(argv)
    rank, ws = start(retries=rendezvous_retries)
    M, N, K = args.m_dim, args.n_dim, args.k_dim
    dtype = DTYPES[args.dtype]
    try:
        sol = cfg.load_config(M, N, K, args.path)
        cfg.validate_stage2(sol, M, N)
    except (FileNotFoundError, ValueError) as exc:
        if rank == 0:
            print(f"no tuned config ({exc}); using the default 256x256 tile")
        algo = 3 if M % 256 == 0 and N % 256 == 0 else 1
        BM, BN, _ = cfg.ALGO_TILES[algo]
        tiles = (M // BM) * (N // BN)
        sol = {"BM": BM, "BN": BN, "Algo": algo, "hint": [], "cSeg": [max(tiles - 1, 1), 1] if tiles > 1 else [1]}
    BM, BN, algo = sol["BM"], sol["BN"], sol["Algo"]
    cseg = [(M // BM) * (N // BN)] if args.single_seg else sol["cSeg"]
    impl, base = make_overlap_impl(), make_baseline_impl()
    impl.set_raster_group(int(sol.get("raster_group", 0)))
    A, B, C = make_inputs(M, N, K, dtype)
    W = torch.empty(N, dtype=dtype, device="cuda").normal_(1.0, 0.1)
    D = torch.empty((M // ws, N), dtype=dtype, device="cuda")
    O = torch.empty_like(C if args.comm_op == "all_reduce" else D)
    tm, tn = div_up(M, BM), div_up(N, BN)
    RA = reorder_indices(tm * tn, sol["hint"], device="cuda").reshape(tm, tn)
    MM = torch.zeros(max(tn, len(cseg)), dtype=torch.int32, device="cuda")
    cs_cpu = torch.tensor(cseg, dtype=torch.int32)
    cs_gpu = cs_cpu.cuda()
    RE = generate_row_mapping(M, N, BM, BN, cseg, ws, device="cuda") if args.comm_op == "reduce_scatter" else None
    ar = args.comm_op == "all_reduce"
    r = args.reps
    t_gemm = mean_time_ms(lambda: impl.cutlass_gemm(A, B, C, algo), 20, r)
    t_vendor = mean_time_ms(lambda: base.cublas_gemm(A, B, C), 20, r)
    t_comm = mean_time_ms((lambda: base.nccl_allreduce(C)) if ar else (lambda: base.nccl_reducescatter(C)), 20, r)

    def baseline():
        if ar:
            base.gemm_allreduce(A, B, C)
        else:
            base.gemm_reducescatter(A, B, C, D)
        if args.rmsnorm:
            torch.ops.flashoverlap_op.rmsnorm(C if ar else D, O, W, 1e-5)

    def overlap():
        if args.single_seg:
            if ar:
                impl.gemm_allreduce(A, B, C, algo)
            else:
                impl.gemm_reducescatter(A, B, C, D, algo)
            if args.rmsnorm:
                torch.ops.flashoverlap_op.rmsnorm(C if ar else D, O, W, 1e-5)
        elif args.rmsnorm:
            if ar:
                impl.gemm_allreduce_fused(A, B, W, 1e-5, algo)
            else:
                impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, algo, False)
        elif ar:
            impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cs_cpu, cs_gpu, algo, False)
        else:
            impl.gemm_reducescatter_overlap(A, B, C, D, MM, RA, RE, 1, cs_cpu, cs_gpu, algo, False)

    def two_stream():
        if ar:
            impl.gemm_allreduce_twostream(A, B, C, MM, RA, 1, cs2_cpu, cs2_gpu, algo, 0)
        else:
            impl.gemm_reducescatter_twostream(A, B, C, D, MM, RA, RE2, 1, cs2_cpu, cs2_gpu, algo, 0)
        if args.rmsnorm:
            torch.ops.flashoverlap_op.reorder_rmsnorm(C if ar else D, O, W, BM if ar else BM // ws, BN, 1, RA)

    # The reference's own design on this machine, with the wave grouping its
    # search found for this shape (the tuned file's cSeg) or, without a tuned
    # file, the best of a quick timed search over compositions of <= 4 units.
    tiles = tm * tn
    if "two_stream_dur" in sol and sum(sol["cSeg"]) == tiles and len(sol["cSeg"]) < tn:
        groups = list(sol["cSeg"])
    elif ws > 1:
        groups, _, _ = search_two_stream(impl, M, N, K, algo, args.comm_op, dtype, max_units=4, warmup=3, reps=10,
                                         hint=sol["hint"])
    else:
        groups = [tiles]
    cs2_cpu = torch.tensor(groups, dtype=torch.int32)
    cs2_gpu = cs2_cpu.cuda()
    RE2 = generate_row_mapping(M, N, BM, BN, groups, ws, device="cuda") if not ar else None
    MM = torch.zeros(max(tn, len(groups), len(cseg)), dtype=torch.int32, device="cuda")
    t_two = mean_time_ms(two_stream, 20, r)
    t_base = mean_time_ms(baseline, 20, r)
    t_over = mean_time_ms(overlap, 20, r)
    impl.check_status()
    # roofline: the slower of the GEMM at the measured peak and the bytes one GPU must move per NVLink direction
    # at the measured link bandwidth; both numbers come from measurement files, none is typed in here
    flop = 2.0 * M * N * K
    peaks = measured_peaks(args.peaks)
    link_gbs, link_src = measured_link_gbs(ws, path=args.path)
    nvls = impl.nvls_available()
    S = M * N * A.element_size()
    if ws == 1:
        out_bytes = 0.0
    elif ar:
        out_bytes = S * (1 + 1 / ws) if nvls else 2 * S * (ws - 1) / ws
    else:
        out_bytes = S * (ws - 1) / ws
    roof_ms = None
    if peaks.get("bf16_tflops") and (ws == 1 or link_gbs):
        roof_ms = max(flop / (peaks["bf16_tflops"] * 1e12), out_bytes / (link_gbs * 1e9) if ws > 1 else 0.0) * 1e3
    if rank == 0:
        print(f"M={M} N={N} K={K} (per rank) TP={ws} {args.dtype} comm_op={args.comm_op} Algo={algo} cSeg={cseg}")
        print("GEMM dur:        %.4f ms" % t_gemm)
        print("vendor GEMM dur: %.4f ms" % t_vendor)
        print("comm dur:        %.4f ms" % t_comm)
        print("baseline dur:    %.4f ms" % t_base)
        print("overlap dur:     %.4f ms" % t_over)
        print("two-stream dur:  %.4f ms   (reference design: signalling GEMM + stream waits + %d NCCL calls)" % (t_two, len(groups)))
        print("speedup:         %.4f" % (t_base / t_over))
        if roof_ms is not None:
            print("roofline:        %.4f ms -> fused reaches %.1f %% of it (of measured: %.0f TFLOP/s, %s GB/s from %s)"
                  % (roof_ms, 100 * roof_ms / t_over, peaks["bf16_tflops"], link_gbs, link_src or "-"))
        else:
            print("roofline:        not computed (no measured peaks / link curve found)")
        if args.jsonl:
            with open(args.jsonl, "a") as fh:
                fh.write(json.dumps({"M": M, "N": N, "K": K, "tp": ws, "dtype": args.dtype, "comm_op": args.comm_op,
                                     "rmsnorm": args.rmsnorm, "single_seg": args.single_seg, "algo": algo,
                                     "gemm_ms": t_gemm, "vendor_gemm_ms": t_vendor, "comm_ms": t_comm,
                                     "baseline_ms": t_base, "overlap_ms": t_over, "two_stream_ms": t_two, "speedup": t_base / t_over,
                                     "two_stream_cseg": groups, "roofline_ms": roof_ms,
                                     "roofline_frac": (roof_ms / t_over) if roof_ms else None}) + "\n")
    finish()


if __name__ == "__main__":
    main()
