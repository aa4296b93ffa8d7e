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

from _common import DTYPES, finish, make_baseline_impl, make_overlap_impl, start, torch

from flashoverlap_b200.tune.model import div_up
from flashoverlap_b200.tune.runtime import make_inputs, mean_time_ms
from flashoverlap_b200.utils import config as cfg
from flashoverlap_b200.utils.reorder import generate_row_mapping, reorder_indices

PEAK_TFLOPS = 1629.4   # measured cuBLAS bf16 burst on this pool
LINK_GBS = 770.0       # measured peer copy bandwidth per direction


def main():
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
    args = ap.parse_args()
    rank, ws = start()
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
    impl.set_reduce_group(int(sol.get("reduce_group", 0)))
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

    # the reference's own design on this machine: wave groups of (SMs - 16) tiles
    ctas_per_tile = BM // 128
    wave = max(1, (torch.cuda.get_device_properties(0).multi_processor_count - 16) // ctas_per_tile)
    tiles = tm * tn
    groups = [min(wave, tiles - i) for i in range(0, tiles, wave)]
    if len(groups) >= tn:
        groups = [tiles]
    cs2_cpu = torch.tensor(groups, dtype=torch.int32)
    cs2_gpu = cs2_cpu.cuda()
    RE2 = generate_row_mapping(M, N, BM, BN, groups, ws, device="cuda") if not ar else None
    MM = torch.zeros(max(tn, len(groups), len(cseg)), dtype=torch.int32, device="cuda")
    t_two = mean_time_ms(two_stream, 20, r)
    t_base = mean_time_ms(baseline, 20, r)
    t_over = mean_time_ms(overlap, 20, r)
    impl.check_status()
    flop = 2.0 * M * N * K
    out_bytes = M * N * A.element_size() * (ws - 1) / ws * (2 if ar else 1)
    roof_ms = max(flop / (PEAK_TFLOPS * 1e12), out_bytes / (LINK_GBS * 1e9)) * 1e3
    if rank == 0:
        print(f"M={M} N={N} K={K} (per rank) TP={ws} {args.dtype} comm_op={args.comm_op} Algo={algo} cSeg={cseg}")
        print("GEMM dur:        %.4f ms" % t_gemm)
        print("vendor GEMM dur: %.4f ms" % t_vendor)
        print("comm dur:        %.4f ms" % t_comm)
        print("baseline dur:    %.4f ms" % t_base)
        print("overlap dur:     %.4f ms" % t_over)
        print("two-stream dur:  %.4f ms   (reference design: signalling GEMM + stream waits + %d NCCL calls)" % (t_two, len(groups)))
        print("speedup:         %.4f" % (t_base / t_over))
        print("roofline:        %.4f ms -> fused reaches %.1f %% of it" % (roof_ms, 100 * roof_ms / t_over))
        if args.jsonl:
            with open(args.jsonl, "a") as fh:
                fh.write(json.dumps({"M": M, "N": N, "K": K, "tp": ws, "dtype": args.dtype, "comm_op": args.comm_op,
                                     "rmsnorm": args.rmsnorm, "single_seg": args.single_seg, "algo": algo,
                                     "gemm_ms": t_gemm, "vendor_gemm_ms": t_vendor, "comm_ms": t_comm,
                                     "baseline_ms": t_base, "overlap_ms": t_over, "two_stream_ms": t_two, "speedup": t_base / t_over,
                                     "roofline_ms": roof_ms, "roofline_frac": roof_ms / t_over}) + "\n")
    finish()


if __name__ == "__main__":
    main()
