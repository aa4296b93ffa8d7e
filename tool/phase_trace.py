"""Device-side phase trace of the fused kernels on the GPUs of this job.

A profiler cannot replay a kernel that waits for other ranks, so the fused
kernels can record their own timeline (``OverlapImpl.set_phase_trace``): per
CTA the kernel start, the end of the GEMM phase, the first and the last row
this CTA reduced and, for an all-reduce, the moment every row had been
delivered to this rank; for all-gather -> GEMM the moment this rank's pushes
were out and the moment the first tile that needs another rank's rows could
start.  This tool runs the named shapes with the trace on and prints one line
per rank (microseconds after the kernel start).

    torchrun --nproc_per_node=8 tool/phase_trace.py [--md profiles/x.md]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from flashoverlap_b200.cli import DTYPES, finish, make_overlap_impl, start  # noqa: E402
from flashoverlap_b200.utils.timing import flush_l2, time_steps  # noqa: E402

SHAPES = [  # (name, op, M, N, K before the split, dtype)
    ("AR fp16 M4096 N8192 K8192", "all_reduce", 4096, 8192, 8192, "float16"),
    ("RS bf16 M8192 N8192 K28672", "reduce_scatter", 8192, 8192, 28672, "bfloat16"),
]


def gather_trace(impl, rank, ws, sms, args):
    """All-gather -> GEMM on the decoder block's QKV shape (M 8192 tokens, K 8192, N 10240 / ranks, bf16)."""
    from flashoverlap_b200.tune.model import gather_algo_candidates
    from flashoverlap_b200.utils.config import ALGO_TILES

    M, K, N = 8192, 8192, 10240 // ws
    algo = args.ag_algo if args.ag_algo >= 0 else (gather_algo_candidates(M // ws, N)[0] if ws > 1 else args.algo)
    dt = torch.bfloat16
    shard = (torch.randn(M // ws, K, device="cuda") / K ** 0.5).to(dt)
    full = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dt)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
    C = torch.empty(M, N, device="cuda", dtype=dt)
    ts = time_steps(lambda: impl.allgather_gemm(shard, B, C, algo), 10, 3)
    tg = time_steps(lambda: impl.cutlass_gemm(full, B, C, algo), 10, 3)
    trace = torch.zeros(8 * sms, dtype=torch.int64, device="cuda")
    impl.set_phase_trace(trace)
    flush_l2()
    if ws > 1:
        dist.barrier()
    impl.allgather_gemm(shard, B, C, algo)
    torch.cuda.synchronize()
    impl.set_phase_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
    impl.check_status()
    t = trace.view(sms, 8).cpu()
    t0 = t[:, 0].min()
    ge = (t[:, 1] - t0).double() / 1e3
    push = ((t[:, 2] - t0).double() / 1e3).max().item() if (t[:, 2] > 0).any() else float("nan")
    started = t[:, 4][(t[:, 4] > 0) & (t[:, 4] != -1)]  # -1 = never waited for a remote row
    first_remote = (started.min() - t0).item() / 1e3 if started.numel() else float("nan")
    row = torch.tensor([sorted(ts)[len(ts) // 2] * 1e3, sorted(tg)[len(tg) // 2] * 1e3, push, first_remote,
                        ge.min().item(), ge.median().item(), ge.max().item()], dtype=torch.float64, device="cuda")
    rows = [torch.zeros_like(row) for _ in range(ws)]
    if ws > 1:
        dist.all_gather(rows, row)
    else:
        rows = [row]
    out = []
    if rank == 0:
        tile = ALGO_TILES[algo]
        sent = (ws - 1) * shard.numel() * 2 / 1e6
        out.append(f"\n### all-gather -> GEMM bf16 M{M} K{K} N{N} per rank, TP={ws}, Algo {algo} "
                   f"({tile[0]}x{tile[1]}x{tile[2]}), {sent:.0f} MB pushed per rank\n")
        out.append("| rank | fused (us, events) | GEMM alone on gathered rows | own pushes out | first tile on remote rows "
                   "starts | GEMM phase ends min / median / max | push GB/s (sent / time of the pushes) |\n"
                   "|---|---|---|---|---|---|---|")
        for r, v in enumerate(rows):
            v = v.tolist()
            gbs = sent * 1e6 / (v[2] * 1e-6) / 1e9 if v[2] == v[2] and v[2] > 0 else float("nan")
            out.append(f"| {r} | {v[0]:.0f} | {v[1]:.0f} | {v[2]:.0f} | {v[3]:.0f} | {v[4]:.0f} / {v[5]:.0f} / {v[6]:.0f} | "
                       f"{gbs:.0f} |")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--algo", type=int, default=8)
    ap.add_argument("--ag_algo", type=int, default=-1, help="tile configuration of the all-gather GEMM (-1: by model)")
    ap.add_argument("--md", default=None)
    args = ap.parse_args()
    rank, ws = start()
    impl = make_overlap_impl()
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    lines = []
    for name, op, M, N, Kt, dtn in SHAPES:
        dt = DTYPES[dtn]
        K = Kt // ws
        A = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dt)
        B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
        W = torch.ones(N, device="cuda", dtype=dt)
        D = torch.empty(M // ws, N, device="cuda", dtype=dt)
        C = torch.empty(M, N, device="cuda", dtype=dt)

        def fused():
            if op == "all_reduce":
                impl.gemm_allreduce_fused(A, B, W, 1e-5, args.algo)
            else:
                impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, args.algo, False)

        ts = time_steps(fused, 10, 3)
        tg = time_steps(lambda: impl.cutlass_gemm(A, B, C, args.algo), 10, 3)
        trace = torch.zeros(8 * sms, dtype=torch.int64, device="cuda")
        rows_t = torch.zeros(6 * M, dtype=torch.int64, device="cuda")
        impl.set_phase_trace(trace)
        impl.set_row_trace(rows_t)
        flush_l2()
        if ws > 1:
            dist.barrier()
        fused()
        torch.cuda.synchronize()
        impl.set_phase_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
        impl.set_row_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
        impl.check_status()
        t = trace.view(sms, 8).cpu().double()
        t0 = t[:, 0].min()
        used = t[:, 5] > 0
        ge = (t[:, 1] - t0) / 1e3
        first = ((t[used, 4] - t0) / 1e3).min().item() if used.any() else float("nan")
        last = ((t[:, 2] - t0) / 1e3).max().item()
        delivered = (t[0, 6] - t0).item() / 1e3 if t[0, 6] > 0 else float("nan")
        # row timeline of the reduce phase (rows this rank owns): stages of one row, and how many rows were
        # already stored when the last CTA left the GEMM phase
        R = rows_t.view(6, M).cpu().double()
        mine = R[1] > 0
        stage_us = [float("nan")] * 4
        done_early = 0.0
        if mine.any():
            claim, end, ready, summed, bar = R[0][mine], R[1][mine], R[3][mine], R[4][mine], R[5][mine]
            stage_us = [((ready - claim) / 1e3).median().item(), ((summed - ready) / 1e3).median().item(),
                        ((bar - summed) / 1e3).median().item(), ((end - bar) / 1e3).median().item()]
            done_early = ((end - t0) / 1e3 <= ge.max()).double().mean().item()
        row = torch.tensor([sorted(ts)[len(ts) // 2] * 1e3, sorted(tg)[len(tg) // 2] * 1e3, ge.min().item(),
                            ge.median().item(), ge.max().item(), first, last, delivered, *stage_us, done_early],
                           dtype=torch.float64, device="cuda")
        rows = [torch.zeros_like(row) for _ in range(ws)]
        if ws > 1:
            dist.all_gather(rows, row)
        else:
            rows = [row]
        if rank == 0:
            transport = "NVLS" if (op == "all_reduce" and impl.allreduce_uses_nvls()) else "P2P"
            lines.append(f"\n### {name}, TP={ws}, Algo {args.algo}, {transport}\n")
            lines.append("| rank | fused (us, events) | GEMM alone | GEMM phase ends min / median / max | first row reduced "
                         "| last row reduced | all rows delivered |\n|---|---|---|---|---|---|---|")
            for r, v in enumerate(rows):
                v = v.tolist()
                lines.append(f"| {r} | {v[0]:.0f} | {v[1]:.0f} | {v[2]:.0f} / {v[3]:.0f} / {v[4]:.0f} | {v[5]:.0f} | "
                             f"{v[6]:.0f} | {v[7]:.0f} |")
            lines.append("\nOne row in its row group (median, us): wait for the partials / load and sum / barrier / scale "
                         "and store; share of the rank's rows stored before the last CTA left the GEMM phase:\n")
            lines.append("| rank | wait | load + sum | barrier | scale + store | rows stored during the GEMM phase |\n"
                         "|---|---|---|---|---|---|")
            for r, v in enumerate(rows):
                v = v.tolist()
                lines.append(f"| {r} | {v[8]:.2f} | {v[9]:.2f} | {v[10]:.2f} | {v[11]:.2f} | {100 * v[12]:.0f} % |")
    lines += gather_trace(impl, rank, ws, sms, args)
    if rank == 0:
        text = "\n".join(lines) + "\n"
        print(text)
        if args.md:
            with open(args.md, "w") as fh:
                fh.write(text)
    finish()


if __name__ == "__main__":
    main()
