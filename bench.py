#!/usr/bin/env python
"""Headline benchmark: the row-parallel attention out-projection of the
reference's headline configuration, GEMM + AllReduce + RMSNorm in fp16 with
M = 4096 tokens, N = 8192 hidden, K = 8192 split over the GPUs, as ONE fused
sm_100a kernel per step.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints one JSON line.  ``value`` is the aggregate rate of the whole job
(2*M*N*K_total FLOP per step over the slowest rank's device time), measured with
CUDA events around every step with an L2 flush before each; ``e2e`` is the same
step through ``FusedRowParallelLinear.forward`` including the host-to-device
copy of the step's activations and the device-to-host read of a result row.
The same run also times the non-overlapped path the reference calls its
baseline (vendor GEMM, then one NCCL collective, then RMSNorm; reference:
src/baseline_impl.cu:35-70) and a second shape (reduce-scatter, bf16) and
reports them in ``detail``.

``--impl reference`` reports that the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REFERENCE_UNAVAILABLE = (
    "reference cannot be installed: the checkout is the MUSA port (needs mcc, MUTlass, MCCL, torch_musa), "
    "has no setup.py/pyproject.toml (pip: 'Neither setup.py nor pyproject.toml found') and its CUTLASS submodule is empty"
)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", type=int, default=3, help="tile configuration (3 = 256x256 CTA pair)")
    ap.add_argument("--no-detail", action="store_true", help="skip the baseline and the second shape")
    return ap.parse_args()


def main():
    args = parse()
    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    import flashoverlap_b200  # noqa: F401
    from flashoverlap_b200.models import FusedRowParallelLinear
    from flashoverlap_b200.parallel import init_distributed, make_baseline_impl, make_overlap_impl, max_over_ranks
    from flashoverlap_b200.utils.clocks import ClockSampler
    from flashoverlap_b200.utils.timing import time_pairs, time_steps

    if not torch.cuda.is_available():
        print(json.dumps({"error": "bench.py needs a CUDA device"}))
        return 1
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    rank, world, local_rank = init_distributed()
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE is {world}; using {world}", file=sys.stderr)
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234 + rank)

    M, N, K_total = 4096, 8192, 8192
    K = K_total // world
    eps = 1e-5
    dtype = torch.float16
    impl = make_overlap_impl()
    layer = FusedRowParallelLinear(impl, K, N, comm_op="all_reduce", norm=True, eps=eps, algo=args.algo,
                                   dtype=dtype, device=dev)
    # random-init weights ~ N(0,1)/sqrt(K); activations ~ N(0,1)/sqrt(K)
    with torch.no_grad():
        layer.weight.copy_((torch.randn(N, K, device=dev) / K ** 0.5).to(dtype))
        layer.norm_weight.copy_((1 + 0.1 * torch.randn(N, device=dev)).to(dtype))
    x_host = (torch.randn(M, K) / K ** 0.5).to(dtype).pin_memory()
    x = x_host.to(dev)
    row_host = torch.empty(N, dtype=dtype).pin_memory()

    def step():
        layer(x)

    # ---- device-timed steps ---------------------------------------------------
    with ClockSampler(torch.cuda.current_device()) as sampler:
        times = time_steps(step, steps, warmup, flush=True)
    clocks = sampler.summary()
    impl.check_status()
    total_ms = max_over_ranks(sum(times))
    ms_per_step = total_ms / steps
    flop = 2.0 * M * N * K_total
    value = flop / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API -------------------------------------
    # Every step copies its activations from pinned host memory and reads a row of
    # the result back.  The copy of step i+1 runs on a copy stream while step i
    # computes (HostFeeder); every timed step still issues exactly one H2D copy
    # and one D2H read inside the timed region.
    from flashoverlap_b200.utils.pipeline import HostFeeder

    feeder = HostFeeder((M, K), dtype, dev)
    feeder.submit(x_host)

    def e2e_step():
        xd = feeder.take()
        feeder.submit(x_host)          # next step's input starts travelling now
        out = layer(xd)
        feeder.release(xd)
        row_host.copy_(out[0], non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the result row has arrived on the host

    for _ in range(warmup):
        e2e_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / steps
    if world > 1:
        dist.barrier()
    impl.check_status()
    e2e_value = flop / (e2e_ms * 1e-3) / 1e12

    detail = {}
    if not args.no_detail:
        # non-overlapped baseline: cuBLAS GEMM, NCCL all-reduce, RMSNorm kernel
        base = make_baseline_impl()
        C = torch.empty(M, N, device=dev, dtype=dtype)
        O = torch.empty(M, N, device=dev, dtype=dtype)

        def base_step():
            base.gemm_allreduce(x, layer.weight, C)
            torch.ops.flashoverlap_op.rmsnorm(C, O, layer.norm_weight, eps)

        # fused and baseline steps alternate so that both see the same clocks
        ft, bt = time_pairs(step, base_step, steps, warmup)
        fused_ms2 = max_over_ranks(sum(ft)) / steps
        base_ms = max_over_ranks(sum(bt)) / steps
        gt, ct = time_pairs(lambda: impl.cutlass_gemm(x, layer.weight, C, args.algo),
                            lambda: base.cublas_gemm(x, layer.weight, C), steps, warmup)
        gemm_ms = max_over_ranks(sum(gt)) / steps
        cublas_ms = max_over_ranks(sum(ct)) / steps
        detail["ar_fp16"] = {
            "fused_ms": round(fused_ms2, 4), "nccl_baseline_ms": round(base_ms, 4),
            "speedup_vs_nccl_baseline": round(base_ms / fused_ms2, 3), "measured": "alternating steps",
            "own_gemm_ms": round(gemm_ms, 4), "cublas_gemm_ms": round(cublas_ms, 4),
        }
        # second shape: MLP down-projection, GEMM + ReduceScatter + RMSNorm, bf16
        M2, N2, K2_total = 8192, 8192, 28672
        K2 = K2_total // world
        A2 = (torch.randn(M2, K2, device=dev) / K2 ** 0.5).to(torch.bfloat16)
        B2 = (torch.randn(N2, K2, device=dev) / K2 ** 0.5).to(torch.bfloat16)
        W2 = (1 + 0.1 * torch.randn(N2, device=dev)).to(torch.bfloat16)
        D2 = torch.empty(M2 // world, N2, device=dev, dtype=torch.bfloat16)
        C2 = torch.empty(M2, N2, device=dev, dtype=torch.bfloat16)
        O2 = torch.empty_like(D2)
        def base_rs():
            base.gemm_reducescatter(A2, B2, C2, D2)
            torch.ops.flashoverlap_op.rmsnorm(D2, O2, W2, eps)

        rt, brt = time_pairs(lambda: impl.gemm_reducescatter_fused(A2, B2, O2, W2, eps, args.algo, False), base_rs,
                             steps, warmup)
        rs_ms = max_over_ranks(sum(rt)) / steps
        base_rs_ms = max_over_ranks(sum(brt)) / steps
        detail["rs_bf16"] = {
            "M": M2, "N": N2, "K_per_rank": K2, "fused_ms": round(rs_ms, 4), "nccl_baseline_ms": round(base_rs_ms, 4),
            "speedup_vs_nccl_baseline": round(base_rs_ms / rs_ms, 3),
            "tflops": round(2.0 * M2 * N2 * K2_total / (rs_ms * 1e-3) / 1e12, 1),
        }
        impl.check_status()

    if rank == 0:
        line = {
            "metric": "fused GEMM+AllReduce+RMSNorm throughput (aggregate TFLOP/s; latency in ms_per_step)",
            "value": round(value, 2),
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp16",
            "data": "synthetic (random-init weights and activations ~ N(0,1)/sqrt(K))",
            "config": {
                "model": "row-parallel attention out-projection, GEMM+AllReduce+RMSNorm",
                "M": M, "N": N, "K_total": K_total, "K_per_rank": K,
                "global_batch": M, "seq_len": M, "parallelism": f"tp{world}",
                "l2": "flushed between timed iterations (256 MB write)",
                "timing": "CUDA events per step, max over ranks",
                "algo": args.algo,
            },
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "power_w_max": clocks["power_w_max"], "samples": clocks["samples"],
                       "samples_under_load": clocks["samples_under_load"]},
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 5),
                    "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": row_host.numel() * row_host.element_size(),
                    "api": "HostFeeder + FusedRowParallelLinear.forward", "timing": "wall clock, max over ranks",
                    "note": "H2D of the next step overlaps the current step (double-buffered)"},
            "gpu_launches": steps,
            "impl": "ours",
            "detail": detail,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
