#!/usr/bin/env python
"""Headline benchmark: the row-parallel attention out-projection of the
reference's headline configuration, GEMM + AllReduce + RMSNorm in fp16 with
M = 4096 tokens, N = 8192 hidden, K = 8192 split over the GPUs, as ONE fused
sm_100a kernel per step.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints one JSON line.

* ``value`` / ``ms_per_step``: the fused kernel alone, CUDA events around every
  step with an L2 flush before each, slowest rank; ``value`` is the aggregate
  rate of the whole job (2*M*N*K_total FLOP per step).
* ``vs_baseline``: speed-up over the non-overlapped path the reference calls its
  baseline (vendor GEMM, one NCCL collective on the same stream, RMSNorm kernel;
  reference: src/baseline_impl.cu:35-70), measured in alternation with the
  fused step in the same process.
* ``e2e``: the same step through ``FusedRowParallelLinear.forward`` including,
  every step, the host-to-device copy of the step's activations from pinned
  memory and the device-to-host copy of the WHOLE result.
* ``detail``: the baseline, the reference's two-stream overlap design with a
  searched wave grouping, the second named shape (GEMM + ReduceScatter + RMSNorm
  in bf16), all-gather->GEMM and all-to-all->GEMM timings, and numerical checks
  of every fused operation against fp32 PyTorch and against the NCCL baseline.
  A failed check makes the process exit non-zero.

``--impl reference`` reports that the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
    ap.add_argument("--algo", type=int, default=8, help="tile configuration (8 = 256x256x128 CTA pair)")
    ap.add_argument("--no-detail", action="store_true", help="skip the baseline, the checks and the other shapes")
    return ap.parse_args()


def stats(ts):
    return {"min": round(min(ts), 4), "median": round(statistics.median(ts), 4), "max": round(max(ts), 4)}


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
    from flashoverlap_b200.tune.runtime import search_two_stream
    from flashoverlap_b200.utils.clocks import ClockSampler
    from flashoverlap_b200.utils.pipeline import HostFeeder, ResultReader
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
        # the RMSNorm weight is replicated: the same values on every rank
        gw = torch.Generator(device="cpu").manual_seed(4321)
        layer.norm_weight.copy_((1 + 0.1 * torch.randn(N, generator=gw)).to(dev, dtype))
    x_host = (torch.randn(M, K) / K ** 0.5).to(dtype).pin_memory()
    x = x_host.to(dev)

    def step():
        layer(x)

    def mx(ts):
        """Per-step times of the slowest rank: element-wise maximum over the ranks."""
        if world == 1:
            return list(ts)
        t = torch.tensor(ts, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # ---- device-timed steps ---------------------------------------------------
    with ClockSampler(torch.cuda.current_device()) as sampler:
        times = mx(time_steps(step, steps, warmup, flush=True))
    clocks = sampler.summary()
    impl.check_status()
    ms_per_step = sum(times) / steps
    flop = 2.0 * M * N * K_total
    value = flop / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API -------------------------------------
    # Every step copies its activations from pinned host memory and copies the
    # whole result back into pinned host memory.  Both copies are double
    # buffered (the input of step i+1 and the result of step i-1 travel while
    # step i computes), and every timed step issues exactly one of each inside
    # the timed region; the last result is waited for before the clock stops.
    feeder = HostFeeder((M, K), dtype, dev)
    reader = ResultReader((M, N), dtype, dev)
    feeder.submit(x_host)

    def e2e_step():
        xd = feeder.take()
        feeder.submit(x_host)          # next step's input starts travelling now
        reader.before_step()           # the result buffer of two steps ago has been read out
        out = layer(xd)
        feeder.release(xd)
        reader.fetch(out)              # device -> pinned host on the copy stream, once the kernel is done

    for _ in range(warmup):
        e2e_step()
    reader.wait_all()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    reader.wait_all()                  # the last result has arrived on the host
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / steps
    if world > 1:
        dist.barrier()
    impl.check_status()
    e2e_value = flop / (e2e_ms * 1e-3) / 1e12
    # the parts, each alone (device time, this rank): input copy, kernel, result copy
    dst = torch.empty(M, K, dtype=dtype, device=dev)
    res = layer(x)
    host_out = torch.empty(M, N, dtype=dtype).pin_memory()
    h2d_ms = statistics.median(time_steps(lambda: dst.copy_(x_host, non_blocking=True), 5, 2, flush=False,
                                          barrier=False))
    d2h_ms = statistics.median(time_steps(lambda: host_out.copy_(res, non_blocking=True), 5, 2, flush=False,
                                          barrier=False))

    detail = {"per_step_ms": stats(times)}
    vs_baseline = None
    ok = True
    if not args.no_detail:
        from bench_detail import run_detail  # beside this file

        detail_more, vs_baseline, ok = run_detail(impl, layer, x, steps, warmup, args.algo, mx, stats)
        detail.update(detail_more)

    if rank == 0:
        line = {
            "metric": "fused GEMM+AllReduce+RMSNorm: aggregate TFLOP/s (value), latency (ms_per_step) and speed-up "
                      "over the non-overlapped cuBLAS+NCCL+RMSNorm path (vs_baseline)",
            "value": round(value, 2),
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": vs_baseline,
            "dtype": "fp16",
            "data": "synthetic (random-init weights and activations ~ N(0,1)/sqrt(K))",
            "config": {
                "model": "row-parallel attention out-projection, GEMM+AllReduce+RMSNorm",
                "M": M, "N": N, "K_total": K_total, "K_per_rank": K,
                "global_batch": M, "seq_len": M, "parallelism": f"tp{world}",
                "l2": "flushed between timed iterations (256 MB write)",
                "timing": "CUDA events per step, max over ranks",
                "algo": args.algo,
                "transport": "NVLS multimem" if impl.allreduce_uses_nvls() else "P2P stores",
                "vs_baseline_is": "nccl_baseline_ms / fused_ms, alternating steps (no published B200 number exists)",
            },
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "power_w_max": clocks["power_w_max"], "samples": clocks["samples"],
                       "samples_under_load": clocks["samples_under_load"]},
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 5),
                    "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": M * N * 2,
                    "breakdown_ms": {"h2d_alone": round(h2d_ms, 4), "kernel_alone": round(ms_per_step, 4),
                                     "d2h_alone": round(d2h_ms, 4)},
                    "api": "HostFeeder + FusedRowParallelLinear.forward + ResultReader",
                    "timing": "wall clock, max over ranks",
                    "note": "both copies are double-buffered: the input of step i+1 and the result of step i-1 "
                            "travel while step i computes; the whole [M, N] result is copied every step"},
            "gpu_launches": steps,
            "impl": "ours",
            "detail": detail,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
