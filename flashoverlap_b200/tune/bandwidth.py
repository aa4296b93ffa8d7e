"""Bandwidth curves: time of a collective against message size, stored as
``[elements, bus bandwidth GB/s]`` (reference: tune/bandwidth.py:56-158; 36 sizes
2**(20 + i/4) 16-bit elements, 20 warm-ups, 200 repetitions).  Besides the NCCL
collectives the reference measures, this tool can time the library's own
peer-to-peer store kernel (``p2p_push``), the transport of the fused kernels."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .model import bus_bandwidth_gbs
from .runtime import dbg, mean_time_ms, world


def curve_sizes(points: int = 36, max_elements: Optional[int] = None) -> List[int]:
    sizes = [int(2 ** (20 + 0.25 * i)) // 1024 * 1024 for i in range(points)]
    if max_elements is not None:
        sizes = [s for s in sizes if s <= max_elements]
    return sizes


def measure_curve(impl, comm_op: str, dtype=torch.float16, points: int = 36, warmup: int = 20, reps: int = 200,
                  max_elements: Optional[int] = None) -> torch.Tensor:
    """Collective.  ``comm_op``: all_reduce | reduce_scatter (NCCL through
    ``impl``) or p2p_push (own kernel; 'elements' is then the total each GPU
    sends, split evenly over its peers)."""
    rank, ws = world()
    rows = []
    sizes = curve_sizes(points, max_elements)
    buf = torch.empty(max(sizes), dtype=dtype, device="cuda").normal_(0.0, 0.5) if comm_op != "p2p_push" else None
    for n in sizes:
        n = n // (16 * max(ws, 1)) * (16 * max(ws, 1))
        if comm_op == "all_reduce":
            view = buf[:n]
            ms = mean_time_ms(lambda: impl.nccl_allreduce(view), warmup, reps)
        elif comm_op == "reduce_scatter":
            view = buf[:n]
            ms = mean_time_ms(lambda: impl.nccl_reducescatter(view), warmup, reps)
        elif comm_op == "p2p_push":
            per_peer = n * 2 // max(ws - 1, 1) // 16 * 16
            ms = mean_time_ms(lambda: impl.p2p_push(per_peer, 0), warmup, reps)
        else:
            raise ValueError(f"unknown comm_op {comm_op!r}")
        if comm_op == "p2p_push":
            bw = n * 2 / (ms * 1e-3) / 1024 ** 3 if ws > 1 else 0.0
        else:
            bw = bus_bandwidth_gbs(n, ms * 1e-3, ws, comm_op)
        dbg(f"bandwidth {comm_op}: {n} elements {ms:.4f} ms {bw:.1f} GB/s")
        rows.append([float(n), float(bw)])
        if dist.is_initialized():
            dist.barrier()
    return torch.tensor(rows, dtype=torch.float32)


def plot_curve(curve: torch.Tensor, title: str, path: str) -> bool:
    """PNG of the curve when matplotlib is available (the reference always plots)."""
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return False
    fig = plt.figure(figsize=(6, 4))
    plt.semilogx(curve[:, 0].numpy() * 2 / 2 ** 20, curve[:, 1].numpy(), marker="o")
    plt.xlabel("message size (MiB)")
    plt.ylabel("bus bandwidth (GB/s)")
    plt.title(title)
    plt.grid(True, which="both", alpha=0.3)
    fig.savefig(path, dpi=120, bbox_inches="tight")
    plt.close(fig)
    return True
