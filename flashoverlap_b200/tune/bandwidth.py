"""Bandwidth curves: time of a collective against message size, stored as
``[elements, bus bandwidth GB/s]`` (reference: tune/bandwidth.py:56-158; 36 sizes
2**(20 + i/4) 16-bit elements, 20 warm-ups, 200 repetitions).  Besides the NCCL
collectives the reference measures, this tool can time the library's own
transports: peer-to-peer stores (``p2p_push``, ``p2p_push_bulk``) and the NVLink
SHARP primitives (``multimem_ld_reduce``, ``multimem_st``, ``multimem_allreduce``)."""
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


NCCL_OPS = ("all_reduce", "reduce_scatter")
# the library's own transports: peer-to-peer stores from registers, bulk stores out of shared memory, and the
# NVLink SHARP primitives (switch-side reduction, multicast store, both = an all-reduce of every rank's share)
OWN_OPS = ("p2p_push", "p2p_push_bulk", "multimem_ld_reduce", "multimem_st", "multimem_allreduce")
COMM_OPS = NCCL_OPS + OWN_OPS


def link_bytes_per_direction(comm_op: str, nbytes: float, ws: int) -> float:
    """Bytes that cross one GPU's NVLink in the busier direction when the
    primitive moves a message of ``nbytes`` (what the own-transport curves
    divide by the time)."""
    if ws <= 1:
        return 0.0
    if comm_op in ("p2p_push", "p2p_push_bulk"):
        return nbytes                     # everything the GPU sends to its peers
    if comm_op == "multimem_ld_reduce":
        return nbytes                     # the switch pulls every GPU's copy of every share
    if comm_op == "multimem_st":
        return nbytes                     # every GPU receives all shares
    if comm_op == "multimem_allreduce":
        return nbytes * (1.0 + 1.0 / ws)  # pull all partials once, receive all results once
    raise ValueError(comm_op)


def measure_curve(impl, comm_op: str, dtype=torch.float16, points: int = 36, warmup: int = 20, reps: int = 200,
                  max_elements: Optional[int] = None, chunk_bytes: int = 8192, ctas: int = 0,
                  gather_ranks: bool = False):
    """Collective.  ``[elements, GB/s]`` per message size.

    ``comm_op``: all_reduce | reduce_scatter (NCCL through ``impl``, bus
    bandwidth as the reference defines it) or one of ``OWN_OPS`` (this
    library's kernels; 'elements' is the message: what one GPU sends in total
    for the push kernels, the whole symmetric buffer for the multimem
    primitives; GB/s is bytes per NVLink direction per GPU over the time).
    With ``gather_ranks`` the per-rank times of every size are returned as
    well (second value, ``[sizes, ranks]`` in ms), the way the reference's
    multi-node tool gathers them (reference: tune/bandwidth_multinode.py:100-101)."""
    rank, ws = world()
    rows, per_rank = [], []
    sizes = curve_sizes(points, max_elements)
    buf = torch.empty(max(sizes), dtype=dtype, device="cuda").normal_(0.0, 0.5) if comm_op in NCCL_OPS else None
    esz = torch.empty(0, dtype=dtype).element_size()
    for n in sizes:
        n = n // (16 * max(ws, 1)) * (16 * max(ws, 1))
        if comm_op == "all_reduce":
            view = buf[:n]
            fn = lambda: impl.nccl_allreduce(view)  # noqa: E731
        elif comm_op == "reduce_scatter":
            view = buf[:n]
            fn = lambda: impl.nccl_reducescatter(view)  # noqa: E731
        elif comm_op in ("p2p_push", "p2p_push_bulk"):
            per_peer = n * esz // max(ws - 1, 1) // 16 * 16
            if comm_op == "p2p_push":
                fn = lambda: impl.p2p_push(per_peer, ctas)  # noqa: E731
            else:
                fn = lambda: impl.p2p_push_bulk(per_peer, chunk_bytes, ctas)  # noqa: E731
        elif comm_op in OWN_OPS:
            kind = comm_op[len("multimem_"):]
            nbytes = n * esz
            fn = lambda: impl.multimem_bench(kind, nbytes, ctas, dtype == torch.bfloat16)  # noqa: E731
        else:
            raise ValueError(f"unknown comm_op {comm_op!r}")
        ms, local_ms = mean_time_ms(fn, warmup, reps, return_local=True)
        if comm_op in NCCL_OPS:
            bw = bus_bandwidth_gbs(n, ms * 1e-3, ws, comm_op, esz)
        else:
            moved = per_peer * (ws - 1) if comm_op.startswith("p2p") else link_bytes_per_direction(comm_op, n * esz, ws)
            bw = moved / (ms * 1e-3) / 1e9 if ws > 1 else 0.0
        dbg(f"bandwidth {comm_op}: {n} elements {ms:.4f} ms {bw:.1f} GB/s")
        rows.append([float(n), float(bw)])
        if gather_ranks and dist.is_initialized():
            t = torch.tensor([local_ms], dtype=torch.float64, device="cuda")
            allt = [torch.zeros_like(t) for _ in range(ws)]
            dist.all_gather(allt, t)
            per_rank.append([float(v.item()) for v in allt])
        if dist.is_initialized():
            dist.barrier()
    curve = torch.tensor(rows, dtype=torch.float32)
    if gather_ranks:
        return curve, torch.tensor(per_rank, dtype=torch.float64)
    return curve


def curve_table(curve: torch.Tensor, comm_op: str, ws: int, elem_bytes: int = 2) -> str:
    """The curve as a text table (message size in MiB, GB/s)."""
    unit = "bus GB/s (GiB-based)" if comm_op in NCCL_OPS else "GB/s per NVLink direction per GPU"
    lines = [f"# {comm_op}, {ws} ranks: message MiB, {unit}"]
    for n, bw in curve.tolist():
        lines.append(f"{n * elem_bytes / 2 ** 20:10.2f} {bw:9.1f}")
    return "\n".join(lines) + "\n"


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
