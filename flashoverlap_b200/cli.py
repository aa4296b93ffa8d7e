"""Start-up shared by the command-line tools under ``tune/``, ``test/``,
``example/`` and ``tool/``: dtype names, one process per GPU, and the measured
machine numbers (peak GEMM rate, link bandwidth) that the tools report
fractions of.  Nothing about a particular machine is typed into the tools:
the peaks come from a measurement file, the link bandwidth from the curve
files ``tune/bandwidth.py`` writes."""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Optional, Tuple

import torch

from .parallel import init_distributed, make_baseline_impl, make_overlap_impl  # noqa: F401  (re-exported)
from .utils import config as cfg

DTYPES = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def start(retries: int = 0, retry_wait_s: float = 5.0) -> Tuple[int, int]:
    """(rank, world_size) after process-group and device set-up.  With
    ``retries`` the rendezvous is tried again after a failure (nodes of a
    multi-node job rarely start in the same second; reference:
    tune/bandwidth_multinode.py:27-39)."""
    attempt = 0
    while True:
        try:
            rank, world, _ = init_distributed()
            return rank, world
        except RuntimeError:
            attempt += 1
            if attempt > retries:
                raise
            time.sleep(retry_wait_s)


def finish() -> None:
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def measured_peaks(path: Optional[os.PathLike] = None) -> dict:
    """Measured peaks of this machine: ``{"bf16_tflops", "bf16_tflops_sustained",
    "hbm_gbs"}`` from the JSON file named by ``path`` / ``$FLASHOVERLAP_PEAKS`` /
    ``MEASURED_PEAKS.json`` at the repository root.  Empty when no such file
    exists (callers then print times without roofline fractions)."""
    cand = [path, os.environ.get("FLASHOVERLAP_PEAKS"), cfg.REPO_ROOT / "MEASURED_PEAKS.json"]
    for c in cand:
        if c and Path(c).exists():
            try:
                return json.loads(Path(c).read_text())
            except (OSError, ValueError):
                continue
    return {}


def measured_link_gbs(world_size: int, multinode: bool = False, path=None) -> Tuple[Optional[float], str]:
    """Best measured one-direction bandwidth out of one GPU (GB/s) among the
    transport curves in the config directory, and the curve it came from."""
    best, name = None, ""
    for op in ("p2p_push", "p2p_push_bulk", "multimem_allreduce", "multimem_ld_reduce", "multimem_st"):
        try:
            c = cfg.load_bandwidth(op, world_size, multinode, path)
        except FileNotFoundError:
            continue
        v = float(c[:, 1].max())
        if best is None or v > best:
            best, name = v, op
    return best, name
