"""Device-side timing the way every benchmark of this repository does it:
CUDA events on the launching stream, warm-up first, an L2 flush between timed
iterations, the maximum over ranks for multi-GPU numbers (reference:
test/test.py:157-164,205-207 times with events and reduces with MAX)."""
from __future__ import annotations

from typing import Callable, Optional

import torch

_flush_buf: Optional[torch.Tensor] = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so that the next kernel
    starts from DRAM."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.numel() < nbytes:
        _flush_buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_steps(fn: Callable[[], None], steps: int, warmup: int, flush: bool = True, group=None,
               barrier: bool = True) -> list[float]:
    """Per-step device times in milliseconds (this rank).  Every step is
    bracketed by its own pair of events so that the flush is not timed."""
    import torch.distributed as dist

    for _ in range(warmup):
        if flush:
            flush_l2()
        fn()
    torch.cuda.synchronize()
    if barrier and dist.is_available() and dist.is_initialized():
        dist.barrier(group)
        torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if flush:
            flush_l2()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    if barrier and dist.is_available() and dist.is_initialized():
        dist.barrier(group)
        torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def time_pairs(fn_a: Callable[[], None], fn_b: Callable[[], None], steps: int, warmup: int, flush: bool = True,
               group=None) -> tuple[list[float], list[float]]:
    """Per-step device times of two alternatives measured in alternation
    (a, b, a, b, ...) so that clock and power drift hit both alike."""
    import torch.distributed as dist

    for _ in range(warmup):
        for fn in (fn_a, fn_b):
            if flush:
                flush_l2()
            fn()
    torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group)
        torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    for i in range(steps):
        for j, fn in enumerate((fn_a, fn_b)):
            if flush:
                flush_l2()
            ev[i][2 * j].record()
            fn()
            ev[i][2 * j + 1].record()
    torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group)
        torch.cuda.synchronize()
    return ([e[0].elapsed_time(e[1]) for e in ev], [e[2].elapsed_time(e[3]) for e in ev])
