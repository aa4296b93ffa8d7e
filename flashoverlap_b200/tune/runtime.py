"""GPU-side building blocks of the tuner and of the benchmark scripts: timing
loops in the reference's style (CUDA events, warm-up, mean, MAX over ranks;
reference: test/test.py:157-164,205-207), GEMM tile profiling, completion-order
sampling and the timed run of one fused configuration."""
from __future__ import annotations

import os
import sys
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..parallel import make_overlap_impl, max_over_ranks
from ..utils.config import ALGO_TILES
from ..utils.reorder import generate_row_mapping, reorder_indices
from ..utils.timing import flush_l2
from .model import div_up, gather_algo_candidates, hint_from_samples  # noqa: F401


def dbg(msg: str) -> None:
    """Debug line on stderr when FLASH_DEBUG is set (reference: tune/search.py:16-20)."""
    if os.getenv("FLASH_DEBUG"):
        print(f"[rank={os.getenv('LOCAL_RANK', '?')}] {msg}", flush=True, file=sys.stderr)


def world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def mean_time_ms(fn: Callable[[], None], warmup: int = 20, reps: int = 200, flush: bool = False,
                 return_local: bool = False):
    """Mean device time of ``fn`` in ms, maximum over the ranks (with
    ``return_local`` also this rank's own mean)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    for i in range(reps):
        if flush:
            flush_l2()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    local = sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / reps
    if return_local:
        return max_over_ranks(local), local
    return max_over_ranks(local)


def make_inputs(M: int, N: int, K: int, dtype=torch.float16, std: float = 0.5):
    A = torch.empty((M, K), dtype=dtype, device="cuda").normal_(mean=0.0, std=std)
    B = torch.empty((N, K), dtype=dtype, device="cuda").normal_(mean=0.0, std=std)
    C = torch.empty((M, N), dtype=dtype, device="cuda")
    return A, B, C


def usable_algos(M: int, N: int) -> List[int]:
    return [i for i, (bm, bn, _) in enumerate(ALGO_TILES) if M % bm == 0 and N % bn == 0]


RASTER_CHOICES = (1, 2, 4, 8)


def profile_gemm(impl, M: int, N: int, K: int, dtype=torch.float16, warmup: int = 10, reps: int = 100,
                 keep: int = 10, rasters: Sequence[int] = (), with_raster_table: bool = False):
    """Times every tile configuration that fits the shape and returns the
    ``keep`` fastest as stage-1 lists ``(BM, BN, dur, Algo)`` (reference:
    tune/profile_config.py:18-74).  With ``rasters`` every configuration is also
    timed for those raster groups (how many tile rows the kernel walks together:
    L2 reuse against how early rows complete); ``dur`` is then the best of them
    and, with ``with_raster_table``, a fifth value ``{raster: [ms per kept
    configuration]}`` is returned for the predictive search."""
    A, B, C = make_inputs(M, N, K, dtype)
    rows = []
    table = {}
    for algo in usable_algos(M, N):
        best = None
        for rg in (tuple(rasters) or (0,)):
            impl.set_raster_group(rg)
            try:
                ms = mean_time_ms(lambda: impl.cutlass_gemm(A, B, C, algo), warmup, reps)
            finally:
                impl.set_raster_group(0)
            table[(algo, rg)] = ms
            best = ms if best is None else min(best, ms)
            dbg(f"profile_gemm: algo {algo} {ALGO_TILES[algo]} raster {rg}: {ms:.4f} ms")
        rows.append((best, algo))
    if not rows:
        raise ValueError(f"no tile configuration divides M={M}, N={N}")
    rows.sort()
    rows = rows[:keep]
    out = ([ALGO_TILES[a][0] for _, a in rows], [ALGO_TILES[a][1] for _, a in rows], [ms for ms, _ in rows],
           [a for _, a in rows])
    if with_raster_table:
        return out + ({int(rg): [table[(a, rg)] for _, a in rows] for rg in rasters},)
    return out


def compute_hint(impl, M: int, N: int, K: int, BM: int, BN: int, algo: int, wave_size: int, comm_op: str,
                 dtype=torch.float16, warmup: int = 20, samples: int = 20, min_agree: int = 0
                 ) -> Tuple[bool, List[int]]:
    """Measured tile completion order -> tile-order hint (reference:
    tune/search.py:131-291).  Runs the fused operation in monitor mode with the
    identity order, collects the completion ticket of every tile ``samples``
    times and votes.  Collective; the result of rank 0 is used by all ranks."""
    rank, ws = world()
    tm, tn = div_up(M, BM), div_up(N, BN)
    tiles = tm * tn
    waves = div_up(tiles, wave_size)
    cseg = [min(wave_size, tiles - i * wave_size) for i in range(waves)]
    if tn <= len(cseg):
        # the monitor keeps its ticket counter in MM[N/BN - 1]: fold the groups
        cseg = [tiles]
    cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
    cseg_gpu = cseg_cpu.cuda()
    A, B, C = make_inputs(M, N, K, dtype)
    MM = torch.zeros((tm + 1, tn), dtype=torch.int32, device="cuda")
    RA = torch.arange(tiles, dtype=torch.int32, device="cuda").reshape(tm, tn)
    D = RE = None
    if comm_op == "reduce_scatter":
        D = torch.empty((M // ws, N), dtype=dtype, device="cuda")
        RE = generate_row_mapping(M, N, BM, BN, cseg, ws, device="cuda")

    def run(monitor: bool):
        if comm_op == "all_reduce":
            impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, monitor)
        else:
            impl.gemm_reducescatter_overlap(A, B, C, D, MM, RA, RE, 1, cseg_cpu, cseg_gpu, algo, monitor)

    ok, hint = False, []
    try:
        for _ in range(warmup):
            run(True)
        torch.cuda.synchronize()
        got = torch.empty((samples, tiles), dtype=torch.int32, device="cuda")
        for i in range(samples):
            MM[0] = 0
            run(True)
            got[i] = MM[1:].reshape(-1)
        torch.cuda.synchronize()
        impl.check_status()
        ok, hint = hint_from_samples(got.cpu(), wave_size, min_agree)
    except RuntimeError as exc:
        dbg(f"compute_hint: sampling failed: {exc}")
    if ws > 1:
        flag = torch.tensor([int(ok), len(hint)], dtype=torch.int64, device="cuda")
        dist.broadcast(flag, src=0)
        ok = bool(flag[0].item())
        if ok:
            h = torch.tensor(hint if rank == 0 else [0] * int(flag[1].item()), dtype=torch.int64, device="cuda")
            dist.broadcast(h, src=0)
            hint = h.cpu().tolist()
        dist.barrier()
    return ok, hint


def perf_running(impl, M: int, N: int, K: int, BM: int, BN: int, algo: int, cseg: Sequence[int],
                 hint: Sequence[int], comm_op: str, dtype=torch.float16, warmup: int = 20, reps: int = 200,
                 raster_group: int = 0, two_stream: bool = False, gemm_ctas: int = 0) -> float:
    """Mean time (ms, MAX over ranks) of the overlapped operation for one
    solution (reference: tune/search.py:357-459).  A single group means "no
    overlap": GEMM, then one collective.  ``two_stream=False`` runs this
    library's fused kernel through the reference-compatible entry point (the
    wave grouping does not change what that kernel does); ``two_stream=True``
    runs the reference's own design (signalling GEMM, stream waits, one NCCL
    call per wave group on a second stream), whose speed the grouping decides."""
    _, ws = world()
    tm, tn = div_up(M, BM), div_up(N, BN)
    tiles = tm * tn
    cseg_cpu = torch.tensor(list(cseg), dtype=torch.int32)
    cseg_gpu = cseg_cpu.cuda()
    A, B, C = make_inputs(M, N, K, dtype)
    MM = torch.zeros((max(tn, len(cseg)),), dtype=torch.int32, device="cuda")
    RA = reorder_indices(tiles, hint, device="cuda").reshape(tm, tn)
    D = torch.empty((M // ws, N), dtype=dtype, device="cuda") if comm_op == "reduce_scatter" else None
    RE = generate_row_mapping(M, N, BM, BN, list(cseg), ws, device="cuda") if comm_op == "reduce_scatter" else None
    impl.set_raster_group(raster_group)
    if len(cseg) == 1:
        if comm_op == "all_reduce":
            fn = lambda: impl.gemm_allreduce(A, B, C, algo)  # noqa: E731
        else:
            fn = lambda: impl.gemm_reducescatter(A, B, C, D, algo)  # noqa: E731
    elif two_stream and comm_op == "all_reduce":
        fn = lambda: impl.gemm_allreduce_twostream(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, gemm_ctas)  # noqa: E731
    elif two_stream:
        fn = lambda: impl.gemm_reducescatter_twostream(A, B, C, D, MM, RA, RE, 1, cseg_cpu, cseg_gpu, algo,  # noqa: E731
                                                       gemm_ctas)
    elif comm_op == "all_reduce":
        fn = lambda: impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, False)  # noqa: E731
    else:
        fn = lambda: impl.gemm_reducescatter_overlap(A, B, C, D, MM, RA, RE, 1, cseg_cpu, cseg_gpu, algo,  # noqa: E731
                                                     False)
    try:
        ms = mean_time_ms(fn, warmup, reps)
        impl.check_status()
    finally:
        impl.set_raster_group(0)
    return ms


def wave_units(tiles: int, wave: int, max_units: int = 10) -> Tuple[int, int]:
    """(units, tiles per unit): the wave count folded to at most ``max_units``
    units, as the reference normalises it (reference: tune/search.py:545-548,564)."""
    waves = div_up(tiles, wave)
    per_unit = div_up(waves, max_units)
    return div_up(waves, per_unit), per_unit * wave


def search_two_stream(impl, M: int, N: int, K: int, algo: int, comm_op: str, dtype=torch.float16,
                      curve: Optional[torch.Tensor] = None, gemm_ms: Optional[float] = None, max_units: int = 10,
                      top_k: int = 0, warmup: int = 5, reps: int = 20, gemm_ctas: int = 0,
                      hint: Sequence[int] = ()) -> Tuple[List[int], float, List[Tuple[List[int], float]]]:
    """Searches the wave grouping ``cSeg`` of the reference's two-stream overlap
    design by TIMING candidates (reference: tune/search.py:473-526 exhaustive,
    :529-596 predictive).  Collective.

    Every composition of the (folded) wave count is a candidate, minus the
    reference's "cold start" rule (more than five groups with a first group
    above two units).  Without a bandwidth ``curve`` all candidates are timed;
    with one (and the GEMM time ``gemm_ms``) they are ranked by the pipeline
    model and only the ``top_k`` best (default 3) are timed.  Returns
    ``(best cSeg, its time in ms, [(cSeg, ms) for every timed candidate])``."""
    from .model import compositions, predict_segmented_ms, scale_groups

    rank, ws = world()
    BM, BN, _ = ALGO_TILES[algo]
    tiles = div_up(M, BM) * div_up(N, BN)
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    ctas_per_tile = BM // 128
    gemm_sms = gemm_ctas if gemm_ctas > 0 else sms - 16
    wave = max(1, gemm_sms // ctas_per_tile)
    units, unit_tiles = wave_units(tiles, wave, max_units)
    cands: List[List[int]] = []
    for parts in compositions(units):
        if len(parts) > 5 and parts[0] > 2:
            continue
        try:
            g = scale_groups(parts, unit_tiles, tiles)
        except ValueError:
            continue
        if comm_op == "reduce_scatter" and any((x * BM) % ws for x in g):
            continue
        if g not in cands:
            cands.append(g)
    if [tiles] not in cands:
        cands.append([tiles])
    if curve is not None and gemm_ms is not None:
        scored = sorted(cands, key=lambda g: predict_segmented_ms(M, N, gemm_ms, curve, g, tiles, comm_op, ws, sms,
                                                                  sms - gemm_sms))
        cands = scored[:top_k if top_k > 0 else 3]
    elif top_k > 0:
        cands = cands[:top_k]
    timed: List[Tuple[List[int], float]] = []
    for g in cands:
        ms = perf_running(impl, M, N, K, BM, BN, algo, g, hint, comm_op, dtype, warmup=warmup, reps=reps,
                          two_stream=True, gemm_ctas=gemm_ctas)
        dbg(f"search_two_stream: cSeg {g} -> {ms:.4f} ms")
        timed.append((g, ms))
    best = min(timed, key=lambda t: t[1])
    return best[0], best[1], timed


def pick_algo_by_timing(run: Callable[[int], None], algos: Sequence[int], warmup: int = 2, reps: int = 5):
    """Times ``run(algo)`` for every candidate (L2 flushed, slowest rank) and
    returns ``(best algo, [(algo, ms), ...])``: the stage-1 search of the
    tuner for operations whose best tile depends on the ranks' arrival pattern
    (reference: tune/profile_config.py times every instance and keeps the
    fastest)."""
    timed = []
    for a in algos:
        timed.append((a, mean_time_ms(lambda: run(a), warmup, reps, flush=True)))
    best = min(timed, key=lambda t: t[1])[0]
    return best, timed


def measure_row_us(impl, N: int, comm_op: str, dtype=torch.float16, algo: int = 0, M: int = 4096, K: int = 64,
                   warmup: int = 3, reps: int = 10, sms: int = 148, groups: int = 3) -> float:
    """Time one row group needs for one row of ``N`` values in the reduce phase
    of ``comm_op`` on this machine, in us: a GEMM with a negligible K leaves the
    fused kernel's time to its reduce phase, in which every SM runs ``groups``
    row groups: (fused - GEMM alone) * groups * SMs / rows per rank.  It is the
    one number the fused cost model needs besides the GEMM time and the link
    bandwidth (memory, link and latency cost of a row, measured rather than
    assumed)."""
    _, ws = world()
    while M % ws or (M // ws) % 128:
        M *= 2
    A, B, C = make_inputs(M, N, K, dtype)
    W = torch.ones(N, device="cuda", dtype=dtype)
    D = torch.empty(M // ws, N, device="cuda", dtype=dtype)
    if comm_op == "all_reduce":
        fused = lambda: impl.gemm_allreduce_fused(A, B, W, 1e-5, algo)  # noqa: E731
    else:
        fused = lambda: impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, algo, False)  # noqa: E731
    t_fused = mean_time_ms(fused, warmup, reps, flush=True)
    t_gemm = mean_time_ms(lambda: impl.cutlass_gemm(A, B, C, algo), warmup, reps, flush=True)
    rows = M // ws
    return max((t_fused - t_gemm) * 1e3, 1.0) * groups * sms / rows
