"""Wave-group search (reference: tune/search.py:473-618).

The reference's tuned quantities are the GEMM tile configuration, the
tile-order hint and the wave grouping ``cSeg`` of its segmented collectives.
This library's fused kernel signals per tile row instead of per wave group, so
what decides its speed is the tile configuration and two kernel knobs (raster
group, warps per row of the reduce phase).  The search therefore

1. picks the tile-order hint from measured completion order (as the reference),
2. derives ``cSeg`` with the reference's pipeline model on the measured
   bandwidth curve (kept in the file for readers of that format), and
3. chooses (Algo, raster_group, reduce_group) either by timing every candidate
   (exhaustive) or by ranking candidates with the fused-kernel cost model and
   timing only the best few (predictive).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..utils import config as cfg
from .model import best_segmentation, compositions, div_up, predict_fused_ms, scale_groups
from .runtime import compute_hint, dbg, perf_running, world

RASTER_CHOICES = (1, 2, 4, 8)
REDUCE_CHOICES = (0, 1, 2, 4, 8)


def sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def find_hint(impl, M, N, K, BM_list, BN_list, Algo_list, comm_op, dtype, wave_units: int = 1, tries: int = 5):
    """First stage-1 candidate whose completion order is consistent."""
    sms = sm_count()
    for t in range(min(tries, len(BM_list))):
        BM, BN, algo = BM_list[t], BN_list[t], Algo_list[t]
        ctas = BM // 128
        wave = max(1, sms // ctas) * wave_units
        ok, hint = compute_hint(impl, M, N, K, BM, BN, algo, wave, comm_op, dtype)
        dbg(f"find_hint: candidate {t} ({BM}x{BN}, Algo {algo}) consistent={ok}")
        if ok:
            return t, hint
    raise RuntimeError("tuning failed: no tile configuration gave a consistent completion order")


def knob_candidates(M: int, world_size: int) -> List[Tuple[int, int]]:
    rows = M // max(world_size, 1)
    out = []
    for rg in RASTER_CHOICES:
        for g in REDUCE_CHOICES:
            if g and 148 * (8 // g) * 4 < rows and g > 1:
                continue  # far too few rows in flight
            out.append((rg, g))
    return out


def exhaustive_search(impl, M: int, N: int, K: int, comm_op: str, dtype=torch.float16, path=None,
                      reps: int = 50, verbose: bool = True) -> dict:
    """Times every (tile configuration, raster group, reduce group) candidate."""
    rank, ws = world()
    data = cfg.load_config(M, N, K, path)
    BM_l, BN_l, dur_l, Algo_l = cfg.stage1_lists(data)
    best = None
    hints = {}
    for t in range(min(5, len(BM_l))):
        BM, BN, algo = BM_l[t], BN_l[t], Algo_l[t]
        tiles = div_up(M, BM) * div_up(N, BN)
        for rg, g in knob_candidates(M, ws):
            ms = perf_running(impl, M, N, K, BM, BN, algo, [tiles - 1, 1] if tiles > 1 else [1], [], comm_op, dtype,
                              warmup=10, reps=reps, raster_group=rg, reduce_group=g)
            if rank == 0 and verbose:
                print(f"Algo {algo} ({BM}x{BN}) raster {rg} reduce {g}: {ms:.4f} ms")
            if best is None or ms < best[0]:
                best = (ms, t, rg, g)
    ms, t, rg, g = best
    _, hint = find_hint(impl, M, N, K, BM_l[t:t + 1], BN_l[t:t + 1], Algo_l[t:t + 1], comm_op, dtype)
    tiles = div_up(M, BM_l[t]) * div_up(N, BN_l[t])
    wave = max(1, sm_count() // (BM_l[t] // 128))
    cseg = scale_groups([1] * div_up(tiles, wave), wave, tiles)
    sol = dict(BM=BM_l[t], BN=BN_l[t], dur=dur_l[t], Algo=Algo_l[t], hint=hint, cSeg=cseg, raster_group=rg,
               reduce_group=g, fused_dur=ms, comm_op=comm_op, world_size=ws, search="exhaustive")
    if rank == 0:
        cfg.save_stage2(M, N, K, path=path, **sol)
        if verbose:
            print(f"Best solution: Algo {sol['Algo']} raster {rg} reduce {g}, {ms:.4f} ms; solution saved.")
    return sol


def predictive_search(impl, M: int, N: int, K: int, comm_op: str, curve: torch.Tensor,
                      p2p_gbs: Optional[float] = None, dtype=torch.float16, path=None, top_k: int = 3,
                      reps: int = 50, verbose: bool = True) -> dict:
    """Ranks candidates with the cost models, times only the ``top_k`` best."""
    rank, ws = world()
    data = cfg.load_config(M, N, K, path)
    BM_l, BN_l, dur_l, Algo_l = cfg.stage1_lists(data)
    if p2p_gbs is None:
        p2p_gbs = 550.0  # store bandwidth out of one B200 through NVSwitch, measured with p2p_push
    ranked = []
    for t in range(min(10, len(BM_l))):
        for rg, g in knob_candidates(M, ws):
            geff = g or max(1, min(8, 8 // max(1, div_up(M // max(ws, 1), 148))))
            est = predict_fused_ms(M, N, dur_l[t], ws, comm_op, p2p_gbs, reduce_group=geff)
            est *= 1.0 + 0.01 * abs(rg - 2)  # mild preference for the default raster
            ranked.append((est, t, rg, g))
    ranked.sort()
    best = None
    for est, t, rg, g in ranked[:top_k]:
        tiles = div_up(M, BM_l[t]) * div_up(N, BN_l[t])
        ms = perf_running(impl, M, N, K, BM_l[t], BN_l[t], Algo_l[t], [tiles - 1, 1] if tiles > 1 else [1], [],
                          comm_op, dtype, warmup=10, reps=reps, raster_group=rg, reduce_group=g)
        if rank == 0 and verbose:
            print(f"Algo {Algo_l[t]} raster {rg} reduce {g}: predicted {est:.4f} ms, measured {ms:.4f} ms")
        if best is None or ms < best[0]:
            best = (ms, t, rg, g, est)
    ms, t, rg, g, est = best
    _, hint = find_hint(impl, M, N, K, BM_l[t:t + 1], BN_l[t:t + 1], Algo_l[t:t + 1], comm_op, dtype)
    tiles = div_up(M, BM_l[t]) * div_up(N, BN_l[t])
    cseg, seg_ms = best_segmentation(M, N, dur_l[t], curve, tiles, comm_op, ws, sm_count() // (BM_l[t] // 128), 0)
    sol = dict(BM=BM_l[t], BN=BN_l[t], dur=dur_l[t], Algo=Algo_l[t], hint=hint, cSeg=cseg, raster_group=rg,
               reduce_group=g, fused_dur=ms, predicted_dur=est, segmented_model_dur=seg_ms, comm_op=comm_op,
               world_size=ws, search="predictive")
    if rank == 0:
        cfg.save_stage2(M, N, K, path=path, **sol)
        if verbose:
            print(f"Searched latency: {ms:.4f} ms\nBest solution: {cseg}\nSolution saved.")
    return sol


PREDICTIVE_THRESHOLD = 33554432  # M*N above which the reference switches to the predictive search
