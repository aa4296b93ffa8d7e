"""Wave-group search (reference: tune/search.py:473-618).

The reference tunes three things: the GEMM tile configuration, the tile-order
hint and the wave grouping ``cSeg`` of its segmented collectives, the last by
timing every composition of the wave count (exhaustive) or by predicting with
a pipeline model on a measured bandwidth curve and timing the pick
(predictive).  Both drivers exist here and do the same, for two consumers:

* the reference's own two-stream design (``gemm_*_twostream``) and the
  reference-compatible file format: ``cSeg`` is searched by TIMING compositions
  on that path, exactly the reference's procedure;
* this library's fused kernel, which signals per tile row instead of per wave
  group: what decides its speed is the tile configuration, the raster group
  (how many tile rows are walked together, i.e. how early rows complete: the
  fused kernel's "wave group") and the transport.  Candidates
  ``(Algo, raster_group)`` are timed (exhaustive) or ranked by a cost model
  on measured link bandwidth and then timed (predictive).

Every number a model uses comes from a measured curve file; nothing about the
machine is typed in here.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..utils import config as cfg
from .model import best_segmentation, div_up, predict_fused_ms
from .runtime import compute_hint, dbg, measure_row_us, perf_running, search_two_stream, world

RASTER_CHOICES = (1, 2, 4, 8)


def sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


# Sampling rule of the tile-order hint: (samples, minimum agreement).  The
# single-node search votes over 20 samples; the multi-node search of the
# reference takes 10 and wants a tile in the same wave in 9 of them.
HINT_RULE = {"samples": 20, "min_agree": 0}


def find_hint(impl, M, N, K, BM_list, BN_list, Algo_list, comm_op, dtype, wave_units: int = 1, tries: int = 5):
    """First stage-1 candidate whose completion order is consistent."""
    sms = sm_count()
    for t in range(min(tries, len(BM_list))):
        BM, BN, algo = BM_list[t], BN_list[t], Algo_list[t]
        ctas = BM // 128
        wave = max(1, sms // ctas) * wave_units
        ok, hint = compute_hint(impl, M, N, K, BM, BN, algo, wave, comm_op, dtype, samples=HINT_RULE["samples"],
                                min_agree=HINT_RULE["min_agree"])
        dbg(f"find_hint: candidate {t} ({BM}x{BN}, Algo {algo}) consistent={ok}")
        if ok:
            return t, hint
    raise RuntimeError("tuning failed: no tile configuration gave a consistent completion order")


def knob_candidates(M: int, BM: int) -> List[int]:
    """Raster groups worth trying for a matrix of M rows and tiles of BM rows."""
    tm = max(1, M // BM)
    out = [rg for rg in RASTER_CHOICES if rg <= tm]
    return out or [1]


def _fused_time(impl, M, N, K, BM, BN, algo, comm_op, dtype, rg, reps):
    tiles = div_up(M, BM) * div_up(N, BN)
    return perf_running(impl, M, N, K, BM, BN, algo, [tiles - 1, 1] if tiles > 1 else [1], [], comm_op, dtype,
                        warmup=10, reps=reps, raster_group=rg)


def exhaustive_search(impl, M: int, N: int, K: int, comm_op: str, dtype=torch.float16, path=None,
                      reps: int = 50, verbose: bool = True, max_units: int = 10, seg_reps: int = 20) -> dict:
    """Times every fused candidate (tile configuration x raster group) and every
    composition of the wave count on the two-stream path."""
    rank, ws = world()
    data = cfg.load_config(M, N, K, path)
    BM_l, BN_l, dur_l, Algo_l = cfg.stage1_lists(data)
    best = None
    for t in range(min(5, len(BM_l))):
        BM, BN, algo = BM_l[t], BN_l[t], Algo_l[t]
        for rg in knob_candidates(M, BM):
            ms = _fused_time(impl, M, N, K, BM, BN, algo, comm_op, dtype, rg, reps)
            if rank == 0 and verbose:
                print(f"Algo {algo} ({BM}x{BN}) raster {rg}: {ms:.4f} ms")
            if best is None or ms < best[0]:
                best = (ms, t, rg)
    ms, t, rg = best
    _, hint = find_hint(impl, M, N, K, BM_l[t:t + 1], BN_l[t:t + 1], Algo_l[t:t + 1], comm_op, dtype)
    # the reference's composition loop: every candidate grouping is timed
    cseg, seg_ms, timed = search_two_stream(impl, M, N, K, Algo_l[t], comm_op, dtype, max_units=max_units,
                                            reps=seg_reps, hint=hint)
    if rank == 0 and verbose:
        for g, tms in timed:
            print(f"cSeg {g}: two-stream {tms:.4f} ms")
    sol = dict(BM=BM_l[t], BN=BN_l[t], dur=dur_l[t], Algo=Algo_l[t], hint=hint, cSeg=cseg, raster_group=rg,
               fused_dur=ms, two_stream_dur=seg_ms, candidates_timed=len(timed), comm_op=comm_op, world_size=ws,
               search="exhaustive")
    if rank == 0:
        cfg.save_stage2(M, N, K, path=path, **sol)
        if verbose:
            print(f"Best solution: Algo {sol['Algo']} raster {rg}, fused {ms:.4f} ms; cSeg {cseg}, two-stream "
                  f"{seg_ms:.4f} ms; solution saved.")
    return sol


def link_bandwidth_from_curves(world_size: int, multinode: bool = False, path=None,
                               nvls: bool = False) -> Tuple[Optional[float], str]:
    """Peak of the measured curve of the transport the fused kernel uses, in
    GB/s, and the name of the file it came from: peer-to-peer stores, or with
    ``nvls`` (the engine's all-reduce is set to NVLink SHARP) the ``multimem``
    all-reduce primitive if that curve was measured."""
    order = ("multimem_allreduce", "p2p_push", "p2p_push_bulk") if nvls else ("p2p_push", "p2p_push_bulk")
    for op in order:
        try:
            c = cfg.load_bandwidth(op, world_size, multinode, path)
        except FileNotFoundError:
            continue
        return float(c[:, 1].max()), op
    return None, ""


def predictive_search(impl, M: int, N: int, K: int, comm_op: str, curve: torch.Tensor,
                      link_gbs: Optional[float] = None, dtype=torch.float16, path=None, top_k: int = 3,
                      reps: int = 50, verbose: bool = True, link_kind: str = "p2p", seg_reps: int = 20,
                      row_us: Optional[float] = None) -> dict:
    """Ranks candidates with the cost models on measured bandwidth, then times
    only the best few.  ``curve`` is the measured NCCL curve of ``comm_op``
    (for the two-stream grouping), ``link_gbs`` the measured bandwidth of the
    fused kernel's transport (``link_kind``: "p2p" or "nvls"), ``row_us`` the
    measured time of one row in the reduce phase (measured here if not given)."""
    rank, ws = world()
    if link_gbs is None:
        if ws > 1:
            raise ValueError("predictive_search needs the measured link bandwidth (run tune/bandwidth.py --comm_op "
                             "p2p_push or multimem_allreduce first)")
        link_gbs = 1.0  # unused with one rank
    data = cfg.load_config(M, N, K, path)
    BM_l, BN_l, dur_l, Algo_l = cfg.stage1_lists(data)
    by_raster = cfg.stage1_raster_table(data)  # GEMM time per (configuration, raster group), if profiled
    if row_us is None:
        row_us = measure_row_us(impl, N, comm_op, dtype, algo=Algo_l[0])  # what one row costs a row group here
    if rank == 0 and verbose:
        print(f"Measured row time of the reduce phase: {row_us:.2f} us per row group.")
    ranked = []
    for t in range(min(10, len(BM_l))):
        for rg in knob_candidates(M, BM_l[t]):
            gemm_ms = by_raster[rg][t] if rg in by_raster else dur_l[t]
            est = predict_fused_ms(M, N, gemm_ms, ws, comm_op, link_gbs, transport=link_kind, tile_m=BM_l[t],
                                   raster_group=rg, row_us=row_us, sm_count=sm_count())
            ranked.append((est, t, rg))
    ranked.sort()
    best = None
    for est, t, rg in ranked[:top_k]:
        ms = _fused_time(impl, M, N, K, BM_l[t], BN_l[t], Algo_l[t], comm_op, dtype, rg, reps)
        if rank == 0 and verbose:
            print(f"Algo {Algo_l[t]} raster {rg}: predicted {est:.4f} ms, measured {ms:.4f} ms")
        if best is None or ms < best[0]:
            best = (ms, t, rg, est)
    ms, t, rg, est = best
    _, hint = find_hint(impl, M, N, K, BM_l[t:t + 1], BN_l[t:t + 1], Algo_l[t:t + 1], comm_op, dtype)
    # grouping: predicted on the measured curve, then the pick is timed (reference: tune/search.py:529-596)
    cseg, seg_ms, timed = search_two_stream(impl, M, N, K, Algo_l[t], comm_op, dtype, curve=curve, gemm_ms=dur_l[t],
                                            top_k=1, reps=seg_reps, hint=hint)
    tiles = div_up(M, BM_l[t]) * div_up(N, BN_l[t])
    _, seg_pred = best_segmentation(M, N, dur_l[t], curve, tiles, comm_op, ws, sm_count() // (BM_l[t] // 128), 16)
    sol = dict(BM=BM_l[t], BN=BN_l[t], dur=dur_l[t], Algo=Algo_l[t], hint=hint, cSeg=cseg, raster_group=rg,
               fused_dur=ms, predicted_dur=est, two_stream_dur=seg_ms, segmented_model_dur=seg_pred,
               candidates_timed=len(timed), comm_op=comm_op, world_size=ws, search="predictive")
    if rank == 0:
        cfg.save_stage2(M, N, K, path=path, **sol)
        if verbose:
            print(f"Searched latency: {ms:.4f} ms\nBest solution: {cseg}\nSolution saved.")
    return sol


PREDICTIVE_THRESHOLD = 33554432  # M*N above which the reference switches to the predictive search
