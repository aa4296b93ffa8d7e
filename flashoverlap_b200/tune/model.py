"""Analytical pieces of the tuner, free of any GPU call so that they can be
unit-tested: compositions of the wave count, bus-bandwidth formulas, the
latency interpolation on a measured curve, the reference's pipeline model of
segmented overlap, the majority-vote tile-order hint, and the cost model of
this library's fused kernel.

Reference counterparts: tune/search.py:294-344 (interpolate_latency,
predict_lat), :462-471 (integer_partitions), :210-263 (hint vote and
rebalance), tune/bandwidth.py:128-135 (bus bandwidth).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

import torch

GIB = 1024 ** 3


def div_up(x: int, y: int) -> int:
    return (x + y - 1) // y


def compositions(n: int) -> List[List[int]]:
    """All ordered ways to write ``n`` as a sum of positive integers (2**(n-1) of
    them), in the order the reference enumerates them: first part ascending."""
    if n < 0:
        raise ValueError("n must be >= 0")
    out: List[List[int]] = []

    def rec(rest: int, path: List[int]):
        if rest == 0:
            out.append(path)
            return
        for first in range(1, rest + 1):
            rec(rest - first, path + [first])

    rec(n, [])
    return out


def bus_bandwidth_gbs(elements: float, seconds: float, world_size: int, comm_op: str, elem_bytes: int = 2) -> float:
    """Bus bandwidth in GiB-based GB/s: all-reduce moves 2(n-1)/n of the message
    per rank, reduce-scatter and all-gather (n-1)/n."""
    n = world_size
    if n <= 1 or seconds <= 0:
        return 0.0
    factor = 2.0 * (n - 1) / n if comm_op == "all_reduce" else (n - 1) / n
    return elements * elem_bytes * factor / seconds / GIB


def comm_latency_ms(curve: torch.Tensor, elements: float, world_size: int, comm_op: str, elem_bytes: int = 2) -> float:
    """Time of one collective on ``elements`` values, from a measured
    ``[elements, GB/s]`` curve (linear interpolation, clamped at both ends)."""
    if world_size <= 1 or elements <= 0:
        return 0.0
    curve = torch.as_tensor(curve, dtype=torch.float64)
    xs, ys = curve[:, 0].contiguous(), curve[:, 1].contiguous()
    x = float(elements)
    if x <= float(xs[0]):
        bw = float(ys[0])
    elif x >= float(xs[-1]):
        bw = float(ys[-1])
    else:
        i = int(torch.searchsorted(xs, torch.tensor(x, dtype=torch.float64)))
        x0, x1, y0, y1 = float(xs[i - 1]), float(xs[i]), float(ys[i - 1]), float(ys[i])
        bw = y0 + (y1 - y0) * (x - x0) / (x1 - x0)
    n = world_size
    factor = 2.0 * (n - 1) / n if comm_op == "all_reduce" else (n - 1) / n
    return x * elem_bytes * factor / max(bw, 1e-9) / GIB * 1e3


def predict_segmented_ms(M: int, N: int, gemm_ms: float, curve: torch.Tensor, groups: Sequence[int], tile_num: int,
                         comm_op: str, world_size: int, sm_count: int = 148, comm_sms: int = 2) -> float:
    """The reference's model of its two-stream overlap: the GEMM runs in waves of
    ``sm_count - comm_sms`` tiles (the collective's kernel occupies ``comm_sms``
    SMs); the collective of wave group i may start when group i is computed and
    the collective of group i-1 is done."""
    groups = list(groups)
    per_tile = M * N // tile_num
    if len(groups) == 1:
        return comm_latency_ms(curve, per_tile * groups[0], world_size, comm_op) + gemm_ms
    wave = sm_count - comm_sms
    old_waves = div_up(tile_num, sm_count)
    new_waves = div_up(tile_num, wave)
    gemm_ms = gemm_ms / old_waves * new_waves
    acc_comm = 0.0
    acc_comp = 0.0
    for i, g in enumerate(groups):
        comm = 0.0 if i == 0 else comm_latency_ms(curve, per_tile * groups[i - 1], world_size, comm_op)
        acc_comm = max(acc_comp, acc_comm) + comm
        acc_comp += gemm_ms / new_waves * div_up(g, wave)
    return max(acc_comp, acc_comm) + comm_latency_ms(curve, per_tile * groups[-1], world_size, comm_op)


def scale_groups(parts: Sequence[int], unit: int, tile_num: int) -> List[int]:
    """Turn a composition in units of ``unit`` tiles into tiles per group; the
    last group takes what is left."""
    out, acc = [], 0
    for j, p in enumerate(parts):
        if j < len(parts) - 1:
            g = p * unit
            acc += g
        else:
            g = min(p * unit, tile_num - acc)
        out.append(int(g))
    if any(g <= 0 for g in out) or sum(out) != tile_num:
        raise ValueError(f"composition {list(parts)} x {unit} does not cover {tile_num} tiles")
    return out


def best_segmentation(M: int, N: int, gemm_ms: float, curve: torch.Tensor, tile_num: int, comm_op: str,
                      world_size: int, sm_count: int = 148, comm_sms: int = 2, max_units: int = 10
                      ) -> Tuple[List[int], float]:
    """Predictive search of the reference: at most ``max_units`` wave units, every
    composition scored by the pipeline model; compositions with more than five
    groups and a first group above two units are skipped (cold start)."""
    wave = sm_count - comm_sms
    wave_num = div_up(tile_num, wave)
    min_group = div_up(wave_num, max_units)
    units = div_up(wave_num, min_group)
    best, best_ms = None, float("inf")
    for parts in compositions(units):
        if len(parts) > 5 and parts[0] > 2:
            continue
        try:
            groups = scale_groups(parts, wave * min_group, tile_num)
        except ValueError:
            continue
        ms = predict_segmented_ms(M, N, gemm_ms, curve, groups, tile_num, comm_op, world_size, sm_count, comm_sms)
        if ms < best_ms:
            best, best_ms = groups, ms
    if best is None:
        best, best_ms = [tile_num], predict_segmented_ms(M, N, gemm_ms, curve, [tile_num], tile_num, comm_op,
                                                         world_size, sm_count, comm_sms)
    return best, best_ms


def hint_from_samples(samples: torch.Tensor, wave_size: int) -> Tuple[bool, List[int]]:
    """Tile order from completion-ticket samples ``[n_samples, tiles]``: every
    tile goes to the wave (ticket // wave_size) it lands in most often; waves are
    then trimmed to exactly ``wave_size`` tiles, keeping the tiles that agreed
    most, and topped up from the surplus.  Returns (consistent, hint)."""
    samples = torch.as_tensor(samples).to(torch.long).cpu()
    if samples.dim() != 2 or samples.numel() == 0:
        raise ValueError("samples must be [n_samples, tiles]")
    tiles = samples.shape[1]
    waves = div_up(tiles, wave_size)
    wave_of = (samples // wave_size).clamp(max=waves - 1)
    modes = torch.mode(wave_of, dim=0).values
    agree = (wave_of == modes.unsqueeze(0)).sum(dim=0)
    targets = [wave_size if w < waves - 1 else tiles - w * wave_size for w in range(waves)]
    assigned: List[List[int]] = []
    surplus: List[int] = []
    for w in range(waves):
        members = (modes == w).nonzero(as_tuple=True)[0].tolist()
        members.sort(key=lambda t: (-int(agree[t]), -t))
        assigned.append(members[:targets[w]])
        surplus.extend(members[targets[w]:])
    for w in range(waves):
        while len(assigned[w]) < targets[w] and surplus:
            assigned[w].append(surplus.pop())
    ok = all(len(a) == t for a, t in zip(assigned, targets))
    hint = [t for a in assigned for t in a] if ok else []
    return ok, hint


def predict_fused_ms(M: int, N: int, gemm_ms: float, world_size: int, comm_op: str, p2p_gbs: float,
                     hbm_gbs: float = 6500.0, elem_bytes: int = 2, tail_us_per_row_round: float = 4.0,
                     sm_count: int = 148, reduce_group: int = 1) -> float:
    """Cost model of this library's fused kernel (one launch: GEMM phase that
    pushes partial tiles to their owners, then a reduce phase).

    * GEMM phase: the slower of the GEMM itself and pushing (n-1)/n of the output
      over NVLink at ``p2p_gbs`` (measured store bandwidth out of one GPU).
    * reduce phase: every rank reads n partial copies of its M/n rows from HBM;
      an all-reduce then stores those rows to all n ranks (again (n-1)/n of the
      output over NVLink), a reduce-scatter stores them once locally.  Rows are
      processed ``sm_count * 8 / reduce_group`` at a time with a fixed latency per
      round.
    """
    n = max(world_size, 1)
    out_bytes = float(M) * N * elem_bytes
    link_ms = out_bytes * (n - 1) / n / (p2p_gbs * 1e9) * 1e3 if n > 1 else 0.0
    phase1 = max(gemm_ms, link_ms)
    rows = M // n
    rounds = div_up(rows, max(1, sm_count * 8 // max(reduce_group, 1)))
    read_ms = out_bytes / (hbm_gbs * 1e9) * 1e3  # n copies of 1/n of the matrix
    if comm_op == "all_reduce":
        phase2 = max(link_ms, read_ms) + out_bytes / n / (hbm_gbs * 1e9) * 1e3
    else:
        phase2 = read_ms + out_bytes / n / (hbm_gbs * 1e9) * 1e3
    phase2 += rounds * tail_us_per_row_round * 1e-3
    return phase1 + phase2
