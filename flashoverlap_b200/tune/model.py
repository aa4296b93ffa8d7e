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


def hint_from_samples(samples: torch.Tensor, wave_size: int, min_agree: int = 0) -> Tuple[bool, List[int]]:
    """Tile order from completion-ticket samples ``[n_samples, tiles]``: every
    tile goes to the wave (ticket // wave_size) it lands in most often; waves are
    then trimmed to exactly ``wave_size`` tiles, keeping the tiles that agreed
    most, and topped up from the surplus.  Returns (consistent, hint).

    ``min_agree`` > 0 is the stricter rule of the reference's multi-node search
    (reference: tune/search_multinode.py:165-182): a tile only counts for its
    wave when it landed there in at least ``min_agree`` samples (9 of 10
    there); if that leaves a wave short by more than the surplus can fill, the
    order is reported inconsistent."""
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
        if min_agree > 0:
            unsure = [t for t in members if int(agree[t]) < min_agree]
            if len(unsure) * 10 > max(1, len(members)):  # more than a tenth of the wave is unstable
                return False, []
        assigned.append(members[:targets[w]])
        surplus.extend(members[targets[w]:])
    for w in range(waves):
        while len(assigned[w]) < targets[w] and surplus:
            assigned[w].append(surplus.pop())
    ok = all(len(a) == t for a, t in zip(assigned, targets))
    hint = [t for a in assigned for t in a] if ok else []
    return ok, hint


def raster_group_sizes(tile_rows: int, raster_group: int, taper: bool = True) -> List[int]:
    """Tile rows per raster group in the order the kernel walks them: full
    groups, and with ``taper`` the last ones shrink by halves down to 1, 1 (the
    same rule as ``tile_coords`` in the kernel)."""
    G = max(int(raster_group), 1)
    remaining, size, out = int(tile_rows), G, []
    if not taper:
        while remaining > 0:
            out.append(min(G, remaining))
            remaining -= out[-1]
        return out
    while remaining > 0:
        if remaining <= size:
            size = (remaining + 1) // 2 if remaining > 1 else 1
        out.append(size)
        remaining -= size
    return out


def predict_fused_ms(M: int, N: int, gemm_ms: float, world_size: int, comm_op: str, link_gbs: float,
                     transport: str = "p2p", hbm_gbs: float = 6500.0, elem_bytes: int = 2, tile_m: int = 256,
                     raster_group: int = 2, sm_count: int = 148, latency_us: float = 8.0, taper: bool = True,
                     row_us: float = 0.0, groups_gemm: int = 1, groups_tail: int = 3) -> float:
    """Cost model of this library's fused kernel: one launch in which row
    groups (4 warps) reduce and deliver finished rows while the tensor cores
    compute later tiles.

    The rows of a raster group can be reduced once the whole group is computed.
    The model walks the groups in the kernel's order: group j completes at
    ``gemm_ms`` times its share of the tiles and adds its rows (this rank's
    1/n of them) to a queue; the queue drains at ``groups_gemm`` row groups per
    SM while the GEMM runs and ``groups_tail`` per SM after it, each taking
    ``row_us`` per row (MEASURED by ``tune.runtime.measure_row_us``: it holds
    the memory, link and latency cost of one row on this machine).  What is
    left in the queue when the last tile is done is the tail.  Without a
    measured ``row_us`` the row time is taken from the bytes of one row at the
    link (or, with one rank, HBM) bandwidth.

    The result is never below the time the collective's bytes need at
    ``link_gbs``, the MEASURED bandwidth of the transport.  Bytes per NVLink
    direction, with S = M*N*elem_bytes and n ranks: all-reduce over
    peer-to-peer stores 2*S*(n-1)/n, over NVLink SHARP S*(1+1/n);
    reduce-scatter S*(n-1)/n (S over NVLink SHARP); one rank: HBM, 2*S.
    """
    n = max(world_size, 1)
    S = float(M) * N * elem_bytes
    if n == 1:
        per_dir, bw = 2.0 * S, hbm_gbs
    elif comm_op == "all_reduce":
        per_dir = S * (1.0 + 1.0 / n) if transport == "nvls" else 2.0 * S * (n - 1) / n
        bw = link_gbs
    else:
        per_dir = S if transport == "nvls" else S * (n - 1) / n
        bw = link_gbs
    comm_us = per_dir / (bw * 1e9) * 1e6
    rows_owned = M / n
    if row_us <= 0.0:
        # all row groups of the GPU together move the collective's bytes at the measured bandwidth
        row_us = comm_us / max(rows_owned, 1.0) * sm_count * groups_tail
    gemm_us = gemm_ms * 1e3
    sizes = raster_group_sizes(div_up(M, tile_m), raster_group, taper)
    total = float(sum(sizes))
    rate_gemm = sm_count * groups_gemm / row_us   # rows per us while the GEMM runs
    rate_tail = sm_count * groups_tail / row_us
    t_prev, backlog, done = 0.0, 0.0, 0.0
    for size in sizes:
        done += size
        t = gemm_us * done / total
        backlog = max(0.0, backlog - rate_gemm * (t - t_prev))
        backlog += size * tile_m / n
        t_prev = t
    end_us = gemm_us + backlog / rate_tail + latency_us
    first_us = gemm_us * sizes[0] / total
    return max(end_us, first_us + comm_us * (1.0 - 1.0 / len(sizes)) + latency_us, comm_us + latency_us) * 1e-3


def _algo_tiles():
    from ..utils.config import ALGO_TILES

    return ALGO_TILES


def gather_algo_candidates(rows_per_source: int, n: int, sms: int = 148) -> List[int]:
    """Tile configurations worth timing for all-gather -> GEMM and all-to-all
    dispatch -> GEMM.  The GEMM consumes the gathered matrix source by source
    as the blocks arrive, so what matters is how many tiles ONE source's block
    gives: a block of 1024 rows and 1280 columns is 20 tiles of 256 x 256 (a
    quarter of the machine busy per step) but 80 tiles of 128 x 128.  Returns
    the configurations ordered by the estimated time per block, best first:
    waves needed for the block's tiles times the area of a tile, with small
    tiles charged for their measured lower throughput."""
    rows = max(int(rows_per_source), 1)
    # time per output element relative to the 256 x 256 CTA-pair tile, from the stage-1 profile of a
    # 4096 x 8192 x 4096 GEMM (tune/profile_config.py) on a B200
    penalty = {(256, 256): 1.0, (128, 256): 1.13, (128, 128): 1.34, (256, 128): 1.6, (128, 64): 2.3, (256, 64): 2.8}
    scored = []
    for algo, (bm, bn, bk) in enumerate(_algo_tiles()):
        if bk != 128 and (bm, bn) != (128, 256):   # one K depth per tile shape
            continue
        if n % bn:
            continue
        ctas = bm // 128
        tiles = -(-rows // bm) * (n // bn)
        slots = max(1, sms // ctas)
        waves = -(-tiles // slots)
        per_tile = bm * bn / ctas * penalty.get((bm, bn), 2.0)
        scored.append((waves * per_tile, -bm * bn, algo))
    scored.sort()
    return [a for _, _, a in scored]
