"""Device-independent emulation of the fused kernel's data flow with
``torch.distributed`` collectives (works on CPU with the gloo backend).

It follows the kernel step by step (who owns which row, what is pushed where,
in which layout the result is stored) so that the host-side logic and the
semantics of every fused entry point can be checked without a GPU, and it is
the oracle the GPU tests compare layouts with.  It is not a fast path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..utils.reorder import to_tile_order


def _world(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 statistics, result rounded to the input type, then multiplied by the
    weight in the input type: the rounding order of the kernels."""
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return y * weight.to(x.dtype)


def owned_rows(M: int, rank: int, world: int, interleave: bool) -> torch.Tensor:
    """Global row indices owned by ``rank`` in the reduce phase."""
    if interleave:
        return torch.arange(rank, M, world)
    rows = M // world
    return torch.arange(rank * rows, (rank + 1) * rows)


def push_and_reduce(partial: torch.Tensor, interleave: bool, group=None) -> torch.Tensor:
    """GEMM-phase push + reduce-phase sum: every rank sends each owner its rows
    of the partial product (rounded to the partial's dtype, as the epilogue
    stores it); the owner adds the ``world`` copies in fp32 and rounds once."""
    rank, world = _world(group)
    M, N = partial.shape
    if world == 1:
        return partial.clone()
    send = torch.cat([partial[owned_rows(M, r, world, interleave)] for r in range(world)]).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(world, M // world, N).float().sum(0).to(partial.dtype)


def gemm_reducescatter(a: torch.Tensor, b: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                       eps: float = 1e-5, interleave: bool = False, group=None) -> torch.Tensor:
    """Rows owned by this rank of ``sum_r a_r @ b_r^T`` (optionally RMS-normalised)."""
    partial = (a.float() @ b.float().t()).to(a.dtype)
    mine = push_and_reduce(partial, interleave, group)
    return rmsnorm_reference(mine, norm_weight, eps) if norm_weight is not None else mine


def gemm_allreduce(a: torch.Tensor, b: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-5,
                   group=None) -> torch.Tensor:
    """Full ``sum_r a_r @ b_r^T`` on every rank: interleaved reduce-scatter, then
    every owner delivers its (normalised) rows to all ranks."""
    rank, world = _world(group)
    mine = gemm_reducescatter(a, b, norm_weight, eps, True, group)
    if world == 1:
        return mine
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine.contiguous(), group=group)
    M = a.shape[0]
    out = torch.empty((M, b.shape[0]), dtype=a.dtype, device=a.device)
    for r in range(world):
        out[owned_rows(M, r, world, True)] = parts[r]
    return out


def gemm_allreduce_overlap(a, b, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1, group=None) -> torch.Tensor:
    """What ``OverlapImpl.gemm_allreduce_overlap`` leaves in C: the all-reduced
    product in tile-reordered layout."""
    return to_tile_order(gemm_allreduce(a, b, group=group), BM, BN, RA.cpu(), rldn)


def gemm_reducescatter_overlap(a, b, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1, group=None) -> torch.Tensor:
    """What ``OverlapImpl.gemm_reducescatter_overlap`` leaves in D: this rank's
    interleaved rows, tile-reordered with tiles of ``BM / world`` rows."""
    _, world = _world(group)
    mine = gemm_reducescatter(a, b, None, 0.0, True, group)
    return to_tile_order(mine, BM // world, BN, RA.cpu(), rldn)
