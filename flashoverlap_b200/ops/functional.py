"""Functional interface to the sm_100a kernels.  All functions require CUDA
tensors and raise if the native library is missing."""
from __future__ import annotations

from typing import Optional

import torch


def _check(x: torch.Tensor):
    if not x.is_cuda:
        raise RuntimeError("flashoverlap_b200 ops run on CUDA tensors only")


def gemm(impl, a: torch.Tensor, b: torch.Tensor, algo: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T`` on the tcgen05 kernel (reference: cutlass_gemm)."""
    _check(a)
    if out is None:
        out = torch.empty((a.size(0), b.size(0)), dtype=a.dtype, device=a.device)
    impl.cutlass_gemm(a, b, out, algo)
    return out


def gemm_rmsnorm(impl, a, b, weight, eps: float = 1e-5, algo: int = 0):
    """GEMM followed by RMSNorm in one launch on one GPU; returns (product, normalised)."""
    _check(a)
    c = torch.empty((a.size(0), b.size(0)), dtype=a.dtype, device=a.device)
    o = torch.empty_like(c)
    impl.gemm_rmsnorm(a, b, c, o, weight, eps, algo)
    return c, o


def gemm_allreduce(impl, a, b, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-5, algo: int = 0):
    """Fused GEMM + all-reduce (+ RMSNorm).  The result aliases the symmetric
    result buffer of ``impl`` (valid until the second next fused call)."""
    _check(a)
    return impl.gemm_allreduce_fused(a, b, norm_weight, eps, algo)


def gemm_reducescatter(impl, a, b, world_size: int, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-5,
                       algo: int = 0, interleave: bool = False, out: Optional[torch.Tensor] = None):
    """Fused GEMM + reduce-scatter (+ RMSNorm) into ``[M / world_size, N]``."""
    _check(a)
    if out is None:
        out = torch.empty((a.size(0) // world_size, b.size(0)), dtype=a.dtype, device=a.device)
    impl.gemm_reducescatter_fused(a, b, out, norm_weight, eps, algo, interleave)
    return out


def allgather_gemm(impl, a_shard, b, world_size: int, algo: int = 0, out: Optional[torch.Tensor] = None):
    """Fused all-gather + GEMM: ``gather(a_shard)[M, K] @ b[N, K]^T`` with the
    gather pushed over NVLink by the same kernel that computes the product."""
    _check(a_shard)
    if out is None:
        out = torch.empty((a_shard.size(0) * world_size, b.size(0)), dtype=a_shard.dtype, device=a_shard.device)
    impl.allgather_gemm(a_shard, b, out, algo)
    return out


def a2a_dispatch_gemm(impl, a_send, b, mlen_cpu: torch.Tensor, rank: int, algo: int = 0):
    """Fused all-to-all dispatch + GEMM: ``mlen_cpu[i][j]`` rows travel from rank i
    to rank j (``a_send`` holds this rank's rows in destination order); returns
    the product of the rows received here, in source order, with ``b^T``."""
    _check(a_send)
    m_pad = impl.a2a_padded_rows(mlen_cpu, algo)
    out = torch.empty((m_pad, b.size(0)), dtype=a_send.dtype, device=a_send.device)
    impl.a2a_dispatch_gemm(a_send, b, out, mlen_cpu, algo)
    return out[: int(mlen_cpu[:, rank].sum())]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    _check(x)
    out = torch.empty_like(x)
    torch.ops.flashoverlap_op.rmsnorm(x, out, weight, eps)
    return out


def reorder_rmsnorm(x, weight, bm: int, bn: int, ra: torch.Tensor, rldn: int = 1, eps: float = 1e-5):
    _check(x)
    out = torch.empty_like(x)
    torch.ops.flashoverlap_op.reorder_rmsnorm_eps(x, out, weight, bm, bn, rldn, ra, eps)
    return out
