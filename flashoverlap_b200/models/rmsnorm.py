"""RMSNorm modules (reference: example/RMSNorm.py:10-37)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from ..utils.reorder import div_up, reorder_indices


def _device(device):
    if device is not None:
        return torch.device(device)
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


class RMSNorm(nn.Module):
    """Plain PyTorch RMSNorm: fp32 statistics, result cast to the input dtype,
    then multiplied by the weight (the golden path of the correctness checks)."""

    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.float16, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.empty(dim, dtype=dtype, device=_device(device)).normal_(mean=0.0, std=0.5))

    def _norm(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)

    def forward(self, x):
        return self._norm(x.float()).type_as(x) * self.weight


class KernelRMSNorm(RMSNorm):
    """RMSNorm through the sm_100a kernel (natural layout in and out)."""

    def forward(self, x):
        if not x.is_cuda:
            return super().forward(x)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        out = torch.empty_like(x2)
        torch.ops.flashoverlap_op.rmsnorm(x2, out, self.weight, float(self.eps))
        return out.reshape(shape)


class ReorderRMSNorm(nn.Module):
    """RMSNorm that reads its input in the tile-reordered layout written by
    ``gemm_allreduce_overlap`` / ``gemm_reducescatter_overlap`` and writes rows
    in natural order (reference: example/RMSNorm.py:23-37).  Unlike the
    reference, ``eps`` is honoured by the kernel."""

    def __init__(self, dim: int, M: int, BM: int, BN: int, hint: Sequence[int], eps: float = 1e-5,
                 dtype=torch.float16, device=None):
        super().__init__()
        self.eps = eps
        dev = _device(device)
        self.weight = nn.Parameter(torch.empty(dim, dtype=dtype, device=dev).normal_(mean=0.0, std=0.5))
        self.bm, self.bn = BM, BN
        tm, tn = div_up(M, BM), div_up(dim, BN)
        self.register_buffer("reorder_array", reorder_indices(tm * tn, hint, device=dev).reshape(tm, tn),
                             persistent=False)

    def forward(self, x):
        out = torch.empty_like(x)
        torch.ops.flashoverlap_op.reorder_rmsnorm_eps(x, out, self.weight, self.bm, self.bn, 1, self.reorder_array,
                                                      float(self.eps))
        return out
