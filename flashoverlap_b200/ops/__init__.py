"""Functional wrappers over the native operators."""
from .functional import (  # noqa: F401
    a2a_dispatch_gemm,
    allgather_gemm,
    gemm,
    gemm_allreduce,
    gemm_reducescatter,
    gemm_rmsnorm,
    reorder_rmsnorm,
    rmsnorm,
)
