"""Functional wrappers over the native operators."""
from .functional import (  # noqa: F401
    allgather_gemm,
    gemm,
    gemm_allreduce,
    gemm_reducescatter,
    gemm_rmsnorm,
    reorder_rmsnorm,
    rmsnorm,
)
