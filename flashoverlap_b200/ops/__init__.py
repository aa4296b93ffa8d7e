"""Functional wrappers over the native operators."""
from .functional import (  # noqa: F401
    gemm,
    gemm_allreduce,
    gemm_reducescatter,
    gemm_rmsnorm,
    reorder_rmsnorm,
    rmsnorm,
)
