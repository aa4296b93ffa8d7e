"""nn.Modules built on the fused operations."""
from .rmsnorm import RMSNorm, ReorderRMSNorm  # noqa: F401
from .row_parallel import (  # noqa: F401
    FusedRowParallelLinear,
    HierarchicalRowParallelLinear,
    OverlapRowParallelLayer,
    RowParallelLayer,
)
