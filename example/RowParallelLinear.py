"""Row-parallel layers under the reference's module name (reference: example/RowParallelLinear.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flashoverlap_b200.models.row_parallel import (  # noqa: F401,E402
    FusedRowParallelLinear,
    OverlapRowParallelLayer,
    RowParallelLayer,
)
