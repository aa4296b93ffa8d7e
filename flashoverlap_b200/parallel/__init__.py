"""Process-group bootstrap and construction of the communication objects."""
from .bootstrap import (  # noqa: F401
    attach_symmetric_memory,
    workspace_bytes,
    broadcast_nccl_id,
    init_distributed,
    make_baseline_impl,
    make_overlap_impl,
    max_over_ranks,
)
from .hierarchy import Hierarchy, build_hierarchy, make_intra_node_impl, node_layout  # noqa: F401,E402
