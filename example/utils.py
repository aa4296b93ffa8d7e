"""Index helpers under the reference's module name (reference: example/utils.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flashoverlap_b200.utils.reorder import (  # noqa: F401,E402
    div_up,
    generate_row_mapping,
    reorder_indices,
    reorder_rows_by_world_size,
)
