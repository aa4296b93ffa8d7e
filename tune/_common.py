"""Shared start-up of the command-line tools: make the package importable from
a source checkout and bring up one process per GPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import flashoverlap_b200  # noqa: E402,F401
from flashoverlap_b200.parallel import init_distributed, make_baseline_impl, make_overlap_impl  # noqa: E402

DTYPES = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def start():
    """(rank, world_size) after process-group and device set-up."""
    rank, world, _ = init_distributed()
    return rank, world


def finish():
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
