"""flashoverlap_b200: GEMM + collective overlap for NVIDIA B200 (sm_100a).

The package offers the capabilities of FlashOverlap (fused GEMM+AllReduce /
GEMM+ReduceScatter with tile-order-aware RMSNorm, a non-overlapped baseline,
a wave-group tuner and its config files) on a different engine: every
overlapped operation is one persistent tcgen05/TMEM kernel that pushes
finished tiles to peer GPUs over NVLink and reduces them in a trailing phase.

Importing the package loads the native library and registers
``torch.classes.flashoverlap_class.{OverlapImpl, BaselineImpl}`` and
``torch.ops.flashoverlap_op.*`` (reference: src/pybind.cpp:114-150).
"""
from __future__ import annotations

import torch

from . import _build

__version__ = "0.1.0"

_native_error: Exception | None = None
try:
    _build.load()
except Exception as exc:  # pragma: no cover - depends on the machine
    _native_error = exc
    if torch.cuda.is_available():
        raise RuntimeError(
            "flashoverlap_b200: the native sm_100a library could not be loaded on a machine with a GPU; "
            "build it with `python -m flashoverlap_b200._build`"
        ) from exc


def native_available() -> bool:
    """True when the compiled library is loaded in this process."""
    return _native_error is None


def library_path() -> str:
    """Path of the shared library (what ``torch.ops.load_library`` expects)."""
    return str(_build.library_path())


def require_native() -> None:
    if _native_error is not None:
        raise RuntimeError("flashoverlap_b200: native library unavailable") from _native_error


from .utils.reorder import (  # noqa: E402
    div_up,
    generate_row_mapping,
    reorder_indices,
    reorder_rows_by_world_size,
)

__all__ = [
    "native_available",
    "library_path",
    "require_native",
    "div_up",
    "reorder_indices",
    "generate_row_mapping",
    "reorder_rows_by_world_size",
]
