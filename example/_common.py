"""Start-up shared with the tuning tools (tune/_common.py), loaded by path."""
import importlib.util
import os

_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tune", "_common.py")
_spec = importlib.util.spec_from_file_location("_fo_tune_common", _path)
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)

DTYPES = _mod.DTYPES
finish = _mod.finish
start = _mod.start
make_baseline_impl = _mod.make_baseline_impl
make_overlap_impl = _mod.make_overlap_impl
torch = _mod.torch
