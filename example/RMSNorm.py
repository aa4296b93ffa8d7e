"""RMSNorm modules under the reference's module name (reference: example/RMSNorm.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flashoverlap_b200.models.rmsnorm import KernelRMSNorm, ReorderRMSNorm, RMSNorm  # noqa: F401,E402
