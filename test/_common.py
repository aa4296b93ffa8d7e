import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tune"))
from _common import *  # noqa: F401,F403,E402
from _common import DTYPES, finish, make_baseline_impl, make_overlap_impl, start, torch  # noqa: F401,E402
