"""Stage 1 from a profiler CSV (tune/gen_config.py): row selection on CPU."""
import importlib.util
import os

import pytest

from flashoverlap_b200.utils import config as cfg

HERE = os.path.dirname(os.path.abspath(__file__))


def load_tool():
    spec = importlib.util.spec_from_file_location("fo_gen_config", os.path.join(HERE, "..", "tune", "gen_config.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def write_csv(path, rows, header="Problem,cta_m,cta_n,cta_k,split_k_slices,Runtime"):
    with open(path, "w") as fh:
        fh.write(header + "\n")
        for r in rows:
            fh.write(",".join(str(v) for v in r) + "\n")


def test_rows_are_sorted_by_runtime_and_mapped_to_algos(tmp_path):
    tool = load_tool()
    f = tmp_path / "m4096n8192k1024.gemm.csv"
    write_csv(f, [("g", 128, 128, 64, 1, 0.30), ("g", 256, 256, 64, 1, 0.10), ("g", 64, 64, 32, 1, 0.05),
                  ("g", 128, 256, 64, 1, 0.20), ("g", 256, 256, 64, 1, 0.11)])
    algos = tool.rows_from_csv(str(f), cfg.algo_dict())
    d = cfg.algo_dict()
    # the 64x64x32 shape does not exist in this build and is skipped; duplicates collapse
    assert algos == [d[(256, 256, 64)], d[(128, 256, 64)], d[(128, 128, 64)]]


def test_split_k_rows_are_rejected(tmp_path):
    tool = load_tool()
    f = tmp_path / "x.gemm.csv"
    write_csv(f, [("g", 256, 256, 64, 2, 0.10)])
    with pytest.raises(AssertionError, match="split-K"):
        tool.rows_from_csv(str(f), cfg.algo_dict())


def test_missing_column_is_reported(tmp_path):
    tool = load_tool()
    f = tmp_path / "y.gemm.csv"
    write_csv(f, [("g", 256, 256, 0.1)], header="Problem,cta_m,cta_n,Runtime")
    with pytest.raises(ValueError, match="cta_k"):
        tool.rows_from_csv(str(f), cfg.algo_dict())
