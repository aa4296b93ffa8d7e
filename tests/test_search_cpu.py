"""The two search drivers on CPU with the GPU-side measurements replaced by a
deterministic fake: both must pick the same solution (exhaustive times every
candidate, predictive times only its best-ranked few) and write a valid stage-2
file in the reference's format."""
import json

import pytest
import torch

import types

from flashoverlap_b200.tune import runtime, search
from flashoverlap_b200.utils import config as cfg


def fake_time(algo, raster, cseg, two_stream):
    # fused path: Algo 3 fastest, raster 2 best; two-stream path: three groups best
    if two_stream:
        return 0.5 + 0.02 * abs(len(cseg) - 3) + 0.001 * abs(cseg[0] - cseg[-1]) / max(cseg)
    return 0.2 + 0.01 * abs(algo - 3) + 0.002 * abs(raster - 2)


@pytest.fixture
def patched(monkeypatch, tmp_path):
    calls = []

    def perf_running(impl, M, N, K, BM, BN, algo, cseg, hint, comm_op, dtype=None, warmup=0, reps=0, raster_group=0,
                     two_stream=False, gemm_ctas=0):
        calls.append((algo, raster_group, tuple(cseg), two_stream))
        return fake_time(algo, raster_group, list(cseg), two_stream)

    def compute_hint(impl, M, N, K, BM, BN, algo, wave, comm_op, dtype=None, **kw):
        tiles = (M // BM) * (N // BN)
        return True, list(reversed(range(tiles)))

    monkeypatch.setattr(search, "perf_running", perf_running)
    monkeypatch.setattr(runtime, "perf_running", perf_running)
    monkeypatch.setattr(runtime, "world", lambda: (0, 8))
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda *a, **k: types.SimpleNamespace(multi_processor_count=148))
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(search, "compute_hint", compute_hint)
    monkeypatch.setattr(search, "measure_row_us", lambda *a, **k: 6.0)
    monkeypatch.setattr(search, "sm_count", lambda: 148)
    monkeypatch.setattr(search, "world", lambda: (0, 8))
    monkeypatch.setattr(cfg, "gpu_tag", lambda name=None: "b200")
    M, N, K = 4096, 8192, 1024
    cfg.save_stage1(M, N, K, [256, 128, 128], [256, 256, 128], [0.054, 0.057, 0.08], [3, 0, 1], tmp_path)
    return calls, tmp_path, (M, N, K)


def test_exhaustive_and_predictive_agree(patched):
    calls, path, (M, N, K) = patched
    ex = search.exhaustive_search(None, M, N, K, "all_reduce", path=path, verbose=False)
    n_exhaustive = len(calls)
    assert ex["Algo"] == 3 and ex["raster_group"] == 2
    # the wave grouping was searched by timing compositions on the two-stream path
    timed_groupings = {c[2] for c in calls if c[3]}
    assert len(timed_groupings) == ex["candidates_timed"] > 4
    assert len(ex["cSeg"]) == 3 and ex["two_stream_dur"] == min(fake_time(3, 0, list(g), True) for g in timed_groupings)
    # re-running from the stage-2 file works because the stage-1 lists are kept
    calls.clear()
    curve = torch.tensor([[2.0 ** 20, 150.0], [2.0 ** 26, 420.0]])
    pr = search.predictive_search(None, M, N, K, "all_reduce", curve, 550.0, path=path, verbose=False)
    assert len([c for c in calls if not c[3]]) <= 3 and len(calls) < n_exhaustive
    assert len([c for c in calls if c[3]]) == 1  # the predicted grouping is timed once
    assert (pr["Algo"], pr["raster_group"]) == (ex["Algo"], ex["raster_group"])
    data = json.load(open(cfg.json_path(M, N, K, path)))
    cfg.validate_stage2(data, M, N)
    tiles = (M // 256) * (N // 256)
    assert sum(data["cSeg"]) == tiles and data["rLDN"] == 1 and len(data["hint"]) == tiles
    assert data["search"] == "predictive" and data["stage1"]["Algo"] == [3, 0, 1]


def test_search_fails_loudly_without_consistent_hint(patched, monkeypatch):
    calls, path, (M, N, K) = patched
    monkeypatch.setattr(search, "compute_hint", lambda *a, **k: (False, []))
    with pytest.raises(RuntimeError, match="tuning failed"):
        search.exhaustive_search(None, M, N, K, "all_reduce", path=path, verbose=False)


def test_knob_candidates_cover_defaults():
    assert search.knob_candidates(4096, 256) == [1, 2, 4, 8]
    assert search.knob_candidates(512, 256) == [1, 2]


def test_predictive_search_needs_a_measured_link_bandwidth(patched):
    calls, path, (M, N, K) = patched
    curve = torch.tensor([[2.0 ** 20, 150.0], [2.0 ** 26, 420.0]])
    with pytest.raises(ValueError, match="measured link bandwidth"):
        search.predictive_search(None, M, N, K, "all_reduce", curve, None, path=path, verbose=False)


def test_gather_algo_candidates_prefer_tiles_that_fill_the_machine():
    from flashoverlap_b200.tune.runtime import gather_algo_candidates
    from flashoverlap_b200.utils.config import ALGO_TILES

    # 1024 rows per source, 1280 columns: 256x256 gives 20 tiles per block, too few for 74 CTA pairs
    first = ALGO_TILES[gather_algo_candidates(1024, 1280)[0]]
    assert first[0] * first[1] < 256 * 256
    # a block that fills the machine several times over keeps the large tile
    assert ALGO_TILES[gather_algo_candidates(8192, 10240)[0]][:2] == (256, 256)
    # only tile widths that divide N are offered
    assert all(1280 % ALGO_TILES[a][1] == 0 for a in gather_algo_candidates(1024, 1280))
    assert all(ALGO_TILES[a][1] == 64 for a in gather_algo_candidates(512, 192))


def test_pick_algo_by_timing_keeps_the_fastest(monkeypatch):
    from flashoverlap_b200.tune import runtime

    cost = {0: 3.0, 6: 1.0, 9: 2.0}
    calls = []
    monkeypatch.setattr(runtime, "mean_time_ms", lambda fn, w, r, flush=False: (fn(), cost[calls[-1]])[1])
    best, timed = runtime.pick_algo_by_timing(lambda a: calls.append(a), [0, 6, 9])
    assert best == 6 and [a for a, _ in timed] == [0, 6, 9]
