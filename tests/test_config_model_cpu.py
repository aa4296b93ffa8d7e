"""Config files (reference formats) and the analytical pieces of the tuner."""
import json

import pytest
import torch

from flashoverlap_b200.tune import model
from flashoverlap_b200.utils import config as cfg


def test_gpu_tag_matches_reference_slicing():
    assert cfg.gpu_tag("NVIDIA B200") == "b200"
    assert cfg.gpu_tag("NVIDIA A800-SXM4-80GB") == "a800"


def test_algo_dict_roundtrip(tmp_path):
    f = cfg.save_algo_dict(tmp_path)
    d = cfg.load_algo_dict(tmp_path)
    assert f.name == "AlgoDict.pt" and d[(256, 256, 64)] == 3 and d[(128, 256, 64)] == 0


def test_stage1_stage2_roundtrip_and_rerun(tmp_path):
    M, N, K = 1024, 2048, 512
    cfg.save_stage1(M, N, K, [256, 128], [256, 256], [0.05, 0.06], [3, 0], tmp_path, "b200")
    d = cfg.load_config(M, N, K, tmp_path, "b200")
    assert d["BM"] == [256, 128] and not cfg.is_stage2(d)
    tiles = (M // 256) * (N // 256)
    cfg.save_stage2(M, N, K, 256, 256, 0.05, 3, list(range(tiles)), [tiles // 2, tiles // 2], tmp_path, "b200",
                    raster_group=2)
    d2 = cfg.load_config(M, N, K, tmp_path, "b200")
    assert cfg.is_stage2(d2) and d2["rLDN"] == 1 and d2["BM"] == 256 and d2["raster_group"] == 2
    # the reference's reader sees plain scalars and lists
    raw = json.load(open(cfg.json_path(M, N, K, tmp_path, "b200")))
    assert isinstance(raw["hint"], list) and isinstance(raw["cSeg"], list) and isinstance(raw["dur"], float)
    # stage-1 candidates survive, so the search can be re-run without re-profiling
    assert cfg.stage1_lists(d2)[3] == [3, 0]
    cfg.validate_stage2(d2, M, N)


def test_config_fault_injection(tmp_path):
    M, N, K = 512, 512, 64
    with pytest.raises(FileNotFoundError):
        cfg.load_config(M, N, K, tmp_path, "b200")
    cfg.json_path(M, N, K, tmp_path, "b200").write_text("{ this is not json")
    with pytest.raises(ValueError, match="not valid JSON"):
        cfg.load_config(M, N, K, tmp_path, "b200")
    cfg.json_path(M, N, K, tmp_path, "b200").write_text(json.dumps({"BM": [128]}))
    with pytest.raises(ValueError, match="lacks"):
        cfg.load_config(M, N, K, tmp_path, "b200")
    good = dict(BM=256, BN=256, dur=0.1, Algo=3, hint=[0, 1, 2, 3], cSeg=[2, 2], rLDN=1)
    cfg.validate_stage2(good, M, N)
    for bad in (dict(good, cSeg=[2, 1]), dict(good, hint=[0, 0]), dict(good, hint=[0, 9]), dict(good, Algo=0),
                dict(good, BM=384), dict(good, cSeg=[4, 0])):
        with pytest.raises(ValueError):
            cfg.validate_stage2(bad, M, N)
    with pytest.raises(ValueError):
        cfg.save_stage1(M, N, K, [], [], [], [], tmp_path)


def test_bandwidth_curve_roundtrip(tmp_path):
    curve = torch.tensor([[2.0 ** 20, 100.0], [2.0 ** 24, 400.0]])
    f = cfg.save_bandwidth(curve, "all_reduce", 8, path=tmp_path)
    assert f.name == "bandwidth_all_reduce_tp8.pt"
    assert cfg.bandwidth_path("reduce_scatter", 16, True, tmp_path).name == "bandwidth_reduce_scatter_ws16.pt"
    assert torch.equal(cfg.load_bandwidth("all_reduce", 8, path=tmp_path), curve)
    with pytest.raises(ValueError):
        cfg.save_bandwidth(torch.zeros(3), "all_reduce", 8, path=tmp_path)


def test_compositions():
    for n in range(1, 9):
        c = model.compositions(n)
        assert len(c) == 2 ** (n - 1) and all(sum(p) == n for p in c) and len({tuple(p) for p in c}) == len(c)
    assert model.compositions(3) == [[1, 1, 1], [1, 2], [2, 1], [3]]


def test_bus_bandwidth_and_latency_are_inverse():
    curve = torch.tensor([[2.0 ** 20, 100.0], [2.0 ** 22, 300.0], [2.0 ** 26, 400.0]])
    for op in ("all_reduce", "reduce_scatter"):
        for n in (2.0 ** 21, 2.0 ** 24):
            ms = model.comm_latency_ms(curve, n, 8, op)
            bw = model.bus_bandwidth_gbs(n, ms * 1e-3, 8, op)
            lo, hi = (100.0, 300.0) if n < 2 ** 22 else (300.0, 400.0)
            assert lo <= bw <= hi
    # clamped outside the curve; nothing to send on one rank
    assert model.comm_latency_ms(curve, 2.0 ** 30, 8, "all_reduce") == pytest.approx(
        2.0 ** 30 * 2 * 1.75 / 400.0 / 1024 ** 3 * 1e3)
    assert model.comm_latency_ms(curve, 2.0 ** 22, 1, "all_reduce") == 0.0


def test_segmented_model_matches_hand_computation():
    # flat 100 GB/s curve, 8 ranks, 4 waves of 146 tiles: overlap hides all but the last collective
    curve = torch.tensor([[1.0, 100.0], [1e12, 100.0]])
    sm, lost = 148, 2
    tiles = 4 * (sm - lost)
    M = N = 4096
    one = model.predict_segmented_ms(M, N, 1.0, curve, [tiles], tiles, "all_reduce", 8, sm, lost)
    comm_all = model.comm_latency_ms(curve, M * N, 8, "all_reduce")
    assert one == pytest.approx(1.0 + comm_all, rel=1e-4)
    groups = [sm - lost] * 4
    four = model.predict_segmented_ms(M, N, 1.0, curve, groups, tiles, "all_reduce", 8, sm, lost)
    c = comm_all / 4
    comp, comm = 0.0, 0.0
    for i in range(4):
        comm = max(comp, comm) + (0 if i == 0 else c)
        comp += 1.0 / 4  # ceil(584/148) = ceil(584/146) = 4 waves: the GEMM time is not rescaled
    expect = max(comp, comm) + c
    assert four == pytest.approx(expect, rel=1e-4)  # (M*N // tiles) rounds the message size down
    assert four < one
    best, best_ms = model.best_segmentation(M, N, 1.0, curve, tiles, "all_reduce", 8, sm, lost)
    assert sum(best) == tiles and best_ms <= four + 1e-9


def test_scale_groups():
    assert model.scale_groups([1, 2, 1], 146, 500) == [146, 292, 62]
    with pytest.raises(ValueError):
        model.scale_groups([1, 1], 146, 100)


def test_hint_vote_recovers_order_under_noise():
    torch.manual_seed(0)
    tiles, wave = 64, 16
    order = torch.randperm(tiles)            # order[i] = tile finishing i-th
    ticket = torch.empty(tiles, dtype=torch.long)
    ticket[order] = torch.arange(tiles)
    samples = ticket.repeat(20, 1)
    # in a quarter of the samples two tiles of neighbouring waves swap
    for s in range(0, 20, 4):
        a, b = int(order[15]), int(order[16])
        samples[s, a], samples[s, b] = samples[s, b].clone(), samples[s, a].clone()
    ok, hint = model.hint_from_samples(samples, wave)
    assert ok and sorted(hint) == list(range(tiles))
    for w in range(tiles // wave):
        assert set(hint[w * wave:(w + 1) * wave]) == set(order[w * wave:(w + 1) * wave].tolist())


def test_hint_vote_rebalances_overfull_waves():
    # every sample puts 5 tiles into wave 0 of size 4: one is moved to wave 1
    samples = torch.tensor([[0, 1, 2, 3, 3, 5, 6, 7]] * 10)
    ok, hint = model.hint_from_samples(samples, 4)
    assert ok and sorted(hint) == list(range(8)) and len(set(hint[:4]) & {0, 1, 2, 3, 4}) == 4


def test_fused_cost_model_orders_regimes():
    # link-bound all-reduce costs more than the compute-bound reduce-scatter of the same output
    ar = model.predict_fused_ms(4096, 8192, 0.05, 8, "all_reduce", 550.0)
    rs = model.predict_fused_ms(4096, 8192, 0.05, 8, "reduce_scatter", 550.0)
    assert ar > rs > 0.05
    assert model.predict_fused_ms(4096, 8192, 0.05, 1, "all_reduce", 550.0) < rs
    # NVLink SHARP moves fewer bytes per direction than two rounds of peer-to-peer stores
    assert model.predict_fused_ms(4096, 8192, 0.05, 8, "all_reduce", 550.0, transport="nvls") < ar
    # a compute-bound problem costs its GEMM plus a tail that grows with the raster group
    big = model.predict_fused_ms(8192, 8192, 0.30, 8, "reduce_scatter", 550.0, raster_group=1)
    assert 0.30 < big < model.predict_fused_ms(8192, 8192, 0.30, 8, "reduce_scatter", 550.0, raster_group=8)


def test_raster_group_sizes_follow_the_kernels_taper():
    assert model.raster_group_sizes(16, 8) == [8, 4, 2, 1, 1]
    assert model.raster_group_sizes(16, 4) == [4, 4, 4, 2, 1, 1]
    assert model.raster_group_sizes(16, 8, taper=False) == [8, 8]
    assert model.raster_group_sizes(5, 2) == [2, 2, 1]          # 5 -> 2, 3 -> 2, 1 -> 1
    assert model.raster_group_sizes(1, 8) == [1]
    for tm in range(1, 40):
        for g in (1, 2, 4, 8, 16):
            assert sum(model.raster_group_sizes(tm, g)) == tm
            assert sum(model.raster_group_sizes(tm, g, taper=False)) == tm


def test_fused_model_queues_rows_behind_slow_row_groups():
    # fast rows: the reduce phase hides under the GEMM, the raster group hardly matters
    fast = [model.predict_fused_ms(4096, 8192, 0.36, 1, "all_reduce", 1.0, raster_group=g, row_us=1.0) for g in (1, 8)]
    assert abs(fast[0] - fast[1]) < 0.01 and 0.36 < fast[0] < 0.40
    # slow rows: a large first group leaves a backlog at the end of the GEMM
    slow = [model.predict_fused_ms(4096, 8192, 0.36, 1, "all_reduce", 1.0, raster_group=g, row_us=30.0) for g in (1, 8)]
    assert slow[1] >= slow[0] > fast[0]
    # never below the time the bytes need on the link
    assert model.predict_fused_ms(4096, 8192, 0.01, 8, "all_reduce", 400.0, transport="nvls", row_us=1.0) >= \
        4096 * 8192 * 2 * 1.125 / 400e9 * 1e3
    # without the taper the last group's rows wait for the last tile
    assert model.predict_fused_ms(4096, 8192, 0.17, 2, "all_reduce", 500.0, raster_group=8, row_us=10.0, taper=False) > \
        model.predict_fused_ms(4096, 8192, 0.17, 2, "all_reduce", 500.0, raster_group=8, row_us=10.0, taper=True)
