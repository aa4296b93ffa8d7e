"""Host-side pieces of the command-line tools: measured peaks, transport
curve bookkeeping and the candidate list of the wave-group search."""
import json
import types

import pytest
import torch

from flashoverlap_b200 import cli
from flashoverlap_b200.tune import bandwidth, runtime
from flashoverlap_b200.utils import config as cfg


def test_measured_peaks_come_from_a_file_not_from_constants(tmp_path, monkeypatch):
    monkeypatch.delenv("FLASHOVERLAP_PEAKS", raising=False)
    f = tmp_path / "peaks.json"
    f.write_text(json.dumps({"bf16_tflops": 1500.0, "hbm_gbs": 6000.0}))
    assert cli.measured_peaks(f)["bf16_tflops"] == 1500.0
    monkeypatch.setenv("FLASHOVERLAP_PEAKS", str(f))
    assert cli.measured_peaks()["hbm_gbs"] == 6000.0
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    monkeypatch.setenv("FLASHOVERLAP_PEAKS", str(bad))
    assert isinstance(cli.measured_peaks(bad), dict)  # unreadable file: falls through, never raises


def test_measured_link_bandwidth_is_the_best_transport_curve(tmp_path):
    assert cli.measured_link_gbs(8, path=tmp_path) == (None, "")
    cfg.save_bandwidth(torch.tensor([[1e6, 300.0], [3e7, 540.0]]), "p2p_push", 8, path=tmp_path)
    cfg.save_bandwidth(torch.tensor([[1e6, 310.0], [3e7, 600.0]]), "p2p_push_bulk", 8, path=tmp_path)
    gbs, src = cli.measured_link_gbs(8, path=tmp_path)
    assert gbs == 600.0 and src == "p2p_push_bulk"


def test_link_bytes_per_direction():
    S, n = 64.0, 8
    assert bandwidth.link_bytes_per_direction("p2p_push", S, n) == S
    assert bandwidth.link_bytes_per_direction("multimem_ld_reduce", S, n) == S
    assert bandwidth.link_bytes_per_direction("multimem_allreduce", S, n) == pytest.approx(S * 1.125)
    assert bandwidth.link_bytes_per_direction("multimem_st", S, 1) == 0.0
    with pytest.raises(ValueError):
        bandwidth.link_bytes_per_direction("all_reduce", S, n)


def test_curve_table_is_readable_text():
    text = bandwidth.curve_table(torch.tensor([[1048576.0, 100.0], [2097152.0, 150.5]]), "p2p_push", 4)
    lines = text.strip().splitlines()
    assert lines[0].startswith("# p2p_push, 4 ranks") and lines[1].split() == ["2.00", "100.0"]


def test_wave_units_fold_to_at_most_ten():
    assert runtime.wave_units(512, 66, 10) == (8, 66)
    units, per = runtime.wave_units(4096, 66, 10)
    assert units <= 10 and per % 66 == 0 and units * per >= 4096


@pytest.fixture
def fake_gpu(monkeypatch):
    timed = []

    def perf_running(impl, M, N, K, BM, BN, algo, cseg, hint, comm_op, dtype=None, warmup=0, reps=0, raster_group=0,
                     two_stream=False, gemm_ctas=0):
        assert two_stream
        timed.append(list(cseg))
        return 1.0 + 0.1 * abs(len(cseg) - 2)

    monkeypatch.setattr(runtime, "perf_running", perf_running)
    monkeypatch.setattr(runtime, "world", lambda: (0, 8))
    monkeypatch.setattr(torch.cuda, "get_device_properties",
                        lambda *a, **k: types.SimpleNamespace(multi_processor_count=148))
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    return timed


def test_two_stream_search_times_every_composition(fake_gpu):
    cseg, ms, timed = runtime.search_two_stream(None, 4096, 8192, 1024, 3, "all_reduce", max_units=4)
    tiles = 16 * 32
    assert all(sum(g) == tiles and all(x > 0 for x in g) for g, _ in timed)
    assert [tiles] in [g for g, _ in timed]          # "no overlap" is always a candidate
    assert len(timed) == len(fake_gpu) >= 8          # 2**(4-1) compositions of four units
    assert len(cseg) == 2 and ms == 1.0              # the fake's optimum


def test_two_stream_search_predictive_times_only_its_picks(fake_gpu):
    curve = torch.tensor([[2.0 ** 20, 100.0], [2.0 ** 26, 400.0]])
    cseg, ms, timed = runtime.search_two_stream(None, 4096, 8192, 1024, 3, "all_reduce", curve=curve, gemm_ms=0.055,
                                                top_k=1)
    assert len(timed) == 1 and len(fake_gpu) == 1


def test_reduce_scatter_candidates_keep_rank_blocks_whole(fake_gpu):
    _, _, timed = runtime.search_two_stream(None, 4096, 8192, 1024, 3, "reduce_scatter", max_units=4)
    assert all((x * 256) % 8 == 0 for g, _ in timed for x in g)


def test_clock_sampler_with_a_fake_nvml(monkeypatch):
    """The sampler reads clocks, power and throttle reasons through NVML and never sets anything; a region
    that is over before the polling thread wakes up still gets the sample taken at its end."""
    import sys
    import types

    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    fake.nvmlDeviceGetClockInfo = lambda h, k: 1400
    fake.nvmlDeviceGetPowerUsage = lambda h: 950_000
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    from flashoverlap_b200.utils.clocks import ClockSampler

    with ClockSampler(0, period_ms=1000.0) as s:
        pass  # an empty region
    out = s.summary()
    assert out["samples"] >= 1 and out["sm_mhz"] == 1400 and out["sm_max_mhz"] == 1965
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 950.0
    assert not any(name.startswith("nvmlDeviceSet") for name in dir(fake))


def test_fused_layer_runs_the_searched_configuration():
    """FusedRowParallelLinear.from_config hands the tuner's Algo and raster group to the kernel call."""
    import torch

    from flashoverlap_b200.models import FusedRowParallelLinear

    class FakeImpl:
        def __init__(self):
            self.calls = []

        def set_raster_group(self, g):
            self.calls.append(("raster", g))

        def gemm_allreduce_fused(self, x, w, gamma, eps, algo):
            self.calls.append(("ar", algo, gamma is not None))
            return torch.zeros(x.size(0), w.size(0))

        def gemm_reducescatter_fused(self, x, w, out, gamma, eps, algo, interleave):
            self.calls.append(("rs", algo, interleave))

    impl = FakeImpl()
    cfg_ar = {"Algo": 8, "raster_group": 4, "comm_op": "all_reduce"}
    layer = FusedRowParallelLinear.from_config(impl, cfg_ar, 64, 128, norm=True, device="cpu")
    y = layer(torch.zeros(256, 64, dtype=torch.float16))
    assert y.shape == (256, 128)
    assert impl.calls == [("raster", 4), ("ar", 8, True), ("raster", 0)]   # set for the call, then back to the default
    impl.calls.clear()
    layer = FusedRowParallelLinear.from_config(impl, {"Algo": 3, "comm_op": "reduce_scatter"}, 64, 128, device="cpu")
    out = layer(torch.zeros(256, 64, dtype=torch.float16))
    assert out.shape == (256, 128) and impl.calls == [("rs", 3, False)]    # no raster group in the file: untouched
