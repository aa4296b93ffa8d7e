"""The tuning pipeline end to end on one GPU (world size 1): tile profiling,
bandwidth-curve file, completion-order hint, predictive and exhaustive search,
stage-2 file consumed by the reference-compatible layer."""
import pytest
import torch

import flashoverlap_b200  # noqa: F401
from flashoverlap_b200.models import OverlapRowParallelLayer, ReorderRMSNorm
from flashoverlap_b200.parallel import make_overlap_impl
from flashoverlap_b200.tune import search
from flashoverlap_b200.tune.runtime import compute_hint, profile_gemm
from flashoverlap_b200.utils import config as cfg

pytestmark = pytest.mark.gpu


def tiles_of(data, M, N):
    return (M // data["BM"]) * (N // data["BN"])


def test_profile_hint_search_and_use(tmp_path):
    M, N, K = 1024, 2048, 256
    impl = make_overlap_impl(timeout_ms=3000)
    BM, BN, dur, algo = profile_gemm(impl, M, N, K, torch.float16, warmup=2, reps=5)
    assert len(algo) == min(10, len(cfg.ALGO_TILES)) and dur == sorted(dur) and all(d > 0 for d in dur)
    cfg.save_stage1(M, N, K, BM, BN, dur, algo, tmp_path)

    tiles = (M // BM[0]) * (N // BN[0])
    ok, hint = compute_hint(impl, M, N, K, BM[0], BN[0], algo[0], 148 // (BM[0] // 128), "all_reduce",
                            warmup=2, samples=6)
    assert ok and sorted(hint) == list(range(tiles))

    curve = torch.tensor([[2.0 ** 20, 200.0], [2.0 ** 26, 400.0]])
    cfg.save_bandwidth(curve, "all_reduce", 1, path=tmp_path)
    sol = search.predictive_search(impl, M, N, K, "all_reduce", cfg.load_bandwidth("all_reduce", 1, path=tmp_path),
                                   path=tmp_path, reps=5, verbose=False)
    data = cfg.load_config(M, N, K, tmp_path)
    cfg.validate_stage2(data, M, N)
    assert data["Algo"] == sol["Algo"] and data["search"] == "predictive" and data["fused_dur"] > 0
    assert sum(data["cSeg"]) == tiles_of(data, M, N) and data["two_stream_dur"] > 0 and data["candidates_timed"] >= 1

    # exhaustive search on the same stage-1 lists: every candidate is timed, the file is rewritten
    ex = search.exhaustive_search(impl, M, N, K, "all_reduce", path=tmp_path, reps=3, verbose=False, seg_reps=3)
    data = cfg.load_config(M, N, K, tmp_path)
    cfg.validate_stage2(data, M, N)
    assert data["search"] == "exhaustive" and data["Algo"] == ex["Algo"]

    # the tuned file drives the reference-compatible layer + reorder-aware RMSNorm
    layer = OverlapRowParallelLayer(0, 1, K, N, M, data, "all_reduce", [0] * 16)
    norm = ReorderRMSNorm(N, M, data["BM"], data["BN"], data["hint"], eps=1e-5)
    with torch.no_grad():
        layer.weight.normal_(0.0, 1.0 / K ** 0.5)
        norm.weight.fill_(1.0)
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        y = norm(layer(x))
    torch.cuda.synchronize()
    layer.overlap_class.check_status()
    ref = x.float() @ layer.weight.float().t()
    ref = ref * torch.rsqrt(ref.pow(2).mean(-1, keepdim=True) + 1e-5)
    assert (y.float() - ref).abs().max().item() < 2e-2
    impl.check_status()


def test_measured_row_time_is_sane():
    from flashoverlap_b200.tune.runtime import gather_algo_candidates, measure_row_us, pick_algo_by_timing

    impl = make_overlap_impl(timeout_ms=3000)
    row_ar = measure_row_us(impl, 2048, "all_reduce", torch.float16, reps=3)
    row_rs = measure_row_us(impl, 2048, "reduce_scatter", torch.bfloat16, reps=3)
    assert 0.05 < row_ar < 200.0 and 0.05 < row_rs < 200.0   # microseconds per row and row group
    impl.check_status()
    # the timed tile pick returns one of its candidates and a time for each
    A = torch.randn(1024, 256, device="cuda", dtype=torch.float16)
    B = torch.randn(2048, 256, device="cuda", dtype=torch.float16)
    C = torch.empty(1024, 2048, device="cuda", dtype=torch.float16)
    cands = gather_algo_candidates(1024, 2048)[:3]
    best, timed = pick_algo_by_timing(lambda a: impl.allgather_gemm(A, B, C, a), cands, warmup=1, reps=2)
    assert best in cands and [a for a, _ in timed] == cands and all(t > 0 for _, t in timed)
    impl.check_status()
