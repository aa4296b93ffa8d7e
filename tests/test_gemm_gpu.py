"""Numerics of the sm_100a GEMM kernel against a plain PyTorch fp32 reference."""
import pytest
import torch

import flashoverlap_b200  # noqa: F401  (registers the classes)
from flashoverlap_b200.utils.config import ALGO_TILES

ALGOS = list(range(len(ALGO_TILES)))

pytestmark = pytest.mark.gpu


def _impl():
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.cutlass_init()
    impl.set_timeout_ms(2000)
    return impl


def _ref(A, B):
    return A.float() @ B.float().t()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (512, 1024, 1000), (1024, 2048, 4096)])
def test_gemm_matches_fp32_reference(dtype, algo, shape):
    M, N, K = shape
    K = (K + 7) // 8 * 8
    if M % ALGO_TILES[algo][0] or N % ALGO_TILES[algo][1]:
        pytest.skip("shape is not a multiple of this tile")
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=dtype)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dtype)
    C = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
    impl = _impl()
    impl.cutlass_gemm(A, B, C, algo)
    torch.cuda.synchronize()
    impl.check_status()
    ref = _ref(A, B)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.isfinite(C.float()).all(), "unwritten or non-finite output"
    err = (C.float() - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), f"max abs err {err}"


def test_gemm_many_tiles_persistent_loop():
    # more tiles than SMs: every CTA walks several tiles and both TMEM buffers
    M, N, K = 4096, 4096, 512
    torch.manual_seed(1)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    impl = _impl()
    for algo in ALGOS:
        C.fill_(float("nan"))
        impl.cutlass_gemm(A, B, C, algo)
        torch.cuda.synchronize()
        impl.check_status()
        ref = _ref(A, B)
        err = (C.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), f"algo {algo}: max abs err {err}"


def test_gemm_repeated_calls_are_deterministic():
    M, N, K = 1024, 1024, 1024
    A = torch.randn(M, K, device="cuda", dtype=torch.float16)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).half()
    impl = _impl()
    outs = []
    for _ in range(3):
        C = torch.empty(M, N, device="cuda", dtype=torch.float16)
        impl.cutlass_gemm(A, B, C, 0)
        outs.append(C)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


def test_gemm_rejects_bad_shapes():
    impl = _impl()
    A = torch.randn(100, 64, device="cuda", dtype=torch.float16)
    B = torch.randn(256, 64, device="cuda", dtype=torch.float16)
    C = torch.empty(100, 256, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError):
        impl.cutlass_gemm(A, B, C, 0)
    with pytest.raises(RuntimeError):
        impl.cutlass_gemm(A.float(), B.float(), C.float(), 0)


def test_algo_table_matches_generated_python_copy():
    impl = _impl()
    assert impl.num_algos() == len(ALGO_TILES)
    assert [tuple(impl.algo_tile(a)) for a in ALGOS] == [tuple(t) for t in ALGO_TILES]
