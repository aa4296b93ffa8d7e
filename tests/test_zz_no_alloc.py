"""The allocation-free entry point, called through its exported C symbol.

Some callers of the library cannot allocate device memory when they need the
kernel (a server running with a locked memory pool, a plug-in inside a runtime
that owns the heap, a loop where the synchronising cudaMalloc/cudaFree are
banned).  ``fo_gemm_rmsnorm_noalloc`` serves them from a scratch array built
into the library.  The test checks it against the regular entry point
(``OverlapImpl.gemm_rmsnorm``) on two consecutive calls, the second with other
inputs, because all calls share that array and it keeps the previous call's
contents.  It also checks that a problem larger than the array is refused.
This file is collected last so that a failure here cannot hide other tests.
"""
import ctypes

import pytest
import torch

import flashoverlap_b200

pytestmark = pytest.mark.gpu


def _entry():
    lib = ctypes.CDLL(flashoverlap_b200.library_path())
    fn = lib.fo_gemm_rmsnorm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_size_t]
    return fn


def _call(fn, A, B, W, out, eps, status=None):
    err = ctypes.create_string_buffer(256)
    M, K = A.shape
    N = B.shape[0]
    rc = fn(A.data_ptr(), B.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K,
            1 if A.dtype == torch.bfloat16 else 0, eps, torch.cuda.current_stream().cuda_stream,
            status.data_ptr() if status is not None else None, err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_no_alloc_entry_matches_regular_entry_twice(dtype):
    torch.cuda.set_device(0)
    fn = _entry()
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    impl.overlap_init()
    impl.set_timeout_ms(2000)
    eps = 1e-5
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    # two calls in a row: different shapes and data, the second smaller than the first
    for call, (M, N, K) in enumerate([(1024, 2048, 512), (512, 1024, 256)]):
        torch.manual_seed(10 + call)
        A = torch.randn(M, K, device="cuda", dtype=dtype)
        B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dtype)
        W = (1 + 0.1 * torch.randn(N, device="cuda")).to(dtype)
        want_c = torch.empty(M, N, device="cuda", dtype=dtype)
        want = torch.empty(M, N, device="cuda", dtype=dtype)
        impl.gemm_rmsnorm(A, B, want_c, want, W, eps, 0)
        got = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
        before = torch.cuda.memory_allocated()
        rc, msg = _call(fn, A, B, W, got, eps, status)
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == before  # nothing taken from torch's allocator
        torch.cuda.synchronize()
        impl.check_status()
        assert int(status[0]) == 0, f"kernel reported failure code {int(status[0])}"
        assert torch.isfinite(got.float()).all(), f"call {call}: unwritten output"
        tol = 1e-2 if dtype == torch.float16 else 3e-2
        err = (got.float() - want.float()).abs().max().item()
        assert err <= tol * max(1.0, want.float().abs().max().item()), f"call {call}: max abs err {err}"
        # and against plain PyTorch in fp32
        ref = A.float() @ B.float().t()
        ref = ref * torch.rsqrt(ref.pow(2).mean(-1, keepdim=True) + eps) * W.float()
        err32 = (got.float() - ref).abs().max().item()
        assert err32 <= 2 * tol * max(1.0, ref.abs().max().item()), f"call {call}: max abs err vs fp32 {err32}"


def test_no_alloc_entry_rejects_oversized_and_misshapen_problems():
    torch.cuda.set_device(0)
    fn = _entry()
    A = torch.zeros(128, 64, device="cuda", dtype=torch.float16)
    B = torch.zeros(256, 64, device="cuda", dtype=torch.float16)
    W = torch.ones(256, device="cuda", dtype=torch.float16)
    out = torch.empty(128, 256, device="cuda", dtype=torch.float16)
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    # 8192 x 8192 = 64 Mi values: four times the built-in scratch (pointers are not touched)
    rc = fn(A.data_ptr(), B.data_ptr(), W.data_ptr(), out.data_ptr(), 8192, 8192, 64, 0, 1e-5, stream, None, err,
            len(err))
    assert rc != 0 and b"exceeds" in err.value
    rc = fn(A.data_ptr(), B.data_ptr(), W.data_ptr(), out.data_ptr(), 100, 256, 64, 0, 1e-5, stream, None, err,
            len(err))
    assert rc != 0 and b"M % 128" in err.value
    # a misaligned operand is refused before anything is enqueued
    rc = fn(A.data_ptr() + 2, B.data_ptr(), W.data_ptr(), out.data_ptr(), 128, 256, 56, 0, 1e-5, stream, None, err,
            len(err))
    assert rc != 0 and b"aligned" in err.value
    torch.cuda.synchronize()
