"""The fused kernel's reduce phase on one GPU (world size 1): GEMM + RMSNorm,
all-reduce / reduce-scatter entry points degenerate to a local reduction, the
reference-compatible reordered layout, the completion trace and RMSNorm ops.
Oracle: PyTorch fp32."""
import pytest
import torch

import flashoverlap_b200  # noqa: F401
from flashoverlap_b200.utils.config import ALGO_TILES
from flashoverlap_b200.utils.reorder import from_tile_order, reorder_indices, to_tile_order

pytestmark = pytest.mark.gpu


def rms_ref(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def make_impl():
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    impl.overlap_init()
    impl.set_timeout_ms(2000)
    return impl


def make_inputs(M, N, K, dtype, seed=0):
    torch.manual_seed(seed)
    A = torch.randn(M, K, device="cuda", dtype=dtype)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dtype)
    W = (1 + 0.1 * torch.randn(N, device="cuda")).to(dtype)
    return A, B, W


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("algo", list(range(len(ALGO_TILES))))
def test_gemm_rmsnorm_single_kernel(dtype, algo):
    M, N, K = 1024, 4096, 512
    A, B, W = make_inputs(M, N, K, dtype)
    C = torch.empty(M, N, device="cuda", dtype=dtype)
    O = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
    impl = make_impl()
    impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, algo)
    torch.cuda.synchronize()
    impl.check_status()
    ref = A.float() @ B.float().t()
    tol = 1e-2 if dtype == torch.float16 else 3e-2
    assert (C.float() - ref).abs().max().item() <= tol * ref.abs().max().item()
    want = rms_ref(C, W, 1e-5)  # the kernel normalises the 16-bit product it stored
    assert torch.isfinite(O.float()).all()
    assert (O.float() - want).abs().max().item() <= tol * want.abs().max().item()


@pytest.mark.parametrize("N", [512, 2304, 8192, 16384, 16640])
def test_gemm_rmsnorm_row_widths(N):
    # rows that fill a fraction of the row group's registers (512), that end inside a
    # warp's chunk range (2304), that fill them exactly (8192), and wide rows
    # that take the two-pass path (16384, 16640)
    M, K = 256, 128
    A, B, W = make_inputs(M, N, K, torch.float16, seed=N)
    C = torch.empty(M, N, device="cuda", dtype=torch.float16)
    O = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    impl = make_impl()
    impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, 0)
    torch.cuda.synchronize()
    impl.check_status()
    want = rms_ref(C, W, 1e-5)
    assert torch.isfinite(O.float()).all()
    assert (O.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_gemm_rmsnorm_more_rows_than_one_wave():
    # 8192 rows: every row group takes many rows; the GEMM warps join the reduce phase
    M, N, K = 8192, 2048, 256
    A, B, W = make_inputs(M, N, K, torch.bfloat16, seed=21)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    O = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    impl = make_impl()
    for _ in range(2):
        impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, 3)
    torch.cuda.synchronize()
    impl.check_status()
    want = rms_ref(C, W, 1e-5)
    assert torch.isfinite(O.float()).all()
    assert (O.float() - want).abs().max().item() <= 3e-2 * want.abs().max().item()


def test_phase_trace_records_every_row_once():
    M, N, K = 2048, 2048, 256
    A, B, W = make_inputs(M, N, K, torch.float16, seed=4)
    C = torch.empty(M, N, device="cuda", dtype=torch.float16)
    O = torch.empty(M, N, device="cuda", dtype=torch.float16)
    impl = make_impl()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    trace = torch.zeros(8 * sms, dtype=torch.int64, device="cuda")
    impl.set_phase_trace(trace)
    impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, 0)
    torch.cuda.synchronize()
    impl.set_phase_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
    t = trace.view(sms, 8).cpu()
    assert int(t[:, 5].sum()) == M            # rows reduced, over all CTAs
    assert int(t[:, 3].sum()) == (M // 128) * (N // 256)  # tiles computed
    assert bool((t[:, 1] >= t[:, 0]).all())   # GEMM phase ends after the start


def test_row_trace_has_ordered_stamps_for_every_row():
    M, N, K = 1024, 2048, 256
    A, B, W = make_inputs(M, N, K, torch.float16, seed=5)
    C = torch.empty(M, N, device="cuda", dtype=torch.float16)
    O = torch.empty(M, N, device="cuda", dtype=torch.float16)
    impl = make_impl()
    rows = torch.zeros(6 * M, dtype=torch.int64, device="cuda")
    impl.set_row_trace(rows)
    impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, 0)
    torch.cuda.synchronize()
    impl.set_row_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
    impl.check_status()
    r = rows.view(6, M).cpu()
    claimed, stored, who, ready, summed, barrier = r[0], r[1], r[2], r[3], r[4], r[5]
    assert bool((claimed > 0).all())                       # every row was reduced by somebody
    assert bool((claimed <= ready).all() and (ready <= summed).all() and (summed <= barrier).all()
                and (barrier <= stored).all())
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert int(who.max()) < 4 * sms and int((who % 4).max()) <= 2   # CTA * 4 + row group (0..2)
    want = rms_ref(A.float() @ B.float().t(), W, 1e-5)
    assert (O.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()
    with pytest.raises(RuntimeError):
        impl.set_row_trace(torch.zeros(7, dtype=torch.int64, device="cuda"))  # not a multiple of 6
    # a buffer that is too small for the next call is ignored rather than overrun
    impl.set_row_trace(torch.zeros(6 * 128, dtype=torch.int64, device="cuda"))
    impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, 0)
    torch.cuda.synchronize()
    impl.set_row_trace(torch.empty(0, dtype=torch.int64, device="cuda"))
    impl.check_status()


@pytest.mark.parametrize("with_norm", [False, True])
def test_world1_allreduce_and_reducescatter(with_norm):
    M, N, K = 512, 2048, 256
    A, B, W = make_inputs(M, N, K, torch.float16, seed=3)
    impl = make_impl()
    ref = A.float() @ B.float().t()
    want = rms_ref(ref, W, 1e-5) if with_norm else ref
    for _ in range(3):  # repeated calls alternate between the two buffer sets
        out = impl.gemm_allreduce_fused(A, B, W if with_norm else None, 1e-5, 0)
        torch.cuda.synchronize()
        impl.check_status()
        assert (out.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()
    D = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    impl.gemm_reducescatter_fused(A, B, D, W if with_norm else None, 1e-5, 1, False)
    torch.cuda.synchronize()
    impl.check_status()
    assert (D.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_compat_overlap_api_reordered_layout_and_trace():
    M, N, K, algo = 1024, 2048, 256, 0
    A, B, W = make_inputs(M, N, K, torch.float16, seed=5)
    impl = make_impl()
    bm, bn, _ = impl.algo_tile(algo)
    tm, tn = M // bm, N // bn
    tiles = tm * tn
    hint = [(7 * i + 3) % tiles for i in range(tiles)]  # a permutation since gcd(7, 64) = 1
    RA = reorder_indices(tiles, hint, device="cuda").reshape(tm, tn)
    cseg_cpu = torch.tensor([16, 16, 32], dtype=torch.int32)
    cseg_gpu = cseg_cpu.cuda()
    MM = torch.zeros((tm + 1, tn), dtype=torch.int32, device="cuda")
    C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, True)
    torch.cuda.synchronize()
    impl.check_status()
    ref = A.float() @ B.float().t()
    got = from_tile_order(C, bm, bn, RA)
    assert (got.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
    # oracle for the layout itself
    assert torch.equal(to_tile_order(got, bm, bn, RA), C)
    flat = MM.flatten().cpu()
    assert int(flat[tn - 1]) == tiles  # ticket counter
    assert torch.equal(flat[tn:tn + tiles].sort().values, torch.arange(tiles, dtype=torch.int32))
    assert int(flat[:tn - 1].abs().sum()) == 0  # segment counters end at zero
    # reorder_rmsnorm undoes the layout
    out = torch.empty_like(C)
    torch.ops.flashoverlap_op.reorder_rmsnorm(C, out, W, bm, bn, 1, RA)
    torch.cuda.synchronize()
    want = rms_ref(got, W, 1e-5)
    assert (out.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_index_arrays_are_checked_on_the_host_before_any_launch():
    M, N, K, algo = 256, 512, 64, 0
    A, B, W = make_inputs(M, N, K, torch.float16)
    impl = make_impl()
    MM = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    C = torch.empty(M, N, device="cuda", dtype=torch.float16)
    cseg = torch.tensor([4], dtype=torch.int32)
    out_of_range = torch.tensor([[0, 1], [2, 400]], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="outside"):
        impl.gemm_allreduce_overlap(A, B, C, MM, out_of_range, 1, cseg, cseg.cuda(), algo, False)
    duplicate = torch.tensor([[0, 1], [1, 3]], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="permutation"):
        impl.gemm_allreduce_overlap(A, B, C, MM, duplicate, 1, cseg, cseg.cuda(), algo, False)
    with pytest.raises(RuntimeError, match="outside"):
        torch.ops.flashoverlap_op.reorder_rmsnorm(C, torch.empty_like(C), W, 128, 256, 1, out_of_range)
    # a tensor that passed the check is checked again after it has been written to
    RA = reorder_indices(4, [], device="cuda").reshape(2, 2)
    impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg, cseg.cuda(), algo, False)
    RA[1, 1] = 77
    with pytest.raises(RuntimeError, match="outside"):
        impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg, cseg.cuda(), algo, False)
    torch.cuda.synchronize()
    impl.check_status()


def test_compat_overlap_api_rejects_bad_segments():
    M, N, K, algo = 256, 512, 64, 0
    A, B, _ = make_inputs(M, N, K, torch.float16)
    impl = make_impl()
    RA = reorder_indices(4, [], device="cuda").reshape(2, 2)
    MM = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    C = torch.empty(M, N, device="cuda", dtype=torch.float16)
    bad = torch.tensor([1, 1], dtype=torch.int32)  # sums to 2, not 4: the reference would spin forever
    with pytest.raises(RuntimeError, match="sum"):
        impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, bad, bad.cuda(), algo, False)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dim", [512, 4096, 8192, 16384, 32768, 1000 * 8])
def test_rmsnorm_op(dtype, dim):
    torch.manual_seed(0)
    x = torch.randn(37, dim, device="cuda", dtype=dtype)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(dtype)
    o = torch.empty_like(x)
    torch.ops.flashoverlap_op.rmsnorm(x, o, w, 1e-6)
    torch.cuda.synchronize()
    want = rms_ref(x, w, 1e-6)
    tol = 1e-2 if dtype == torch.float16 else 3e-2
    assert (o.float() - want).abs().max().item() <= tol * want.abs().max().item()


def test_reorder_rmsnorm_rldn2():
    M, N, bm, bn = 512, 1024, 128, 256
    tm, tn = M // bm, N // bn
    torch.manual_seed(1)
    x = torch.randn(M, N, device="cuda", dtype=torch.float16)
    w = (1 + 0.1 * torch.randn(N, device="cuda")).half()
    RA = reorder_indices(tm * tn, [5, 1, 9, 0], device="cuda").reshape(tm, tn)
    for rldn in (1, 2, 4):
        xr = to_tile_order(x, bm, bn, RA, rldn)
        o = torch.empty_like(x)
        torch.ops.flashoverlap_op.reorder_rmsnorm(xr, o, w, bm, bn, rldn, RA)
        torch.cuda.synchronize()
        want = rms_ref(x, w, 1e-5)
        assert (o.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item(), f"rldn={rldn}"


def test_allgather_gemm_world1():
    M, N, K = 512, 1024, 256
    A, B, _ = make_inputs(M, N, K, torch.bfloat16, seed=8)
    impl = make_impl()
    C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    for algo in (0, 3):
        impl.allgather_gemm(A, B, C, algo)
        torch.cuda.synchronize()
        impl.check_status()
        ref = A.float() @ B.float().t()
        assert (C.float() - ref).abs().max().item() <= 3e-2 * ref.abs().max().item()


def test_a2a_dispatch_gemm_world1():
    K, N = 128, 256
    impl = make_impl()
    mlen = torch.tensor([[300]], dtype=torch.int32)
    A = torch.randn(300, K, device="cuda", dtype=torch.float16)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).half()
    m_pad = impl.a2a_padded_rows(mlen, 0)
    assert m_pad == 384
    C = torch.empty(m_pad, N, device="cuda", dtype=torch.float16)
    impl.a2a_dispatch_gemm(A, B, C, mlen, 0)
    torch.cuda.synchronize()
    impl.check_status()
    ref = A.float() @ B.float().t()
    assert (C[:300].float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
    with pytest.raises(RuntimeError):
        impl.a2a_dispatch_gemm(A[:100], B, C, mlen, 0)  # fewer rows than mLen says
    # whole tiles on one rank: the GEMM reads the caller's rows in place
    mlen2 = torch.tensor([[384]], dtype=torch.int32)
    A2 = torch.randn(384, K, device="cuda", dtype=torch.float16)
    C.fill_(float("nan"))
    impl.a2a_dispatch_gemm(A2, B, C, mlen2, 0)
    torch.cuda.synchronize()
    impl.check_status()
    ref2 = A2.float() @ B.float().t()
    assert (C.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item()


def test_host_feeder_double_buffers_inputs():
    from flashoverlap_b200.utils.pipeline import HostFeeder

    feeder = HostFeeder((64, 32), torch.float16)
    batches = [torch.full((64, 32), float(i), dtype=torch.float16).pin_memory() for i in range(5)]
    feeder.submit(batches[0])
    seen = []
    for i in range(1, 6):
        x = feeder.take()
        if i < 5:
            feeder.submit(batches[i])
        y = x.float().mean()  # stands for the step's compute
        feeder.release(x)
        seen.append(y)
    torch.cuda.synchronize()
    assert [float(v) for v in seen] == [0.0, 1.0, 2.0, 3.0, 4.0]
