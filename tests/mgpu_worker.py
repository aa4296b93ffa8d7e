"""Multi-GPU correctness worker, launched by torchrun from test_multigpu.py.

Each check compares a fused operation with the PyTorch semantics it replaces
(matmul + all_reduce / reduce_scatter_tensor + RMSNorm in fp32).
Prints one line per check and exits non-zero on the first failure.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import flashoverlap_b200  # noqa: F401
from flashoverlap_b200.parallel import init_distributed, make_baseline_impl, make_overlap_impl
from flashoverlap_b200.utils.reorder import from_tile_order, generate_row_mapping, reorder_indices


def rms_ref(x, w, eps):
    x = x.float()
    y = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
    return y * w.float()


def main():
    rank, world, _ = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    impl = make_overlap_impl(timeout_ms=4000, max_m=4096, max_n=4096)
    if impl.nvls_available():
        impl.set_use_nvls(True, False)  # exercise the multimem path at every group size
    if rank == 0:
        print(f"mode: {'NVLS multimem' if impl.allreduce_uses_nvls() else 'P2P stores'}", flush=True)
    failures = 0

    def check(name, got, want, tol):
        nonlocal failures
        got = got.float()
        bad = not torch.isfinite(got).all().item()
        err = (got - want).abs().max().item() if not bad else float("inf")
        scale = max(1.0, want.abs().max().item())
        ok = (not bad) and err <= tol * scale
        flag = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(flag)
        if rank == 0:
            print(f"{'PASS' if flag.item() == 0 else 'FAIL'} {name}: rank0 max err {err:.4g} (scale {scale:.3g})",
                  flush=True)
        st = impl.status()
        if st[0] != 0:  # a wait inside a kernel ran out: a failure even if the numbers came out right
            print(f"rank {rank} status: {impl.status_string()}", flush=True)
            failures += 1
        if flag.item() != 0:
            failures += 1
            if os.environ.get("FO_FAIL_FAST"):
                sys.exit(1)

    def inputs(M, N, K, dtype, seed):
        g = torch.Generator(device="cpu").manual_seed(1000 * seed + rank)
        A = torch.randn(M, K, generator=g).to(dev, dtype)
        B = (torch.randn(N, K, generator=g) / K ** 0.5).to(dev, dtype)
        gw = torch.Generator(device="cpu").manual_seed(77 + seed)
        W = (1 + 0.1 * torch.randn(N, generator=gw)).to(dev, dtype)
        return A, B, W

    def full_sum(A, B):
        part = (A.float() @ B.float().t())
        dist.all_reduce(part)
        return part

    shapes = [(256 * world, 512, 128), (1024, 2048, 512), (2048, 4096, 1024)]
    for dtype in (torch.float16, torch.bfloat16):
        tol = 1e-2 if dtype == torch.float16 else 3e-2
        for i, (M, N, K) in enumerate(shapes):
            for algo in (0, 1, 3):
                if algo == 3 and (M // world) % 256:
                    continue
                A, B, W = inputs(M, N, K, dtype, i)
                ref = full_sum(A, B)
                tag = f"{str(dtype)[6:]} M{M} N{N} K{K} algo{algo}"
                # all-reduce
                out = impl.gemm_allreduce_fused(A, B, None, 0.0, algo)
                torch.cuda.synchronize()
                check(f"gemm+AR {tag}", out, ref, tol)
                # all-reduce + RMSNorm
                out = impl.gemm_allreduce_fused(A, B, W, 1e-5, algo)
                torch.cuda.synchronize()
                check(f"gemm+AR+norm {tag}", out, rms_ref(ref, W, 1e-5), tol)
                # reduce-scatter, contiguous rows
                rows = M // world
                if rows % 128 == 0:
                    D = torch.full((rows, N), float("nan"), device=dev, dtype=dtype)
                    impl.gemm_reducescatter_fused(A, B, D, None, 0.0, algo, False)
                    torch.cuda.synchronize()
                    check(f"gemm+RS(block) {tag}", D, ref[rank * rows:(rank + 1) * rows], tol)
                    impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, algo, False)
                    torch.cuda.synchronize()
                    check(f"gemm+RS(block)+norm {tag}", D, rms_ref(ref[rank * rows:(rank + 1) * rows], W, 1e-5), tol)
                # reduce-scatter, interleaved rows
                D = torch.full((rows, N), float("nan"), device=dev, dtype=dtype)
                impl.gemm_reducescatter_fused(A, B, D, W, 1e-5, algo, True)
                torch.cuda.synchronize()
                check(f"gemm+RS(interleave)+norm {tag}", D, rms_ref(ref[rank::world], W, 1e-5), tol)

    # all-gather -> GEMM: every rank contributes M/world rows of A, computes all M rows of the product
    for dtype in (torch.float16, torch.bfloat16):
        for algo in (0, 3):
            M, N, K = 256 * world, 512, 384
            g = torch.Generator(device="cpu").manual_seed(4242)
            A_full = torch.randn(M, K, generator=g).to(dev, dtype)
            g2 = torch.Generator(device="cpu").manual_seed(5000 + rank)
            Bn = (torch.randn(N, K, generator=g2) / K ** 0.5).to(dev, dtype)
            rows = M // world
            C = torch.full((M, N), float("nan"), device=dev, dtype=dtype)
            for rep in range(3):  # repeated calls alternate the gathered-A buffers
                impl.allgather_gemm(A_full[rank * rows:(rank + 1) * rows].contiguous(), Bn, C, algo)
            torch.cuda.synchronize()
            check(f"allgather+gemm {str(dtype)[6:]} algo{algo}", C, A_full.float() @ Bn.float().t(),
                  1e-2 if dtype == torch.float16 else 3e-2)

    # all-to-all dispatch -> GEMM: uneven row counts, some of them zero
    gm = torch.Generator(device="cpu").manual_seed(99)
    mlen = torch.randint(0, 300, (world, world), generator=gm, dtype=torch.int32)
    mlen[0, world - 1] = 0
    mlen[world - 1, world - 1] = 0
    K, N = 256, 512
    sends = []
    for i in range(world):
        gi = torch.Generator(device="cpu").manual_seed(700 + i)
        sends.append(torch.randn(int(mlen[i].sum()), K, generator=gi))
    gb = torch.Generator(device="cpu").manual_seed(800 + rank)
    Bn = (torch.randn(N, K, generator=gb) / K ** 0.5).to(dev, torch.float16)
    recv = []
    for i in range(world):
        off = int(mlen[i, :rank].sum())
        recv.append(sends[i][off:off + int(mlen[i, rank])])
    recv = torch.cat(recv).to(dev, torch.float16)
    for algo in (0, 3):
        m_pad = impl.a2a_padded_rows(mlen, algo)
        C = torch.full((m_pad, N), float("nan"), device=dev, dtype=torch.float16)
        for rep in range(2):
            impl.a2a_dispatch_gemm(sends[rank].to(dev, torch.float16), Bn, C, mlen, algo)
        torch.cuda.synchronize()
        # (every rank takes part in the check, also one that received no rows)
        n = recv.shape[0]
        got = C[:n] if n > 0 else torch.zeros(1, N, device=dev)
        want = recv.float() @ Bn.float().t() if n > 0 else torch.zeros(1, N, device=dev)
        check(f"a2a dispatch+gemm algo{algo} ({n} rows on rank {rank})", got, want, 1e-2)

    # back-to-back calls without host synchronisation (exercises both buffer sets)
    A, B, W = inputs(1024, 2048, 512, torch.float16, 9)
    ref = full_sum(A, B)
    outs = []
    for it in range(6):
        o = impl.gemm_allreduce_fused(A, B, W, 1e-5, 0)
        outs.append(o.clone())
    torch.cuda.synchronize()
    for it, o in enumerate(outs):
        check(f"back-to-back AR+norm call {it}", o, rms_ref(ref, W, 1e-5), 1e-2)

    # reference-compatible overlap API: reordered all-reduce + reorder_rmsnorm
    M, N, K, algo = 1024, 2048, 512, 0
    bm, bn, _ = impl.algo_tile(algo)
    tm, tn = M // bm, N // bn
    A, B, W = inputs(M, N, K, torch.float16, 11)
    ref = full_sum(A, B)
    hint = list(reversed(range(tm * tn)))
    RA = reorder_indices(tm * tn, hint, device=dev).reshape(tm, tn)
    cseg = [tm * tn // 2, tm * tn - tm * tn // 2]
    cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
    cseg_gpu = cseg_cpu.to(dev)
    MM = torch.zeros((tm + 1, tn), dtype=torch.int32, device=dev)
    C = torch.full((M, N), float("nan"), device=dev, dtype=torch.float16)
    impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, True)
    torch.cuda.synchronize()
    check("compat gemm_allreduce_overlap (reordered)", from_tile_order(C, bm, bn, RA), ref, 1e-2)
    tickets = MM.flatten()[tn:tn + tm * tn].sort().values.cpu()
    ok = torch.equal(tickets, torch.arange(tm * tn, dtype=torch.int32)) and int(MM.flatten()[tn - 1]) == tm * tn
    if rank == 0:
        print(f"{'PASS' if ok else 'FAIL'} monitor trace is a permutation of 0..tiles-1", flush=True)
    failures += 0 if ok else 1
    out = torch.empty_like(C)
    torch.ops.flashoverlap_op.reorder_rmsnorm(C, out, W, bm, bn, 1, RA)
    torch.cuda.synchronize()
    check("compat reorder_rmsnorm after overlap AR", out, rms_ref(ref, W, 1e-5), 1e-2)

    # reference-compatible reduce-scatter: interleaved rows, tiles of BM/world rows
    RE = generate_row_mapping(M, N, bm, bn, cseg, world, device=dev)
    MM.zero_()
    Ctmp = torch.empty((M, N), device=dev, dtype=torch.float16)
    D = torch.full((M // world, N), float("nan"), device=dev, dtype=torch.float16)
    impl.gemm_reducescatter_overlap(A, B, Ctmp, D, MM, RA, RE, 1, cseg_cpu, cseg_gpu, algo, False)
    torch.cuda.synchronize()
    check("compat gemm_reducescatter_overlap", from_tile_order(D, bm // world, bn, RA), ref[rank::world], 5e-2)

    # the reference's two-stream design (comparator): signalling GEMM + stream waits + segmented NCCL
    MM.zero_()
    C = torch.full((M, N), float("nan"), device=dev, dtype=torch.float16)
    for rep in range(2):
        impl.gemm_allreduce_twostream(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, 0)
    torch.cuda.synchronize()
    check("two-stream comparator all-reduce (reordered)", from_tile_order(C, bm, bn, RA), ref, 1e-2)
    D = torch.full((M // world, N), float("nan"), device=dev, dtype=torch.float16)
    for rep in range(2):
        impl.gemm_reducescatter_twostream(A, B, Ctmp, D, MM, RA, RE, 1, cseg_cpu, cseg_gpu, algo, 0)
    torch.cuda.synchronize()
    check("two-stream comparator reduce-scatter", from_tile_order(D, bm // world, bn, RA), ref[rank::world], 5e-2)
    ok = int(MM.abs().sum()) == 0
    if rank == 0:
        print(f"{'PASS' if ok else 'FAIL'} two-stream comparator leaves the counters at zero", flush=True)
    failures += 0 if ok else 1

    # NCCL transport (what ranks on different nodes fall back to), forced here on one node
    assert impl.transport() == "p2p"
    impl.set_transport("nccl")
    out = impl.gemm_allreduce_fused(A, B, W, 1e-5, algo)
    torch.cuda.synchronize()
    check("nccl transport: gemm_allreduce_fused + norm", out, rms_ref(ref, W, 1e-5), 1e-2)
    rows = M // world
    Dn = torch.full((rows, N), float("nan"), device=dev, dtype=torch.float16)
    impl.gemm_reducescatter_fused(A, B, Dn, W, 1e-5, algo, False)
    torch.cuda.synchronize()
    check("nccl transport: gemm_reducescatter_fused + norm", Dn, rms_ref(ref[rank * rows:(rank + 1) * rows], W, 1e-5),
          1e-2)
    MM.zero_()
    C = torch.full((M, N), float("nan"), device=dev, dtype=torch.float16)
    impl.gemm_allreduce_overlap(A, B, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, False)
    torch.cuda.synchronize()
    check("nccl transport: gemm_allreduce_overlap", from_tile_order(C, bm, bn, RA), ref, 1e-2)
    g5 = torch.Generator(device="cpu").manual_seed(31337)
    A_full = torch.randn(M, K, generator=g5).to(dev, torch.float16)
    Cg = torch.empty((M, N), device=dev, dtype=torch.float16)
    impl.allgather_gemm(A_full[rank * rows:(rank + 1) * rows].contiguous(), B, Cg, algo)
    torch.cuda.synchronize()
    check("nccl transport: allgather_gemm", Cg, A_full.float() @ B.float().t(), 1e-2)
    impl.set_transport("p2p")

    # non-overlapped paths and the cuBLAS + NCCL baseline
    base = make_baseline_impl()
    C1 = torch.empty((M, N), device=dev, dtype=torch.float16)
    C2 = torch.empty((M, N), device=dev, dtype=torch.float16)
    impl.gemm_allreduce(A, B, C1, algo)
    base.gemm_allreduce(A, B, C2)
    torch.cuda.synchronize()
    check("OverlapImpl.gemm_allreduce (GEMM then NCCL)", C1, ref, 1e-2)
    check("BaselineImpl.gemm_allreduce (cuBLAS then NCCL)", C2, ref, 1e-2)
    D1 = torch.empty((M // world, N), device=dev, dtype=torch.float16)
    D2 = torch.empty((M // world, N), device=dev, dtype=torch.float16)
    impl.gemm_reducescatter(A, B, C1, D1, algo)
    base.gemm_reducescatter(A, B, C2, D2)
    torch.cuda.synchronize()
    rows = M // world
    check("OverlapImpl.gemm_reducescatter", D1, ref[rank * rows:(rank + 1) * rows], 1e-2)
    check("BaselineImpl.gemm_reducescatter", D2, ref[rank * rows:(rank + 1) * rows], 1e-2)

    dist.barrier()
    if rank == 0:
        print(f"DONE failures={failures}", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
