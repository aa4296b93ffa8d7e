"""The ``detail`` block of bench.py: comparators, the other fused operations
and numerical checks, all on the ranks of the running job.

Everything here is outside the headline's timed region.  Times are CUDA-event
times per step with an L2 flush before each step, slowest rank; paired
measurements alternate the two alternatives so that both see the same clocks
(the table the reference's speed test prints: GEMM, vendor GEMM, baseline,
overlap, speed-up; reference: test/test.py:325-391)."""
from __future__ import annotations

import statistics

import torch
import torch.distributed as dist


def rms_ref(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def rel_err(got, want):
    """max |got - want| / max(1, max |want|): the quantity the reference's
    allclose(atol = rtol = tol) bounds (reference: example/correctness_ar.py:123)."""
    got = got.float()
    if not torch.isfinite(got).all().item():
        return float("inf")
    return (got - want.float()).abs().max().item() / max(1.0, want.float().abs().max().item())


def med_ratio(base_ts, fused_ts):
    """Ratio of the median step times: what one slow step (a stray clock dip) does not move."""
    return round(statistics.median(base_ts) / statistics.median(fused_ts), 3)


def run_detail(impl, layer, x, steps, warmup, algo, mx, stats):
    from flashoverlap_b200.parallel import make_baseline_impl
    from flashoverlap_b200.tune.runtime import gather_algo_candidates, pick_algo_by_timing, search_two_stream
    from flashoverlap_b200.utils.config import ALGO_TILES
    from flashoverlap_b200.utils.reorder import generate_row_mapping, reorder_indices
    from flashoverlap_b200.utils.timing import time_pairs, time_steps

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = x.device
    eps = layer.eps
    W, G = layer.weight, layer.norm_weight
    M, K = x.shape
    N = W.shape[0]
    detail, check = {}, {}

    def mean_max(ts):
        return sum(mx(ts)) / len(ts)

    def allsum(t):
        if world > 1:
            dist.all_reduce(t)
        return t

    # ---- headline shape: fused vs cuBLAS + NCCL all-reduce + RMSNorm kernel ------------------
    base = make_baseline_impl()
    C = torch.empty(M, N, device=dev, dtype=x.dtype)
    O = torch.empty(M, N, device=dev, dtype=x.dtype)

    def step():
        return layer(x)

    def base_step():
        base.gemm_allreduce(x, W, C)
        torch.ops.flashoverlap_op.rmsnorm(C, O, G, eps)

    ft, bt = time_pairs(step, base_step, steps, warmup)
    ft, bt = mx(ft), mx(bt)
    fused_ms, base_ms = sum(ft) / steps, sum(bt) / steps
    gt, ct = time_pairs(lambda: impl.cutlass_gemm(x, W, C, algo), lambda: base.cublas_gemm(x, W, C), steps, warmup)
    detail["ar_fp16"] = {
        "fused_ms": round(fused_ms, 4), "nccl_baseline_ms": round(base_ms, 4),
        "speedup_vs_nccl_baseline": round(base_ms / fused_ms, 3), "speedup_of_medians": med_ratio(bt, ft),
        "measured": "alternating steps",
        "fused_per_step_ms": stats(ft), "baseline_per_step_ms": stats(bt),
        "own_gemm_ms": round(mean_max(gt), 4), "cublas_gemm_ms": round(mean_max(ct), 4),
    }
    vs_baseline = round(base_ms / fused_ms, 3)

    # check: fused output against the baseline's output and against fp32 PyTorch on a sample of rows
    out = step().clone()
    base_step()
    torch.cuda.synchronize()
    rows = torch.arange(0, M, max(1, M // 64), device=dev)[:64]
    ref = allsum(x[rows].float() @ W.float().t())
    check["ar_max_err"] = rel_err(out[rows], rms_ref(ref, G, eps))
    check["ar_vs_nccl_baseline_max_err"] = rel_err(out, O)

    # ---- the reference's two-stream overlap design with a searched wave grouping -------------
    if world > 1:
        bm, bn, _ = ALGO_TILES[algo]
        cseg, ts_ms, timed = search_two_stream(impl, M, N, K, algo, "all_reduce", x.dtype, max_units=4, warmup=2,
                                               reps=5)
        tm, tn = M // bm, N // bn
        RA = reorder_indices(tm * tn, [], device=dev).reshape(tm, tn)
        cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
        cseg_gpu = cseg_cpu.to(dev)
        MM = torch.zeros(max(tn, len(cseg)), dtype=torch.int32, device=dev)

        def two_stream_step():
            if len(cseg) == 1:  # the search found that not overlapping is fastest: GEMM, one collective, RMSNorm
                impl.gemm_allreduce(x, W, C, algo)
                torch.ops.flashoverlap_op.rmsnorm(C, O, G, eps)
            else:               # tiles land in slot order, the norm kernel undoes the order
                impl.gemm_allreduce_twostream(x, W, C, MM, RA, 1, cseg_cpu, cseg_gpu, algo, 0)
                torch.ops.flashoverlap_op.reorder_rmsnorm_eps(C, O, G, bm, bn, 1, RA, eps)

        tt = mx(time_steps(two_stream_step, steps, warmup))
        detail["two_stream"] = {
            "ms": round(sum(tt) / steps, 4), "per_step_ms": stats(tt), "cSeg": cseg,
            "searched": [{"cSeg": g, "ms": round(t, 4)} for g, t in timed],
            "what": "signalling GEMM + stream waits + one NCCL all-reduce per wave group on a second stream + "
                    "reorder-RMSNorm; grouping chosen by timing every composition of <= 4 wave units",
        }
        torch.cuda.synchronize()
        check["two_stream_max_err"] = rel_err(O[rows], rms_ref(ref, G, eps))

    # ---- second named shape: GEMM + reduce-scatter + RMSNorm, bf16 ---------------------------
    M2, N2, K2_total = 8192, 8192, 28672
    K2 = K2_total // world
    bf = torch.bfloat16
    A2 = (torch.randn(M2, K2, device=dev) / K2 ** 0.5).to(bf)
    B2 = (torch.randn(N2, K2, device=dev) / K2 ** 0.5).to(bf)
    W2 = (1 + 0.1 * torch.randn(N2, generator=torch.Generator().manual_seed(4322))).to(dev, bf)  # same on every rank
    D2 = torch.empty(M2 // world, N2, device=dev, dtype=bf)
    C2 = torch.empty(M2, N2, device=dev, dtype=bf)
    O2 = torch.empty_like(D2)
    F2 = torch.empty_like(D2)

    # tile configuration and raster group (tile rows walked together) of this shape, searched like the tuner's
    # stage 2: timed candidates
    # (with this much K per rank the 64-deep pipeline stage of Algo 3 can beat the 128-deep one of Algo 8)
    rs_algo, rs_raster, rs_timed = algo, 0, []
    if world > 1:
        def run_cand(c):
            impl.set_raster_group(c[1])
            impl.gemm_reducescatter_fused(A2, B2, F2, W2, eps, c[0], False)

        cands = [(a, rg) for a in dict.fromkeys([algo, 3]) for rg in (4, 8)] + [(algo, 2)]
        (rs_algo, rs_raster), rs_timed = pick_algo_by_timing(run_cand, cands, warmup=1, reps=3)
        impl.set_raster_group(0)

    def fused_rs():
        impl.set_raster_group(rs_raster)
        impl.gemm_reducescatter_fused(A2, B2, F2, W2, eps, rs_algo, False)
        impl.set_raster_group(0)

    def base_rs():
        base.gemm_reducescatter(A2, B2, C2, D2)
        torch.ops.flashoverlap_op.rmsnorm(D2, O2, W2, eps)

    rt, brt = time_pairs(fused_rs, base_rs, steps, warmup)
    rt, brt = mx(rt), mx(brt)
    rs_ms, base_rs_ms = sum(rt) / steps, sum(brt) / steps
    detail["rs_bf16"] = {
        "M": M2, "N": N2, "K_per_rank": K2, "fused_ms": round(rs_ms, 4), "nccl_baseline_ms": round(base_rs_ms, 4),
        "speedup_vs_nccl_baseline": round(base_rs_ms / rs_ms, 3), "speedup_of_medians": med_ratio(brt, rt),
        "fused_per_step_ms": stats(rt), "baseline_per_step_ms": stats(brt),
        "tflops": round(2.0 * M2 * N2 * K2_total / (rs_ms * 1e-3) / 1e12, 1),
        "algo": rs_algo, "raster_group": rs_raster or "default",
        "candidates_timed": [{"algo": c[0], "raster_group": c[1], "ms": round(t, 4)} for c, t in rs_timed],
    }
    fused_rs()
    base_rs()
    torch.cuda.synchronize()
    rl = M2 // world
    rows2 = torch.arange(0, rl, max(1, rl // 32), device=dev)[:32]
    part = torch.zeros(world, rows2.numel(), N2, device=dev)
    for r in range(world):  # every rank contributes its partial of the sampled rows of every owner
        part[r] = A2[r * rl + rows2].float() @ B2.float().t()
    allsum(part)
    check["rs_max_err"] = rel_err(F2[rows2], rms_ref(part[rank], W2, eps))
    check["rs_vs_nccl_baseline_max_err"] = rel_err(F2, O2)
    del A2, B2, C2, D2, O2, F2, part

    # ---- all-gather -> GEMM on the decoder block's QKV shape -----------------------------------
    Mq, Kq, Nq = 8192, 8192, 10240 // world
    Aq_full = (torch.randn(Mq, Kq, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) / Kq ** 0.5).to(bf)
    Bq = (torch.randn(Nq, Kq, device=dev) / Kq ** 0.5).to(bf)
    shard = Aq_full[rank * (Mq // world):(rank + 1) * (Mq // world)].contiguous()
    Cq = torch.empty(Mq, Nq, device=dev, dtype=bf)
    Cb = torch.empty(Mq, Nq, device=dev, dtype=bf)
    gathered = torch.empty(Mq, Kq, device=dev, dtype=bf)

    # the tile configuration of a gather operation is searched like the tuner's stage 1: a few candidates
    # ranked by tiles per source block, each timed briefly, fastest kept
    ag_algo, ag_timed = algo, []
    if world > 1:
        cands = list(dict.fromkeys([algo] + gather_algo_candidates(Mq // world, Nq)[:3]))
        ag_algo, ag_timed = pick_algo_by_timing(lambda a: impl.allgather_gemm(shard, Bq, Cq, a), cands)

    def fused_ag():
        impl.allgather_gemm(shard, Bq, Cq, ag_algo)

    def base_ag():
        if world > 1:
            dist.all_gather_into_tensor(gathered, shard)
            base.cublas_gemm(gathered, Bq, Cb)
        else:
            base.cublas_gemm(shard, Bq, Cb)

    at, bat = time_pairs(fused_ag, base_ag, steps, warmup)
    at, bat = mx(at), mx(bat)
    ag_ms, base_ag_ms = sum(at) / steps, sum(bat) / steps
    push_bytes = (world - 1) * shard.numel() * 2
    detail["allgather_gemm_bf16"] = {
        "M": Mq, "N_per_rank": Nq, "K": Kq, "fused_ms": round(ag_ms, 4), "nccl_plus_cublas_ms": round(base_ag_ms, 4),
        "speedup": round(base_ag_ms / ag_ms, 3), "speedup_of_medians": med_ratio(bat, at),
        "fused_per_step_ms": stats(at), "baseline_per_step_ms": stats(bat),
        "push_gbs_lower_bound": round(push_bytes / (ag_ms * 1e-3) / 1e9, 1) if world > 1 else 0.0,
        "algo": ag_algo, "algos_timed": [{"algo": a, "ms": round(t, 4)} for a, t in ag_timed],
    }
    fused_ag()
    torch.cuda.synchronize()
    rq = torch.arange(0, Mq, Mq // 64, device=dev)
    check["ag_max_err"] = rel_err(Cq[rq], Aq_full[rq].float() @ Bq.float().t())
    del Aq_full, Cq, Cb, gathered, shard, Bq

    # ---- all-to-all dispatch -> GEMM, uneven token routing -------------------------------------
    Ke, Ne, T = 4096, 2048, 4096  # every rank routes T tokens to the ranks' experts
    gm = torch.Generator().manual_seed(99)
    weights = torch.rand(world, world, generator=gm) + 0.25
    weights[:, 0] *= 2.0  # a hot expert rank
    mlen = torch.floor(weights / weights.sum(1, keepdim=True) * T).to(torch.int32)
    mlen[:, -1] += (T - mlen.sum(1)).to(torch.int32)
    send = (torch.randn(T, Ke, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)) / Ke ** 0.5
            ).to(torch.float16)
    Be = (torch.randn(Ne, Ke, device=dev) / Ke ** 0.5).to(torch.float16)
    m_pad = (impl.a2a_padded_rows(mlen, algo) + 255) // 256 * 256  # room for every tile height
    Ce = torch.empty(m_pad, Ne, device=dev, dtype=torch.float16)
    recv_rows = int(mlen[:, rank].sum())
    recv = torch.empty(recv_rows, Ke, device=dev, dtype=torch.float16)
    Cbe = torch.empty(recv_rows, Ne, device=dev, dtype=torch.float16)
    in_split = [int(v) for v in mlen[rank]]
    out_split = [int(v) for v in mlen[:, rank]]

    e_algo, e_timed = algo, []
    if world > 1:
        cands = list(dict.fromkeys([algo] + gather_algo_candidates(T // world, Ne)[:3]))
        e_algo, e_timed = pick_algo_by_timing(lambda a: impl.a2a_dispatch_gemm(send, Be, Ce, mlen, a), cands)

    def fused_a2a():
        impl.a2a_dispatch_gemm(send, Be, Ce, mlen, e_algo)

    def base_a2a():
        if world > 1:
            dist.all_to_all_single(recv, send, out_split, in_split)
            base.cublas_gemm(recv, Be, Cbe)
        else:
            base.cublas_gemm(send, Be, Cbe)

    et, bet = time_pairs(fused_a2a, base_a2a, steps, warmup)
    et, bet = mx(et), mx(bet)
    detail["a2a_gemm_fp16"] = {
        "tokens_per_rank": T, "K": Ke, "N": Ne, "recv_rows_min_max": [int(mlen.sum(0).min()), int(mlen.sum(0).max())],
        "fused_ms": round(sum(et) / steps, 4), "nccl_plus_cublas_ms": round(sum(bet) / steps, 4),
        "speedup": round(sum(bet) / sum(et), 3), "speedup_of_medians": med_ratio(bet, et),
        "fused_per_step_ms": stats(et), "baseline_per_step_ms": stats(bet),
        "algo": e_algo, "algos_timed": [{"algo": a, "ms": round(t, 4)} for a, t in e_timed],
    }
    fused_a2a()
    base_a2a()
    torch.cuda.synchronize()
    if recv_rows > 0:
        got_rows = recv if world > 1 else send
        check["a2a_max_err"] = rel_err(Ce[:recv_rows:97], got_rows[::97].float() @ Be.float().t())
    else:
        check["a2a_max_err"] = 0.0

    # ---- outcome -------------------------------------------------------------------------------
    impl.check_status()
    tol = {"ar_max_err": 1e-2, "ar_vs_nccl_baseline_max_err": 1e-2, "two_stream_max_err": 1e-2, "rs_max_err": 5e-2,
           "rs_vs_nccl_baseline_max_err": 5e-2, "ag_max_err": 5e-2, "a2a_max_err": 1e-2}
    worst = {}
    for k, v in check.items():
        t = torch.tensor([v if v == v and v != float("inf") else 1e30], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst[k] = float(t.item())
    ok = all(worst[k] <= tol[k] for k in worst)
    detail["check"] = {k: round(v, 6) for k, v in worst.items()}
    detail["check"]["tolerances"] = tol
    detail["check"]["what"] = ("max over ranks of max|got-want|/max(1,max|want|); want = fp32 PyTorch on sampled rows "
                               "(matmul, sum over ranks, RMSNorm) or the cuBLAS+NCCL baseline's full output")
    detail["check"]["ok"] = bool(ok)
    return detail, vs_baseline, ok
