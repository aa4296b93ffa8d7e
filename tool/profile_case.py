"""One small case of one kernel, a few launches, for a profiler run:

    python tool/profile_case.py gemm 4096 8192 8192 --algo 3
    python tool/profile_case.py gemm_rmsnorm 4096 8192 1024 --algo 3 --dtype float16
    python tool/profile_case.py rmsnorm 4096 8192

    ncu --set full --clock-control none -k regex:gemm_fused -s 2 -c 1 -o out python tool/profile_case.py gemm ...

(Single GPU only: a profiler replays every kernel many times, which a kernel
that waits for other ranks does not survive.)
"""
import argparse

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "gemm_rmsnorm", "rmsnorm"])
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int, nargs="?", default=1024)
    ap.add_argument("--algo", type=int, default=3)
    ap.add_argument("--raster", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=sorted(DTYPES))
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dt = DTYPES[args.dtype]
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    impl.set_timeout_ms(3000)
    impl.set_raster_group(args.raster)
    M, N, K = args.m, args.n, args.k
    A = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dt)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dt)
    W = torch.ones(N, device="cuda", dtype=dt)
    C = torch.empty(M, N, device="cuda", dtype=dt)
    O = torch.empty_like(C)
    for _ in range(args.launches):
        if args.op == "gemm":
            impl.cutlass_gemm(A, B, C, args.algo)
        elif args.op == "gemm_rmsnorm":
            impl.gemm_rmsnorm(A, B, C, O, W, 1e-5, args.algo)
        else:
            torch.ops.flashoverlap_op.rmsnorm(C, O, W, 1e-5)
    torch.cuda.synchronize()
    impl.check_status()
    print("ok")


if __name__ == "__main__":
    main()
