"""RMSNorm modules under the reference's module name (reference: example/RMSNorm.py),
and, run as a script on a GPU, the three of them side by side:

    python example/RMSNorm.py [--rows 4096 --dim 8192 --dtype bfloat16]

``RMSNorm`` (PyTorch, the golden path), ``KernelRMSNorm`` (the sm_100a kernel on
the natural layout) and ``ReorderRMSNorm`` (the kernel that reads the
tile-reordered buffer the reference-compatible overlap calls write and returns
rows in natural order), with the largest difference to the PyTorch result and
the kernels' times.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from flashoverlap_b200.models.rmsnorm import KernelRMSNorm, ReorderRMSNorm, RMSNorm  # noqa: F401,E402


def main():
    from flashoverlap_b200.cli import DTYPES
    from flashoverlap_b200.utils.reorder import to_tile_order
    from flashoverlap_b200.utils.timing import time_steps

    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--dim", type=int, default=8192)
    ap.add_argument("--dtype", default="float16", choices=sorted(DTYPES))
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("example/RMSNorm.py needs a CUDA device for the kernel modules")
    dt = DTYPES[args.dtype]
    M, N, BM, BN = args.rows, args.dim, 128, 256
    torch.manual_seed(0)
    x = torch.randn(M, N, device="cuda").to(dt)
    golden = RMSNorm(N, dtype=dt)
    kernel = KernelRMSNorm(N, dtype=dt)
    tiles = (M // BM) * (N // BN)
    hint = torch.randperm(tiles, generator=torch.Generator().manual_seed(1)).tolist()   # some completion order
    reorder = ReorderRMSNorm(N, M, BM, BN, hint, dtype=dt)
    with torch.no_grad():
        kernel.weight.copy_(golden.weight)
        reorder.weight.copy_(golden.weight)
        want = golden(x).float()
        got_kernel = kernel(x).float()
        x_tiled = to_tile_order(x, BM, BN, reorder.reorder_array.reshape(-1)).reshape(M, N)
        got_reorder = reorder(x_tiled).float()
    scale = want.abs().max().item()
    print(f"{M} x {N} {args.dtype}: max |kernel - torch| = {(got_kernel - want).abs().max().item():.4g}, "
          f"max |reorder kernel - torch| = {(got_reorder - want).abs().max().item():.4g} (largest value {scale:.3g})")
    t_k = sorted(time_steps(lambda: kernel(x), 10, 3))[5] * 1e3
    t_r = sorted(time_steps(lambda: reorder(x_tiled), 10, 3))[5] * 1e3
    t_t = sorted(time_steps(lambda: golden(x), 10, 3))[5] * 1e3
    gb = 2 * M * N * x.element_size() / 1e9
    print(f"time per call (L2 flushed): kernel {t_k:.1f} us ({gb / t_k * 1e6:.0f} GB/s), reorder kernel {t_r:.1f} us, "
          f"PyTorch {t_t:.1f} us")
    ok = (got_kernel - want).abs().max().item() <= 2e-2 * scale and (got_reorder - want).abs().max().item() <= 2e-2 * scale
    print("PASS" if ok else "FAIL")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
