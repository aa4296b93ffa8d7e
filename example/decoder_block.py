"""Decoder-block forward with the fused kernels against the PyTorch path
(matmul + NCCL collectives): correctness and time per block.

    torchrun --nproc_per_node=8 example/decoder_block.py [--hidden 8192 --ffn 28672 --batch 2 --seq 4096]
"""
import argparse

import torch.distributed as dist
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from flashoverlap_b200.cli import DTYPES, finish, make_overlap_impl, start  # noqa: E402

from flashoverlap_b200.models.decoder_block import TPDecoderBlock
from flashoverlap_b200.parallel import max_over_ranks
from flashoverlap_b200.utils.timing import time_pairs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv_heads", type=int, default=8)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--dtype", default="bfloat16", choices=sorted(DTYPES))
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    rank, ws = start()
    T = args.batch * args.seq
    impl = make_overlap_impl(max_m=T, max_n=max(args.hidden, 8192))
    block = TPDecoderBlock(impl, args.hidden, args.ffn, args.heads, args.kv_heads, dtype=DTYPES[args.dtype])
    g = torch.Generator(device="cpu").manual_seed(7)
    resid = torch.randn(T, args.hidden, generator=g).cuda().to(DTYPES[args.dtype])
    h = (resid.float() * torch.rsqrt(resid.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(resid.dtype)
    q1, r1 = block(h, resid, args.batch, args.seq)
    q2, r2 = block.forward_reference(h, resid, args.batch, args.seq)
    torch.cuda.synchronize()
    impl.check_status()
    e_q = float((q1.float() - q2.float()).abs().max() / q2.float().abs().max())
    e_r = float((r1.float() - r2.float()).abs().max() / r2.float().abs().max())
    ok = e_q < 5e-2 and e_r < 5e-2
    tf, tr = time_pairs(lambda: block(h, resid, args.batch, args.seq),
                        lambda: block.forward_reference(h, resid, args.batch, args.seq), args.steps, 3)
    fused_ms, ref_ms = max_over_ranks(sum(tf)) / args.steps, max_over_ranks(sum(tr)) / args.steps
    if rank == 0:
        print(f"TP={ws} tokens={T} hidden={args.hidden} ffn={args.ffn} {args.dtype}")
        print(f"relative max error: next QKV {e_q:.3e}, residual {e_r:.3e} -> {'PASS' if ok else 'FAIL'}")
        print(f"block forward: fused {fused_ms:.3f} ms, torch matmul + NCCL {ref_ms:.3f} ms, speedup {ref_ms / fused_ms:.2f}x")
    finish()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
