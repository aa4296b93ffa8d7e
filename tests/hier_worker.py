"""Worker of the hierarchical (several nodes) path, run on one machine with
FLASHOVERLAP_FAKE_NODES cutting the GPUs into pretend nodes: fused kernel
inside a node, NCCL across.  Compared with matmul + all_reduce /
reduce_scatter + RMSNorm in fp32."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import flashoverlap_b200  # noqa: F401
from flashoverlap_b200.models import HierarchicalRowParallelLinear
from flashoverlap_b200.parallel import build_hierarchy, init_distributed, make_intra_node_impl


def rms_ref(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def main():
    rank, world, _ = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    h = build_hierarchy()
    impl = make_intra_node_impl(h, timeout_ms=4000)
    if rank == 0:
        print(f"hierarchy: {h.nodes} nodes x {h.local_size} ranks", flush=True)
    failures = 0
    M, N, K = 1024, 2048, 256
    for comm_op in ("all_reduce", "reduce_scatter"):
        for norm in (False, True):
            layer = HierarchicalRowParallelLinear(impl, h, K, N, comm_op=comm_op, norm=norm, algo=0,
                                                  dtype=torch.float16, device=dev)
            g = torch.Generator(device="cpu").manual_seed(10 + rank)
            x = torch.randn(M, K, generator=g).to(dev, torch.float16)
            with torch.no_grad():
                layer.weight.copy_((torch.randn(N, K, generator=g) / K ** 0.5).to(dev, torch.float16))
                if norm:
                    gw = torch.Generator(device="cpu").manual_seed(3)
                    layer.norm_weight.copy_((1 + 0.1 * torch.randn(N, generator=gw)).to(dev, torch.float16))
            ref = x.float() @ layer.weight.float().t()
            dist.all_reduce(ref)
            want = rms_ref(ref, layer.norm_weight, 1e-5) if norm else ref
            for _ in range(2):
                y = layer(x)
            torch.cuda.synchronize()
            impl.check_status()
            if comm_op == "reduce_scatter":
                b, e = layer.owned_rows(M)
                want = want[b:e]
            err = (y.float() - want).abs().max().item()
            ok = torch.tensor([0 if (y.shape == want.shape and err <= 1e-2 * max(1.0, want.abs().max().item())) else 1],
                              device=dev)
            dist.all_reduce(ok)
            if rank == 0:
                print(f"{'PASS' if ok.item() == 0 else 'FAIL'} hierarchical {comm_op} norm={norm}: rank0 max err {err:.4g}",
                      flush=True)
            failures += int(ok.item() != 0)
    dist.barrier()
    if rank == 0:
        print(f"DONE failures={failures}", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
