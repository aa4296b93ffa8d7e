"""One process per GPU: rendezvous, device binding and creation of the
``OverlapImpl`` / ``BaselineImpl`` objects.

The reference repeats this in every script (reference: tune/search.py:31-64,
test/test.py:36-80): initialise ``torch.distributed`` from the environment,
let rank 0 create an NCCL unique id, broadcast it as 16 int64 values and hand
it to ``nccl_init``.  Here it lives in one place and also works on CPU with the
``gloo`` backend (for the host-side logic and the tests that run without a GPU).
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0):
    """Initialise the default process group from RANK / WORLD_SIZE / MASTER_*.

    Returns ``(rank, world_size, local_rank)``.  With a single process (no
    ``WORLD_SIZE`` in the environment) nothing is initialised.
    """
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if use_cuda else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(
            backend=backend,
            rank=rank,
            world_size=world,
            timeout=datetime.timedelta(seconds=timeout_s),
            **kwargs,
        )
    return rank, world, local_rank


def _world(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def broadcast_nccl_id(group=None) -> list[int]:
    """Rank 0 of ``group`` creates an NCCL unique id; everyone receives it as a
    list of 16 ints (reference: tune/search.py:50-64)."""
    rank, world = _world(group)
    if world == 1:
        return [0] * 16
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    if rank == 0:
        words = torch.ops.flashoverlap_op.generate_nccl_id()
        t = torch.tensor(words, dtype=torch.int64, device=device)
    else:
        t = torch.zeros(16, dtype=torch.int64, device=device)
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast(t, src=src, group=group)
    return [int(v) for v in t.cpu().tolist()]


_symmetric_keepalive: list = []


def attach_symmetric_memory(impl, nbytes: int, group=None) -> bool:
    """Allocate ``nbytes`` of symmetric memory with
    ``torch.distributed._symmetric_memory``, map it on all ranks of ``group``
    and hand it to ``impl`` (collective).  When the mapping comes with an
    NVLink SHARP multicast address the fused operations of ``impl`` use
    ``multimem`` instructions.  Returns whether a multicast address exists."""
    import torch.distributed._symmetric_memory as symm

    grp = group if group is not None else dist.group.WORLD
    dev = torch.device("cuda", torch.cuda.current_device())
    buf = symm.empty(int(nbytes), dtype=torch.uint8, device=dev)
    handle = symm.rendezvous(buf, grp)
    off = int(getattr(handle, "offset", 0) or 0)  # position of `buf` inside the mapped block
    mc = int(handle.multicast_ptr) + off if handle.multicast_ptr else 0
    ptrs = [int(p) + off for p in handle.buffer_ptrs]
    if ptrs[dist.get_rank(grp)] != buf.data_ptr():
        raise RuntimeError("symmetric memory handle does not describe the allocated tensor")
    impl.attach_symmetric(ptrs, mc, int(nbytes))
    _symmetric_keepalive.append((buf, handle))  # the engine holds raw pointers into this memory
    return mc != 0


def workspace_bytes(max_m: int, max_n: int) -> int:
    """Symmetric memory the engine needs for problems up to ``max_m x max_n``
    (two staging and two result buffers of 16-bit values plus counters)."""
    return 8 * max_m * max_n + (4 << 20)


def make_overlap_impl(group=None, timeout_ms: Optional[int] = None, nvls: Optional[bool] = None,
                      max_m: int = 8192, max_n: int = 8192):
    """An initialised ``OverlapImpl`` for the ranks of ``group`` (collective).

    ``nvls`` (default: on, unless ``FLASHOVERLAP_NVLS=0``) asks for symmetric
    memory with an NVLink SHARP multicast mapping sized for problems up to
    ``max_m x max_n``.  The ranks agree on the outcome: if the mapping cannot be
    made on ANY rank, every rank falls back together to the peer-mapped memory
    the object allocates itself on first use.

    With the mapping the fused all-reduce CAN reduce with ``multimem``
    instructions (the switch adds the partial tiles and multicasts the results:
    fewer bytes per NVLink direction than two rounds of peer-to-peer stores from
    four ranks on), but it does so only when asked (``FLASHOVERLAP_NVLS_AR=1`` or
    ``impl.set_use_nvls(True, False)``): measured on 4 and 8 B200s the
    peer-to-peer form is faster (0.210 against 0.256 ms with four ranks),
    because its first half, the partial tiles, travels from the GEMM's epilogue
    while the GEMM still runs, whereas the switch can only pull rows that are
    complete.  ``FLASHOVERLAP_NVLS_AR=0`` pins peer-to-peer stores."""
    rank, world = _world(group)
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(rank, world, broadcast_nccl_id(group))
    impl.cutlass_init()
    impl.overlap_init()
    if nvls is None:
        nvls = os.environ.get("FLASHOVERLAP_NVLS", "1") not in ("0", "false", "off")
    if (nvls and world > 1 and torch.cuda.is_available() and dist.get_backend(group) == "nccl"
            and impl.transport() == "p2p"):
        err = None
        try:
            attach_symmetric_memory(impl, workspace_bytes(max_m, max_n), group)
        except Exception as exc:  # noqa: BLE001  (any failure means "no multicast here")
            err = exc
        # every rank learns whether every rank succeeded; a partial success would leave some ranks on the
        # attached memory and others in the collective set-up of their own heap
        flag = torch.tensor([0 if err is None else 1], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        if int(flag.item()) != 0:
            if err is None:
                impl.detach_symmetric()
            if rank == 0:
                why = repr(err) if err is not None else "another rank could not map it"
                print(f"flashoverlap_b200: symmetric memory with multicast unavailable ({why}); using P2P stores")
    force = os.environ.get("FLASHOVERLAP_NVLS_AR")
    if force is not None and world > 1:
        impl.set_use_nvls(force not in ("0", "false", "off"), False)
    env = os.environ.get("FLASHOVERLAP_TIMEOUT_MS")
    if timeout_ms is None and env:
        timeout_ms = int(env)
    if timeout_ms is not None:
        impl.set_timeout_ms(int(timeout_ms))
    return impl


def make_baseline_impl(group=None):
    """An initialised ``BaselineImpl`` (cuBLAS + NCCL) for ``group`` (collective)."""
    rank, world = _world(group)
    impl = torch.classes.flashoverlap_class.BaselineImpl()
    impl.nccl_init(rank, world, broadcast_nccl_id(group))
    impl.cublas_init()
    return impl


def max_over_ranks(value: float, group=None) -> float:
    """Maximum of a host number over the ranks (multi-GPU times are reported as
    the slowest rank's, reference: test/test.py:205-207)."""
    _, world = _world(group)
    if world == 1:
        return float(value)
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
