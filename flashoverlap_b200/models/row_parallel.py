"""Row-parallel linear layers: the K dimension of ``x @ W^T`` is split over
the ranks and the partial products are summed by an all-reduce or a
reduce-scatter (reference: example/RowParallelLinear.py:11-85).

* :class:`RowParallelLayer` is the PyTorch golden path (matmul + collective).
* :class:`OverlapRowParallelLayer` keeps the reference's constructor and
  tile-reordered output so that its scripts and tuned configs work unchanged.
* :class:`FusedRowParallelLinear` is the native interface: natural-order output,
  optional fused RMSNorm, contiguous or interleaved reduce-scatter.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.reorder import div_up, generate_row_mapping, reorder_indices


def _device(device):
    if device is not None:
        return torch.device(device)
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


class RowParallelLayer(nn.Module):
    def __init__(self, in_features: int, out_features: int, comm_op: str, tp_group=None, dtype=torch.float16,
                 device=None):
        super().__init__()
        assert comm_op in ("all_reduce", "reduce_scatter"), f"unknown comm_op {comm_op!r}"
        self.tp_group = tp_group
        self.comm_op = comm_op
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device=_device(device)))

    def forward(self, x):
        out = torch.matmul(x, self.weight.t())
        if not (dist.is_available() and dist.is_initialized()):
            return out
        if self.comm_op == "all_reduce":
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.tp_group)
            return out
        world = dist.get_world_size(self.tp_group)
        cout = torch.empty((x.size(0) // world, self.weight.size(0)), dtype=out.dtype, device=out.device)
        dist.reduce_scatter_tensor(cout, out, group=self.tp_group)
        return cout


class OverlapRowParallelLayer(nn.Module):
    """Reference-compatible layer.  ``config`` is a stage-2 tuning result
    (``BM``, ``BN``, ``Algo``, ``hint``, ``cSeg``); ``nccl_id`` the 16-word id
    broadcast from rank 0.  The all-reduce output is in tile-reordered layout
    (feed it to :class:`ReorderRMSNorm`); the reduce-scatter output holds this
    rank's interleaved rows in the same slot order."""

    def __init__(self, rank: int, world_size: int, in_features: int, out_features: int, M: int, config: dict,
                 comm_op: str, nccl_id, dtype=torch.float16, device=None):
        super().__init__()
        assert comm_op in ("all_reduce", "reduce_scatter"), f"unknown comm_op {comm_op!r}"
        dev = _device(device)
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device=dev))
        self.world_size = world_size
        self.comm_op = comm_op
        self.overlap_class = torch.classes.flashoverlap_class.OverlapImpl()
        self.overlap_class.nccl_init(rank, world_size, [int(v) for v in nccl_id])
        self.overlap_class.cutlass_init()
        self.overlap_class.overlap_init()
        BM, BN = config["BM"], config["BN"]
        hint, cseg = config["hint"], config["cSeg"]
        tm, tn = div_up(M, BM), div_up(out_features, BN)
        self.algo = config["Algo"]
        self.counter = torch.zeros((1, max(tn, len(cseg))), dtype=torch.int32, device=dev)
        self.reorder_array = reorder_indices(tm * tn, hint, device=dev).reshape(tm, tn)
        self.cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
        self.cseg_gpu = self.cseg_cpu.to(dev)
        self.row_array = (generate_row_mapping(M, out_features, BM, BN, cseg, world_size, device=dev)
                          if comm_op == "reduce_scatter" else None)

    def forward(self, x):
        n = self.weight.size(0)
        if self.comm_op == "all_reduce":
            out = torch.empty((x.size(0), n), dtype=x.dtype, device=x.device)
            self.overlap_class.gemm_allreduce_overlap(x, self.weight, out, self.counter, self.reorder_array, 1,
                                                      self.cseg_cpu, self.cseg_gpu, self.algo, False)
            return out
        tmp = torch.empty((x.size(0), n), dtype=x.dtype, device=x.device)
        out = torch.empty((x.size(0) // self.world_size, n), dtype=x.dtype, device=x.device)
        self.overlap_class.gemm_reducescatter_overlap(x, self.weight, tmp, out, self.counter, self.reorder_array,
                                                      self.row_array, 1, self.cseg_cpu, self.cseg_gpu, self.algo,
                                                      False)
        return out


class FusedRowParallelLinear(nn.Module):
    """``y = collective(x @ W^T)`` with an optional RMSNorm, as one kernel.

    ``impl`` is an initialised ``OverlapImpl`` (see
    :func:`flashoverlap_b200.parallel.make_overlap_impl`); ``norm_weight`` turns
    the fused RMSNorm on.  With ``comm_op="all_reduce"`` the returned tensor
    aliases the implementation's symmetric result buffer and stays valid until
    the second next fused call on the same ``impl``.

    ``algo`` and ``raster_group`` are what the tuner searches for a shape
    (``tune/search.py`` stores them as ``Algo`` and ``raster_group`` in the
    stage-2 JSON; :meth:`from_config` reads them); ``raster_group=0`` leaves the
    library's default."""

    def __init__(self, impl, in_features: int, out_features: int, comm_op: str = "all_reduce",
                 norm: bool = False, eps: float = 1e-5, algo: int = 0, interleave: bool = False,
                 dtype=torch.float16, device=None, raster_group: int = 0):
        super().__init__()
        assert comm_op in ("all_reduce", "reduce_scatter"), f"unknown comm_op {comm_op!r}"
        dev = _device(device)
        self.impl = impl
        self.comm_op = comm_op
        self.eps = eps
        self.algo = algo
        self.raster_group = int(raster_group)
        self.interleave = interleave
        self.world_size = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device=dev) /
                                   (in_features * self.world_size) ** 0.5)
        self.norm_weight: Optional[nn.Parameter] = (
            nn.Parameter(torch.ones(out_features, dtype=dtype, device=dev)) if norm else None)

    @classmethod
    def from_config(cls, impl, config: dict, in_features: int, out_features: int, **kwargs):
        """A layer that runs the tile configuration and raster group a search
        found (``config``: the stage-2 dictionary of
        :func:`flashoverlap_b200.utils.config.load_config`)."""
        kwargs.setdefault("comm_op", config.get("comm_op", "all_reduce"))
        return cls(impl, in_features, out_features, algo=int(config["Algo"]),
                   raster_group=int(config.get("raster_group", 0)), **kwargs)

    @torch.no_grad()
    def forward(self, x):
        if self.raster_group:
            self.impl.set_raster_group(self.raster_group)  # a host-side setting of the next launches
        try:
            if self.comm_op == "all_reduce":
                return self.impl.gemm_allreduce_fused(x, self.weight, self.norm_weight, self.eps, self.algo)
            out = torch.empty((x.size(0) // self.world_size, self.weight.size(0)), dtype=x.dtype, device=x.device)
            self.impl.gemm_reducescatter_fused(x, self.weight, out, self.norm_weight, self.eps, self.algo,
                                               self.interleave)
            return out
        finally:
            if self.raster_group:
                self.impl.set_raster_group(0)


class HierarchicalRowParallelLinear(nn.Module):
    """Row-parallel linear (+ RMSNorm) over ``nodes x local`` ranks: fused inside
    a node, NCCL across nodes.

    * inside every node the fused kernel computes the GEMM and reduce-scatters
      the partial products over NVLink: local rank l ends up with rows
      ``[l*M/local, (l+1)*M/local)`` summed over its node;
    * across the nodes the ranks with the same local index sum their slices
      (``all_reduce`` of M/local rows) or, for a reduce-scatter result,
      reduce-scatter them so that every rank keeps M/world rows;
    * RMSNorm runs on the slice each rank holds;
    * for an all-reduce result the node's ranks all-gather their slices.

    With one node this is :class:`FusedRowParallelLinear` with ``comm_op``
    ``reduce_scatter`` followed by an all-gather.  ``impl`` must be an
    ``OverlapImpl`` made for ``hierarchy.intra`` (``make_overlap_impl(group=...)``).

    Row ownership of the reduce-scatter result: rank (node n, local l) holds
    rows ``l*M/local + n*M/world + [0, M/world)``."""

    def __init__(self, impl, hierarchy, in_features: int, out_features: int, comm_op: str = "all_reduce",
                 norm: bool = False, eps: float = 1e-5, algo: int = 0, dtype=torch.float16, device=None):
        super().__init__()
        assert comm_op in ("all_reduce", "reduce_scatter"), f"unknown comm_op {comm_op!r}"
        dev = _device(device)
        self.impl = impl
        self.h = hierarchy
        self.comm_op = comm_op
        self.eps = eps
        self.algo = algo
        world = hierarchy.nodes * hierarchy.local_size
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device=dev) /
                                   (in_features * world) ** 0.5)
        self.norm_weight: Optional[nn.Parameter] = (
            nn.Parameter(torch.ones(out_features, dtype=dtype, device=dev)) if norm else None)

    def owned_rows(self, M: int) -> tuple[int, int]:
        """[begin, end) of the rows a reduce-scatter result holds on this rank."""
        per_local = M // self.h.local_size
        per_rank = per_local // self.h.nodes
        begin = self.h.local_rank * per_local + self.h.node * per_rank
        return begin, begin + per_rank

    @torch.no_grad()
    def forward(self, x):
        h = self.h
        M, N = x.size(0), self.weight.size(0)
        rows = M // h.local_size
        part = torch.empty((rows, N), dtype=x.dtype, device=x.device)
        # the RMSNorm can only be fused when the node's sum is already the full sum
        fuse_norm = self.norm_weight is not None and h.nodes == 1
        self.impl.gemm_reducescatter_fused(x, self.weight, part, self.norm_weight if fuse_norm else None, self.eps,
                                           self.algo, False)
        if h.nodes > 1:
            if self.comm_op == "all_reduce":
                dist.all_reduce(part, group=h.inter)
                mine = part
            else:
                mine = torch.empty((rows // h.nodes, N), dtype=x.dtype, device=x.device)
                dist.reduce_scatter_tensor(mine, part, group=h.inter)
            if self.norm_weight is not None:
                out = torch.empty_like(mine)
                torch.ops.flashoverlap_op.rmsnorm(mine, out, self.norm_weight, self.eps)
                mine = out
        else:
            mine = part
        if self.comm_op == "reduce_scatter":
            return mine
        if h.local_size == 1:
            return mine
        full = torch.empty((M, N), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(full, mine, group=h.intra)
        return full
