"""Two-level process groups for jobs that span several nodes.

Ranks on different hosts cannot map one another's memory, so the fused kernels
only reach the GPUs of one node.  A row-parallel layer over ``nodes x local``
ranks is then computed hierarchically: the fused kernel reduces inside every
node over NVLink, NCCL reduces across the nodes between ranks with the same
local index (one slice per rank, so all network cards are busy), and NCCL
gathers inside the node if the full result is wanted.  This module builds the
two families of groups; :class:`flashoverlap_b200.models.HierarchicalRowParallelLinear`
uses them.

The node of a rank is ``rank // local_size`` (torchrun numbers ranks node by
node).  ``FLASHOVERLAP_FAKE_NODES=n`` cuts a single node into ``n`` pretend
nodes, which is how the path is tested on one machine.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist


@dataclass
class Hierarchy:
    nodes: int
    local_size: int
    node: int          # index of this rank's node
    local_rank: int    # index of this rank inside its node
    intra: Optional[object]  # process group of this node's ranks (None when local_size == 1)
    inter: Optional[object]  # process group of the ranks with this local index (None when nodes == 1)


def node_layout(world: int, local_size: Optional[int] = None) -> tuple[int, int]:
    """(nodes, ranks per node) from the launcher's environment."""
    fake = int(os.environ.get("FLASHOVERLAP_FAKE_NODES", "0"))
    if fake > 0:
        if world % fake:
            raise ValueError(f"FLASHOVERLAP_FAKE_NODES={fake} does not divide the world size {world}")
        return fake, world // fake
    if local_size is None:
        local_size = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    if local_size <= 0 or world % local_size:
        raise ValueError(f"local world size {local_size} does not divide the world size {world}")
    return world // local_size, local_size


def build_hierarchy(local_size: Optional[int] = None) -> Hierarchy:
    """Collective over the default group: every rank creates every group
    (``torch.distributed.new_group`` requires that) and keeps its own two."""
    if not (dist.is_available() and dist.is_initialized()):
        return Hierarchy(1, 1, 0, 0, None, None)
    rank, world = dist.get_rank(), dist.get_world_size()
    nodes, local = node_layout(world, local_size)
    node, lrank = rank // local, rank % local
    intra = inter = None
    for n in range(nodes):
        ranks = list(range(n * local, (n + 1) * local))
        g = dist.new_group(ranks) if local > 1 else None
        if n == node:
            intra = g
    for l in range(local):
        ranks = list(range(l, world, local))
        g = dist.new_group(ranks) if nodes > 1 else None
        if l == lrank:
            inter = g
    return Hierarchy(nodes, local, node, lrank, intra, inter)


def make_intra_node_impl(h: Hierarchy, timeout_ms: Optional[int] = None, nvls: Optional[bool] = False):
    """The ``OverlapImpl`` of this rank's node (collective over the node's
    ranks): what the hierarchical layers hand their fused calls to.  NVLink
    SHARP is off by default here; pass ``nvls=None`` to let the usual rule decide."""
    import torch

    from .bootstrap import make_overlap_impl

    if h.intra is None:  # one rank per node: a group of one
        impl = torch.classes.flashoverlap_class.OverlapImpl()
        impl.nccl_init(0, 1, [0] * 16)
        impl.cutlass_init()
        impl.overlap_init()
        if timeout_ms is not None:
            impl.set_timeout_ms(int(timeout_ms))
        return impl
    return make_overlap_impl(group=h.intra, timeout_ms=timeout_ms, nvls=nvls)
