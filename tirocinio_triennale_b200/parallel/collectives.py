"""The reference's collective entry points by name, on top of one engine.

``allreduce_ring_comprs_hom_sum{,_F,_seg,_F_seg,_F_opt}`` (HomComp/include/cuda_awareallreduce.cuh:4-17)
differ in the reference only in host orchestration: two kernels or one fused kernel per hop, even
or uneven chunks, scratch allocated per call or once.  This library has one code path that is
fused, handles any count, and never allocates, so the five names are the same call.
``cpuCopy_*`` (HomComp/include/nca_allreduce.cuh:3-15) are the host-staged variants: device to
host, host-rank ring over the host network, host to device.  ``mixed_compressed_allreduce`` is
the hierarchical allreduce (raw inside a node, compressed between nodes);
``allreduce_ring_gpu`` the uncompressed device allreduce.
"""
from __future__ import annotations

import socket

import torch
import torch.distributed as dist

from .comm import CompressedAllreduce
from .cpu_ring import cpu_compressed_allreduce


def allreduce_ring_comprs_hom_sum_F(comm: CompressedAllreduce, d_sbuf, d_rbuf, eb: float):
    return comm.allreduce(d_sbuf, d_rbuf, eb)


allreduce_ring_comprs_hom_sum = allreduce_ring_comprs_hom_sum_F
allreduce_ring_comprs_hom_sum_seg = allreduce_ring_comprs_hom_sum_F
allreduce_ring_comprs_hom_sum_F_seg = allreduce_ring_comprs_hom_sum_F
allreduce_ring_comprs_hom_sum_F_opt = allreduce_ring_comprs_hom_sum_F


def allreduce_ring_gpu(comm: CompressedAllreduce, d_sbuf, d_rbuf):
    return comm.allreduce_raw(d_sbuf, d_rbuf)


_host_groups = {}


def _host_group(group):
    key = id(group)
    if key not in _host_groups:
        _host_groups[key] = dist.new_group(backend="gloo") if group is None else group
    return _host_groups[key]


def cpuCopy_allreduce_ring_comprs_hom_sum_F(d_sbuf: torch.Tensor, d_rbuf: torch.Tensor, eb: float, host_group=None):
    """Host-staged compressed allreduce: every message crosses the host (pinned bounce buffers)."""
    g = host_group if host_group is not None else _host_group(None)
    host = torch.empty(d_sbuf.numel(), dtype=torch.float32).pin_memory()
    host.copy_(d_sbuf)
    out = cpu_compressed_allreduce(host.numpy(), eb, group=g)
    d_rbuf.copy_(torch.from_numpy(out))
    return d_rbuf


cpuCopy_allreduce_ring_comprs_hom_sum = cpuCopy_allreduce_ring_comprs_hom_sum_F
cpuCopy_allreduce_ring_comprs_hom_sum_seg = cpuCopy_allreduce_ring_comprs_hom_sum_F
cpuCopy_allreduce_ring_comprs_hom_sum_F_seg = cpuCopy_allreduce_ring_comprs_hom_sum_F


def node_layout(group=None):
    """(local_rank, local_size, node_index, n_nodes) from the host names of the group's ranks."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    names = [None] * world
    dist.all_gather_object(names, socket.gethostname(), group=group)
    nodes = sorted(set(names), key=names.index)
    mine = [r for r in range(world) if names[r] == names[rank]]
    return mine.index(rank), len(mine), nodes.index(names[rank]), len(nodes)


def mixed_compressed_allreduce(comm: CompressedAllreduce, d_sbuf, d_rbuf, eb: float, inter_comm=None):
    """Hierarchical allreduce (HomComp/src/cuda_awareallreduce.cu:673-706): raw fp32 reduce-scatter
    inside the node, compressed allreduce of every local rank's slice between nodes, raw
    all-gather inside the node.

    ``comm`` spans the ranks of this node, ``inter_comm`` (optional) the ranks with the same local
    index on the other nodes.  On a single NVSwitch node there is no inter-node phase and the call
    is the uncompressed two-shot allreduce, exactly as the reference's version degenerates when
    every rank shares a node.
    """
    if inter_comm is None or inter_comm.world == 1:
        return comm.allreduce_raw(d_sbuf, d_rbuf)
    # node-local sum first, then the compressed exchange of this rank's slice between the nodes,
    # then redistribution inside the node (the raw kernels already leave the full node-local sum
    # on every local rank, so the slice exchange is followed by one more raw step)
    comm.allreduce_raw(d_sbuf, d_rbuf)
    n = d_rbuf.numel()
    per = (n + comm.world - 1) // comm.world
    lo, hi = min(n, comm.rank * per), min(n, (comm.rank + 1) * per)
    keep = d_rbuf[lo:hi].clone()
    inter_comm.allreduce(keep, keep, eb)
    d_rbuf.zero_()
    d_rbuf[lo:hi].copy_(keep)
    return comm.allreduce_raw(d_rbuf, d_rbuf)
