"""The reference's collective entry points by name, on top of one engine.

``allreduce_ring_comprs_hom_sum{,_F,_seg,_F_seg,_F_opt}`` (HomComp/include/cuda_awareallreduce.cuh:4-17)
differ in the reference only in host orchestration: two kernels or one fused kernel per hop, even
or uneven chunks, scratch allocated per call or once.  This library has one code path that is
fused, handles any count, and never allocates, so the five names are the same call.
``cpuCopy_*`` (HomComp/include/nca_allreduce.cuh:3-15) are the host-staged variants: the device
codec does the work, every compressed chunk crosses the host (pinned bounce buffer, host network).  ``mixed_compressed_allreduce`` is
the hierarchical allreduce (raw inside a node, compressed between nodes);
``allreduce_ring_gpu`` the uncompressed device allreduce.
"""
from __future__ import annotations

import socket

import torch
import torch.distributed as dist

from .comm import CompressedAllreduce
from .cpu_ring import cpu_compressed_allreduce  # noqa: F401  (host-only counterpart)


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


_codecs = {}
_bounces = {}


def _bounce_for(device, nbytes):
    """Pinned host buffer for the device -> host leg, kept between calls: pinning tens of megabytes
    costs milliseconds, more than the copies it serves."""
    key = str(device)
    if key not in _bounces or _bounces[key].numel() < nbytes:
        _bounces[key] = torch.empty(int(nbytes), dtype=torch.uint8).pin_memory()
    return _bounces[key]


def _codec_for(device, max_elems):
    from ..ops import Codec

    key = (str(device), int(max_elems))
    if key not in _codecs:
        _codecs[key] = Codec(max_elems, device=device)
    return _codecs[key]


def cpuCopy_allreduce_ring_comprs_hom_sum_F(d_sbuf: torch.Tensor, d_rbuf: torch.Tensor, eb: float, host_group=None):
    """Host-staged compressed ring allreduce for GPUs that cannot address each other: the codec and
    the fused homomorphic add run on the device, every compressed chunk is copied to pinned host
    memory, travels over the host network (gloo) and is copied back up (the reference's
    non-CUDA-aware variants, HomComp/src/nca_allreduce.cu:195-324).  Same partition, hop order and
    arithmetic as the device ring, hence the same bits."""
    from .. import ops
    from .cpu_ring import _recv, _send

    g = host_group if host_group is not None else _host_group(None)
    P, r = dist.get_world_size(g), dist.get_rank(g)
    n = d_sbuf.numel()
    B = ops.chunk_elems(n, P)
    dev = d_sbuf.device
    codec = _codec_for(dev, B)
    src = d_sbuf.reshape(-1)
    dst = d_rbuf.reshape(-1)
    cap = ops.max_compressed_bytes(B) + 64
    bounce = _bounce_for(dev, cap)

    def chunk(c):
        return src[c * B: min((c + 1) * B, n)]

    def down(stream, size):  # device stream -> host bytes (the size is the one host read per hop)
        nbytes = int(size.item())
        bounce[:nbytes].copy_(stream[:nbytes])
        return bounce[:nbytes].numpy().copy()

    def up(arr):  # host bytes -> device stream, with the slack the bulk copies may read past the end
        t = torch.zeros(arr.size + 64, dtype=torch.uint8, device=dev)
        if arr.size:
            t[: arr.size].copy_(torch.from_numpy(arr))
        return t

    def exchange(out_bytes, what):  # even ranks send first, odd ranks receive first
        if r % 2 == 0:
            _send(out_bytes, (r + 1) % P, g)
            return _recv((r - 1) % P, g, what)
        incoming = _recv((r - 1) % P, g, what)
        _send(out_bytes, (r + 1) % P, g)
        return incoming

    import numpy as np

    empty = np.zeros(0, dtype=np.uint8)
    held = down(*codec.compress(chunk(r), eb)) if chunk(r).numel() else empty
    for s in range(1, P):
        incoming = exchange(held, "reduce-scatter step %d" % s) if P > 1 else held
        c = (r - s) % P
        m = chunk(c).numel()
        if m == 0:
            held = empty
        elif incoming.size:
            held = down(*codec.hom_add(up(incoming), chunk(c), eb, stream_bytes=incoming.size))
        else:
            held = down(*codec.compress(chunk(c), eb))
    held_c = (r + 1) % P
    streams = {held_c: held}
    for s in range(P - 1):
        held = exchange(held, "all-gather step %d" % s)
        held_c = (held_c - 1) % P
        streams[held_c] = held
    for c, st in streams.items():
        m = chunk(c).numel()
        if m:
            codec.decompress(up(st), m, eb, out=dst[c * B: c * B + m], stream_bytes=st.size)
    if codec.status() != 0:
        raise RuntimeError("host-staged allreduce: device codec reported an error")
    return d_rbuf


def host_staged_allreduce_native(codec, rank: int, world: int, send, recv, d_sbuf: torch.Tensor,
                                 d_rbuf: torch.Tensor, eb: float):
    """The library's own host-staged ring (``hc_allreduce_host_staged``) over a transport given as two
    Python callables: ``send(dst: int, data: bytes)`` and ``recv(src: int) -> bytes``.  The device
    codec ``codec`` (``ops.Codec`` for at least ``chunk_elems(n, world)`` values) does the work."""
    import ctypes as C

    from .. import _lib
    from .._lib_ext import RECV_FN, SEND_FN, HostTransport

    def _send(_user, dst, buf, nbytes):
        try:
            send(int(dst), C.string_at(buf, nbytes) if nbytes else b"")
            return 0
        except Exception:  # noqa: BLE001  (reported to the C side as a peer failure)
            return 1

    def _recv(_user, src, buf, cap, out_bytes):
        try:
            data = recv(int(src))
            if len(data) > cap:
                return 2
            if data:
                C.memmove(buf, data, len(data))
            out_bytes[0] = len(data)
            return 0
        except Exception:  # noqa: BLE001
            return 1

    tp = HostTransport(SEND_FN(_send), RECV_FN(_recv), None)
    lib = _lib.cuda()
    with torch.cuda.device(d_sbuf.device):
        rc = lib.hc_allreduce_host_staged(codec._h, C.byref(tp), rank, world, d_sbuf.data_ptr(), d_rbuf.data_ptr(),
                                          d_sbuf.numel(), eb, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "host-staged allreduce")
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
    inside the group, compressed allreduce of every local rank's slice between the groups, raw
    all-gather inside the group (``hc_allreduce_mixed``).

    ``comm`` spans the ranks of this group (the reference takes the ranks that share a node),
    ``inter_comm`` the ranks with the same local index in the other groups; it must take
    ``ops.chunk_elems(n, comm.world)`` values.  Without it there is one group and nothing is compressed,
    exactly as the reference's version degenerates when every rank shares a node.  ``make_hierarchy``
    builds both handles from a group size.
    """
    import ctypes as C

    from .. import _lib

    if d_sbuf.dtype != torch.float32 or not d_sbuf.is_cuda or not d_sbuf.is_contiguous() \
            or d_rbuf.dtype != torch.float32 or not d_rbuf.is_cuda or not d_rbuf.is_contiguous() \
            or d_rbuf.numel() != d_sbuf.numel():
        raise ValueError("expected contiguous float32 CUDA tensors of the same size")
    with torch.cuda.device(comm.device):
        _lib.check(comm.lib.hc_allreduce_mixed(comm._h, inter_comm._h if inter_comm is not None else None,
                                               d_sbuf.data_ptr(), d_rbuf.data_ptr(), d_sbuf.numel(), eb,
                                               torch.cuda.current_stream().cuda_stream), "allreduce_mixed")
    return d_rbuf


def make_hierarchy(max_count: int, group_size: int, transport: str | None = None, timeout_ms: int | None = None):
    """(local, inter) handles for ``mixed_compressed_allreduce``: consecutive ranks form groups of
    ``group_size`` (one node each in a multi-node job; halves or quarters of one NVSwitch box otherwise),
    ``inter`` joins the ranks with the same index in every group.  Collective over the default group."""
    from ..ops import chunk_elems

    world, rank = dist.get_world_size(), dist.get_rank()
    if group_size < 1 or world % group_size:
        raise ValueError("the world size must be a multiple of the group size")
    n_groups = world // group_size
    local_groups = [dist.new_group(list(range(g * group_size, (g + 1) * group_size))) for g in range(n_groups)]
    inter_groups = [dist.new_group(list(range(l, world, group_size))) for l in range(group_size)]
    local = CompressedAllreduce(max_count, group=local_groups[rank // group_size], transport=transport,
                                timeout_ms=timeout_ms)
    inter = None
    if n_groups > 1:
        inter = CompressedAllreduce(max(1, chunk_elems(max_count, group_size)), group=inter_groups[rank % group_size],
                                    transport=transport, timeout_ms=timeout_ms)
    return local, inter


def hierarchy_oracle(bufs, group_size: int, eb: float):
    """Host restatement of ``mixed_compressed_allreduce`` for ``len(bufs)`` ranks (numpy float32 arrays):
    group sums in fp32 in rank order, the host-rank compressed ring between the groups slice by slice.
    Bit-exact expectation for the ``ipc`` transport (a multicast mapping adds in the switch's order)."""
    import numpy as np

    from ..ops import chunk_elems, cpu_ring_allreduce

    world, n = len(bufs), bufs[0].size
    n_groups = world // group_size
    sums = []
    for g in range(n_groups):
        acc = np.zeros(n, dtype=np.float32)
        for l in range(group_size):
            acc = (acc + bufs[g * group_size + l].astype(np.float32)).astype(np.float32)
        sums.append(acc)
    if n_groups == 1:
        return sums[0]
    out = np.zeros(n, dtype=np.float32)
    B = chunk_elems(n, group_size)
    for l in range(group_size):
        lo, hi = min(n, l * B), min(n, (l + 1) * B)
        if hi > lo:
            out[lo:hi] = cpu_ring_allreduce([s[lo:hi] for s in sums], eb)[0]
    return out
