"""Host-rank compressed ring allreduce over ``torch.distributed`` (gloo): real processes, host
buffers, the portable codec.  Same partition, hop order and arithmetic as the device ring, so the
result is bit-identical to it and to ``cpu_ring_allreduce``.

This is the CPU reference path of the collectives (2-rank check of the stream round trip and of
the error bound) and the playground for host-side fault injection: every receive has a timeout,
and a peer that never sends surfaces as ``PeerTimeout`` instead of a hang.  Counterpart of the
host-staged variants of the reference (HomComp/src/nca_allreduce.cu:195-324) with the staging
buffers being the actual transport.
"""
from __future__ import annotations

from datetime import timedelta

import numpy as np
import torch
import torch.distributed as dist

from .. import ops


class PeerTimeout(RuntimeError):
    pass


def _send(arr: np.ndarray, dst: int, group):
    n = torch.tensor([arr.size], dtype=torch.int64)
    dist.send(n, dst, group=group)
    if arr.size:
        dist.send(torch.from_numpy(arr), dst, group=group)


def _recv(src: int, group, what: str) -> np.ndarray:
    n = torch.zeros(1, dtype=torch.int64)
    try:
        dist.recv(n, src, group=group)
        buf = torch.empty(int(n.item()), dtype=torch.uint8)
        if buf.numel():
            dist.recv(buf, src, group=group)
    except RuntimeError as e:  # gloo reports a missed deadline or a dead peer as RuntimeError
        raise PeerTimeout("%s from rank %d failed: %s" % (what, src, str(e).splitlines()[0])) from e
    return buf.numpy()


def cpu_compressed_allreduce(x, eb: float, group=None, drop_hop=None, hop_log=None) -> np.ndarray:
    """Sum of ``x`` (1-D float32, same length on every rank) over the group's ranks.

    ``drop_hop`` = (rank, step) makes that rank skip the send of that step: a host-side fault
    injection used by the tests (its successor then runs into the receive timeout of the group).
    ``hop_log`` (a list) receives the byte count of every stream this rank sends.
    """
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32).reshape(-1))
    P, r = dist.get_world_size(group), dist.get_rank(group)
    n = x.size
    B = ops.chunk_elems(n, P)

    def chunk(c):
        return x[c * B: min((c + 1) * B, n)]

    nxt, prv = (r + 1) % P, (r - 1) % P
    out = np.empty_like(x)
    stream = ops.cpu_compress(chunk(r), eb)
    for s in range(1, P):
        # even ranks send first, odd ranks receive first: no deadlock with blocking calls
        def do_send(st=stream, step=s - 1):
            if drop_hop == (r, step):
                return
            if hop_log is not None:
                hop_log.append(st.size)
            _send(st, nxt, group)

        if r % 2 == 0:
            do_send()
            incoming = _recv(prv, group, "reduce-scatter step %d" % s)
        else:
            incoming = _recv(prv, group, "reduce-scatter step %d" % s)
            do_send()
        c = (r - s) % P
        stream = ops.cpu_hom_add(incoming, chunk(c), eb) if chunk(c).size else ops.cpu_compress(chunk(c), eb)
    # rank r owns the reduced stream of chunk (r + 1) mod P; pass the reduced streams round the ring
    own = (r + 1) % P
    held, held_c = stream, own
    streams = {own: stream}
    for s in range(P - 1):
        if r % 2 == 0:
            _send(held, nxt, group)
            incoming = _recv(prv, group, "all-gather step %d" % s)
        else:
            incoming = _recv(prv, group, "all-gather step %d" % s)
            _send(held, nxt, group)
        held_c = (held_c - 1) % P
        held = incoming
        streams[held_c] = incoming
    for c, st in streams.items():
        m = chunk(c).size
        if m:
            out[c * B: c * B + m] = ops.cpu_decompress(st, m, eb)
    return out


def init_gloo(rank: int, world: int, port: int, timeout_s: float = 30.0):
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method="tcp://127.0.0.1:%d" % port,
                            timeout=timedelta(seconds=timeout_s))
