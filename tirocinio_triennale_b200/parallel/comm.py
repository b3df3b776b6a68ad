"""Compressed allreduce over NVLink peer memory, one process per GPU.

``torch.distributed`` is used for the bootstrap only (exchange of CUDA IPC handles, barriers); the
data path is the library's own kernels storing into peer memory.  The reference passes every
compressed chunk through MPI point-to-point calls (HomComp/src/cuda_awareallreduce.cu:208-255).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _lib


class CompressedAllreduce:
    """Handle-based compressed allreduce for float32 CUDA tensors of up to ``max_count`` values.

    Every call enqueues 3 kernels (``"direct"``, the default; 2 for the small messages that take its
    one-step form, see ``set_small_count``) or ``world + 1`` (``"ring"``) on the current stream: it never allocates, never synchronises the host and never copies a size to the host.  The result is identical on all
    ranks and equals ``2 * eb * sum_r quantise(x_r)``: the error is at most ``world * eb``.
    """

    def __init__(self, max_count: int, group=None, device=None, timeout_ms: int | None = None,
                 algorithm: str = "direct", transport: str | None = None):
        """``transport``: ``"ipc"`` maps every rank's region with CUDA IPC and moves all data with peer
        stores.  ``"mc"`` builds the regions with the library's own bootstrap (``hc_mc_create_shared``:
        driver virtual-memory API, handles passed as file descriptors over a unix socket) and, where
        every GPU supports multicast, pushes the reduced chunk to all ranks with one ``multimem.st`` per
        16 bytes and forms the uncompressed sum inside the switch (peer stores on the same mappings
        otherwise).  ``"nvls"`` is the same data path on a region taken from
        ``torch.distributed._symmetric_memory``.  Default: the ``HC_TRANSPORT`` environment variable,
        else ``"ipc"``."""
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (it carries the IPC handles)")
        import os

        transport = transport or os.environ.get("HC_TRANSPORT", "ipc")
        if transport not in ("ipc", "nvls", "mc"):
            raise ValueError("transport must be 'ipc', 'mc' or 'nvls'")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_count = int(max_count)
        self.lib = _lib.cuda()
        self._peers = {}
        self._base = None
        self._h = None
        self._symm = None
        self._mc_region = None
        self.multicast = False
        with torch.cuda.device(self.device):
            nbytes = int(self.lib.hc_comm_symmetric_bytes(self.world, self.max_count))
            self.symmetric_bytes = nbytes
            ptrs = (C.c_void_p * self.world)()
            mc = None
            if transport == "nvls" and self.world > 1:
                import torch.distributed._symmetric_memory as symm

                region = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
                region.zero_()
                hdl = symm.rendezvous(region, group if group is not None else dist.group.WORLD)
                for r in range(self.world):
                    ptrs[r] = int(hdl.buffer_ptrs[r])
                if int(hdl.multicast_ptr):
                    mc = C.c_void_p(int(hdl.multicast_ptr))
                    self.multicast = True
                self._symm = (region, hdl)
            elif transport == "mc" and self.world > 1:
                import secrets

                token = [("%d_%s" % (os.getpid(), secrets.token_hex(6))) if self.rank == 0 else None]
                dist.broadcast_object_list(token, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                           group=group)
                self.lib.hc_mc_create_shared.restype = C.c_int
                self.lib.hc_mc_create_shared.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_size_t, C.c_char_p]
                self.lib.hc_mc_unicast_ptr.restype = C.c_void_p
                self.lib.hc_mc_unicast_ptr.argtypes = [C.c_void_p, C.c_int]
                self.lib.hc_mc_multicast_ptr.restype = C.c_void_p
                self.lib.hc_mc_multicast_ptr.argtypes = [C.c_void_p]
                self.lib.hc_mc_destroy.restype = None
                self.lib.hc_mc_destroy.argtypes = [C.c_void_p]
                region = C.c_void_p()
                _lib.check(self.lib.hc_mc_create_shared(C.byref(region), self.rank, self.world, nbytes,
                                                        token[0].encode()), "mc_create_shared")
                self._mc_region = region
                for r in range(self.world):
                    ptrs[r] = self.lib.hc_mc_unicast_ptr(region, r)
                mcp = self.lib.hc_mc_multicast_ptr(region)
                if mcp:
                    mc = C.c_void_p(mcp)
                    self.multicast = True
            else:
                base = C.c_void_p()
                handle = C.create_string_buffer(64)
                _lib.check(self.lib.hc_ipc_alloc(C.byref(base), nbytes, handle), "ipc_alloc")
                self._base = base
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                for r in range(self.world):
                    if r == self.rank:
                        ptrs[r] = base.value
                    else:
                        p = C.c_void_p()
                        _lib.check(self.lib.hc_ipc_open(handles[r], C.byref(p)), "ipc_open(rank %d)" % r)
                        self._peers[r] = p
                        ptrs[r] = p.value
            self.transport = transport
            h = C.c_void_p()
            _lib.check(self.lib.hc_comm_create(C.byref(h), self.rank, self.world, self.max_count, ptrs, mc),
                       "comm_create")
            self._h = h
            self.set_algorithm(algorithm)
            if timeout_ms:
                _lib.check(self.lib.hc_comm_set_timeout_ms(self._h, int(timeout_ms)), "set_timeout")
            torch.cuda.synchronize()
        dist.barrier(group=group)  # every region is zeroed and mapped before the first store

    def allreduce(self, send: torch.Tensor, recv: torch.Tensor | None = None, eb: float = 1e-4) -> torch.Tensor:
        if send.dtype != torch.float32 or not send.is_cuda or not send.is_contiguous():
            raise ValueError("expected a contiguous float32 CUDA tensor")
        if recv is None:
            recv = send
        n = send.numel()
        if n > self.max_count or recv.numel() != n or recv.dtype != torch.float32 or not recv.is_cuda \
                or not recv.is_contiguous():
            raise ValueError("recv must be a contiguous float32 CUDA tensor of send's size, at most max_count values")
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_allreduce(self._h, send.data_ptr(), recv.data_ptr(), n, eb,
                                             torch.cuda.current_stream().cuda_stream), "allreduce")
        self._last = (n, eb)
        return recv

    def allreduce_host(self, send: torch.Tensor, recv: torch.Tensor | None = None, eb: float = 1e-4,
                       pieces: int = 0) -> torch.Tensor:
        """The same sum for float32 tensors in host memory (pin them: ``.pin_memory()``).  The message
        crosses PCIe in ``pieces`` pieces (0: pieces of 4 MiB, at most 16) while earlier pieces are being reduced and still earlier ones
        travel back, so a call costs about one direction of the transfer.  Asynchronous: the result is
        on the host once the current CUDA stream has been synchronised."""
        if send.dtype != torch.float32 or send.is_cuda or not send.is_contiguous():
            raise ValueError("expected a contiguous float32 host tensor")
        if recv is None:
            recv = send
        n = send.numel()
        if n > self.max_count or recv.numel() != n or recv.dtype != torch.float32 or recv.is_cuda \
                or not recv.is_contiguous():
            raise ValueError("recv must be a contiguous float32 host tensor of send's size, at most max_count values")
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_allreduce_host(self._h, send.data_ptr(), recv.data_ptr(), n, eb, int(pieces),
                                                  torch.cuda.current_stream().cuda_stream), "allreduce_host")
        self._last = (min(n, -(-n // max(1, pieces))), eb)
        return recv

    def allreduce_raw(self, send: torch.Tensor, recv: torch.Tensor | None = None) -> torch.Tensor:
        """Uncompressed sum with the library's own peer-memory kernels (bit-identical on all ranks)."""
        if send.dtype != torch.float32 or not send.is_cuda or not send.is_contiguous():
            raise ValueError("expected a contiguous float32 CUDA tensor")
        if recv is None:
            recv = send
        if recv.numel() != send.numel() or recv.dtype != torch.float32 or not recv.is_cuda or not recv.is_contiguous():
            raise ValueError("recv must be a contiguous float32 CUDA tensor of send's size")
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_allreduce_raw(self._h, send.data_ptr(), recv.data_ptr(), send.numel(),
                                                 torch.cuda.current_stream().cuda_stream), "allreduce_raw")
        return recv

    def status(self, clear: bool = True) -> int:
        with torch.cuda.device(self.device):
            return int(self.lib.hc_comm_status(self._h, 1 if clear else 0))

    def resync(self) -> int:
        """Collective over the host group.  After a call that some rank did not make (its peers got
        status 6 when their bounded waits ran out), brings the ranks' call numbers back in line, so
        that the handle can be used again; clears the sticky status.  Returns the status it cleared."""
        nums = (C.c_uint32 * 2)()
        _lib.check(self.lib.hc_comm_call_numbers(self._h, nums), "call_numbers")
        everybody = [None] * self.world
        dist.all_gather_object(everybody, (int(nums[0]), int(nums[1])), group=self.group)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_comm_resync(self._h, max(e[0] for e in everybody), max(e[1] for e in everybody)),
                       "resync")
            st = self.status(clear=True)
        dist.barrier(group=self.group)
        return st

    def status_site(self) -> int:
        """After a time-out (status 3): code of the wait that ran out first; call before clearing."""
        with torch.cuda.device(self.device):
            return int(self.lib.hc_comm_status_site(self._h))

    def set_algorithm(self, algorithm: str):
        """``"ring"``: one fused kernel per hop, world + 1 launches (the reference's
        algorithm); ``"direct"``: scatter, reduce, gather in three launches (default); ``"onestep"``:
        every rank broadcasts its whole compressed message and decodes the sum of all streams, two
        launches, for messages of at most ``max_count / world`` values (larger ones go direct).
        Same bits in all three."""
        code = {"ring": 0, "direct": 1, "onestep": 2}[algorithm]
        _lib.check(self.lib.hc_comm_set_algorithm(self._h, code), "set_algorithm")
        self.algorithm = algorithm

    def set_small_count(self, count: int):
        """Direct algorithm: messages of at most ``count`` values that fit one stream slot
        (``max_count / world`` values; ``max_count`` with two ranks) take the one-step form (0: never;
        default 12 Mi values with 2 ranks, 1.5 Mi with 3 or 4, 512 Ki above)."""
        _lib.check(self.lib.hc_comm_set_small_count(self._h, int(count)), "set_small_count")

    def set_overlap(self, on: bool = True):
        """Direct algorithm: let steps 2 and 3 start while their predecessor drains (programmatic
        dependent launch; default on, ignored while tracing).  Results do not depend on it."""
        _lib.check(self.lib.hc_comm_set_overlap(self._h, 1 if on else 0), "set_overlap")

    def set_shares(self, scatter_ctas_per_sm: int = 0, reduce_ctas_per_sm: int = 0, reduce_variant: int = 0):
        """Direct algorithm: CTAs per SM that the scatter and reduce steps may take (0: no limit), so that
        the three steps of a call share the GPU and run side by side; ``reduce_variant`` 0 auto, 1 ring,
        2 in place.  Results do not depend on it."""
        _lib.check(self.lib.hc_comm_set_shares(self._h, int(scatter_ctas_per_sm), int(reduce_ctas_per_sm),
                                               int(reduce_variant)), "set_shares")

    def set_sparse_tiles(self, on: bool = True):
        """Tiles at fixed offsets in the transport buffers (default; no CTA waits for a prefix over other
        CTAs' tiles) or packed back to back (``False``).  Results do not depend on it."""
        _lib.check(self.lib.hc_comm_set_sparse_tiles(self._h, 1 if on else 0), "set_sparse_tiles")

    def set_trace(self, on: bool = True):
        """Record one CUDA event per step of every following allreduce (see ``last_step_ms``)."""
        _lib.check(self.lib.hc_comm_set_trace(self._h, 1 if on else 0), "set_trace")

    def last_step_ms(self):
        """Device time of each step of the last traced call: reduce-scatter steps, then the decode."""
        arr = (C.c_float * 16)()
        with torch.cuda.device(self.device):
            n = int(self.lib.hc_comm_last_step_ms(self._h, arr, 16))
        return list(arr)[:n]

    def last_stream_bytes(self):
        """Stream bytes this rank produced at each step of the last call (synchronises)."""
        arr = (C.c_uint64 * 16)()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_comm_last_stream_bytes(self._h, arr, 16), "last_stream_bytes")
        return list(arr)[: self.world]

    def stats(self, clear_status: bool = False) -> dict:
        """Counters of the last ``allreduce`` call (synchronises the device): bytes of every stream
        this rank produced, compression ratio of its chunks, device time per step when tracing is
        on, and the sticky device status."""
        n, eb = getattr(self, "_last", (0, 0.0))
        sizes = self.last_stream_bytes() if n else []
        produced = [s for s in sizes if s > 0]
        form = ("ring", "direct", "onestep")[int(self.lib.hc_comm_last_form(self._h))]
        # the one-step form produces one stream of the whole message, the others one per chunk
        chunk_bytes = 4.0 * n if form == "onestep" else 4.0 * n / self.world
        return {
            "form": form,
            "world": self.world, "rank": self.rank, "algorithm": self.algorithm, "transport": self.transport,
            "multicast": self.multicast, "count": n, "error_bound": eb, "stream_bytes": sizes,
            "compression_ratio": (chunk_bytes * len(produced) / sum(produced)) if produced else None,
            "step_ms": self.last_step_ms(), "status": self.status(clear=clear_status),
        }

    def close(self, collective: bool = True):
        """Releases the handle and the mappings.  ``collective=True`` (the explicit call) first meets the
        other ranks at a barrier, because nobody may still be storing into a region that is about to go
        away; the destructor passes ``False`` and only releases local resources: garbage collection
        runs at different times on different ranks and must never wait for a peer."""
        if self._h is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if collective:
                try:
                    dist.barrier(group=self.group)
                except Exception:
                    pass
            self.lib.hc_comm_destroy(self._h)
            self._h = None
            for p in self._peers.values():
                self.lib.hc_ipc_close(p)
            self._peers = {}
            if self._base is not None:
                self.lib.hc_ipc_free(self._base)
            self._base = None
            self._symm = None
            if self._mc_region is not None:
                self.lib.hc_mc_destroy(self._mc_region)
                self._mc_region = None

    def __del__(self):
        try:
            self.close(collective=False)
        except Exception:
            pass
