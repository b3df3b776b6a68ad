"""The sm_100a device codec on torch tensors.

Every method only enqueues kernels on the current CUDA stream: no allocation inside the native
call, no host synchronisation, and the exact stream length stays in a device word (``size``).
Reading ``size`` on the host (``int(size)``) is the caller's decision.  The reference returns the
size through a blocking 4-byte copy after every launch (HomComp/src/GSZ_entry.cu:291-295).
"""
from __future__ import annotations

import torch

from .. import _lib, MODES
from .cpu_codec import max_compressed_bytes


def _mode(mode) -> int:
    return MODES[mode] if isinstance(mode, str) else int(mode)


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class Codec:
    """Codec handle for calls of up to ``max_elems`` values on one device."""

    def __init__(self, max_elems: int, device=None, timeout_ms: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("the device codec needs a CUDA device (use the cpu_* functions on the host)")
        self.lib = _lib.cuda()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_elems = int(max_elems)
        nbytes = int(self.lib.hc_codec_workspace_bytes(self.max_elems))
        with torch.cuda.device(self.device):
            self._ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
            import ctypes as C

            h = C.c_void_p()
            _lib.check(self.lib.hc_codec_create_in(C.byref(h), self._ws.data_ptr(), nbytes, self.max_elems,
                                                   _stream_ptr()), "codec_create")
            self._h = h
        if timeout_ms:
            self.set_timeout_ms(timeout_ms)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.hc_codec_destroy(h)
            self._h = None

    def set_timeout_ms(self, ms: int):
        _lib.check(self.lib.hc_codec_set_timeout_ms(self._h, int(ms)), "set_timeout")

    def status_site(self) -> int:
        """After a time-out: code of the wait that ran out first (see ``hc_codec_status_site``)."""
        with torch.cuda.device(self.device):
            return int(self.lib.hc_codec_status_site(self._h))

    def set_prepass(self, on: bool = True):
        """Large stand-alone inputs: tile offsets from a small pre-pass kernel (default) or from a
        look-back inside the consuming kernel (``False``).  Same bytes either way."""
        _lib.check(self.lib.hc_codec_set_prepass(self._h, 1 if on else 0), "set_prepass")

    def status(self, clear: bool = True) -> int:
        """Synchronises and returns the sticky device status (0 = ok)."""
        with torch.cuda.device(self.device):
            return int(self.lib.hc_codec_status(self._h, 1 if clear else 0))

    # -- helpers ---------------------------------------------------------------------------------
    def _out(self, n, out, size):
        if out is None:
            out = torch.empty(max_compressed_bytes(n) + 16, dtype=torch.uint8, device=self.device)
        if size is None:
            size = torch.zeros(1, dtype=torch.int64, device=self.device)
        return out, size

    @staticmethod
    def _check_f32(x):
        if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
            raise ValueError("expected a contiguous float32 CUDA tensor")

    # -- codec -----------------------------------------------------------------------------------
    def compress(self, x: torch.Tensor, eb: float, mode="outlier", out=None, size=None):
        self._check_f32(x)
        n = x.numel()
        out, size = self._out(n, out, size)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_compress(self._h, x.data_ptr(), n, eb, _mode(mode), out.data_ptr(), out.numel(),
                                            size.data_ptr(), _stream_ptr()), "compress")
        return out, size

    def decompress(self, stream: torch.Tensor, n: int, eb: float, mode="outlier", out=None, stream_bytes=None):
        if out is None:
            out = torch.empty(n, dtype=torch.float32, device=self.device)
        self._check_f32(out)
        nbytes = stream.numel() if stream_bytes is None else int(stream_bytes)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_decompress(self._h, stream.data_ptr(), nbytes, n, eb, _mode(mode), out.data_ptr(),
                                              _stream_ptr()), "decompress")
        return out

    def decompress_flagged(self, stream: torch.Tensor, n: int, eb: float, tile_flags: torch.Tensor, want: int,
                           mode="outlier", out=None, stream_bytes=None):
        """Decode tile by tile as the producer publishes ``tile_flags[t] = want << 40 | payload offset``
        (int64, one word per ``tile_elems`` values; ``want`` is a non-zero 24-bit tag)."""
        if out is None:
            out = torch.empty(n, dtype=torch.float32, device=self.device)
        nbytes = stream.numel() if stream_bytes is None else int(stream_bytes)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_decompress_flagged(self._h, stream.data_ptr(), nbytes, n, eb, _mode(mode),
                                                      out.data_ptr(), tile_flags.data_ptr(), int(want),
                                                      _stream_ptr()), "decompress_flagged")
        return out

    @property
    def tile_elems(self) -> int:
        return int(self.lib.hc_tile_elems())

    def hom_add(self, stream: torch.Tensor, local: torch.Tensor, eb: float, mode="outlier", out=None, size=None,
                stream_bytes=None):
        """stream (+) fp32 -> stream (fused quantise + add in the delta domain + re-encode)."""
        self._check_f32(local)
        n = local.numel()
        out, size = self._out(n, out, size)
        nbytes = stream.numel() if stream_bytes is None else int(stream_bytes)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_hom_add_f32(self._h, stream.data_ptr(), nbytes, local.data_ptr(), n, eb,
                                               _mode(mode), out.data_ptr(), out.numel(), size.data_ptr(),
                                               _stream_ptr()), "hom_add")
        return out, size

    def compress_batch(self, xs, eb: float, mode="outlier"):
        """Compress up to 8 tensors with one launch; returns (list of stream buffers, int64 sizes tensor)."""
        import ctypes as C

        k = len(xs)
        for x in xs:
            self._check_f32(x)
        cap = max(max_compressed_bytes(x.numel()) for x in xs) + 16
        outs = [torch.empty(cap, dtype=torch.uint8, device=self.device) for _ in xs]
        sizes = torch.zeros(k, dtype=torch.int64, device=self.device)
        xp = (C.c_void_p * k)(*[x.data_ptr() for x in xs])
        ns = (C.c_size_t * k)(*[x.numel() for x in xs])
        op = (C.c_void_p * k)(*[o.data_ptr() for o in outs])
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_compress_batch(self._h, k, xp, ns, eb, _mode(mode), op, cap, sizes.data_ptr(),
                                                  _stream_ptr()), "compress_batch")
        return outs, sizes

    def hom_add_multi(self, streams, local: torch.Tensor, eb: float, mode="outlier", stream_bytes=None):
        """streams[0] (+) ... (+) streams[k-1] (+) fp32 -> stream, all summed in the delta domain."""
        import ctypes as C

        self._check_f32(local)
        k, n = len(streams), local.numel()
        out, size = self._out(n, None, None)
        sp = (C.c_void_p * k)(*[s.data_ptr() for s in streams])
        nb = (C.c_size_t * k)(*[(s.numel() if stream_bytes is None else int(stream_bytes[i]))
                                for i, s in enumerate(streams)])
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_hom_add_multi(self._h, k, sp, nb, local.data_ptr(), n, eb, _mode(mode),
                                                 out.data_ptr(), out.numel(), size.data_ptr(), _stream_ptr()),
                       "hom_add_multi")
        return out, size

    def decompress_sum(self, streams, n: int, eb: float, out=None, stream_bytes=None):
        """Decode up to 8 streams of the same ``n`` values and add them in the quantised domain with
        one kernel: the values ``decompress(hom_add(... hom_add(s0, s1) ...))`` would give."""
        import ctypes as C

        k = len(streams)
        if out is None:
            out = torch.empty(n, dtype=torch.float32, device=self.device)
        self._check_f32(out)
        sp = (C.c_void_p * k)(*[s.data_ptr() for s in streams])
        nb = (C.c_size_t * k)(*[(s.numel() if stream_bytes is None else int(stream_bytes[i]))
                                for i, s in enumerate(streams)])
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_decompress_sum(self._h, k, sp, nb, n, eb, out.data_ptr(), _stream_ptr()),
                       "decompress_sum")
        return out

    def quant_pred(self, x: torch.Tensor, eb: float, mode="outlier", out=None):
        self._check_f32(x)
        n = x.numel()
        if out is None:
            out = torch.empty((n + 31) // 32 * 32, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_quant_pred(x.data_ptr(), n, eb, _mode(mode), out.data_ptr(), _stream_ptr()),
                       "quant_pred")
        return out

    def hom_add_deltas(self, stream: torch.Tensor, deltas: torch.Tensor, n: int, mode="outlier", out=None, size=None,
                       stream_bytes=None):
        out, size = self._out(n, out, size)
        nbytes = stream.numel() if stream_bytes is None else int(stream_bytes)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_hom_add_i32(self._h, stream.data_ptr(), nbytes, deltas.data_ptr(), n, _mode(mode),
                                               out.data_ptr(), out.numel(), size.data_ptr(), _stream_ptr()),
                       "hom_add_deltas")
        return out, size

    def hom_add_streams(self, a: torch.Tensor, b: torch.Tensor, n: int, mode="outlier", out=None, size=None,
                        a_bytes=None, b_bytes=None):
        out, size = self._out(n, out, size)
        na = a.numel() if a_bytes is None else int(a_bytes)
        nb = b.numel() if b_bytes is None else int(b_bytes)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_hom_add_stream(self._h, a.data_ptr(), na, b.data_ptr(), nb, n, _mode(mode),
                                                  out.data_ptr(), out.numel(), size.data_ptr(), _stream_ptr()),
                       "hom_add_streams")
        return out, size

    def sum(self, dst, a, b, c=None, d=None):
        n = dst.numel()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hc_sum(dst.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else None,
                                       d.data_ptr() if d is not None else None, n, _stream_ptr()), "sum")
        return dst
