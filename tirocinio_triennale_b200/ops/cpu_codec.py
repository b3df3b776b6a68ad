"""NumPy front end of the portable codec (the oracle).

Streams are ``numpy.uint8`` arrays holding exactly the stream bytes.  Behaviour follows the
reference kernels (HomComp/src/GSZ.cu:33-1473, HomComp/src/homcomp.cu:2923-4311) with their
zero-block defects replaced by the intended arithmetic.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib, MODES


def _mode(mode) -> int:
    return MODES[mode] if isinstance(mode, str) else int(mode)


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32).reshape(-1))


def _u8(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.uint8).reshape(-1))


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def max_compressed_bytes(n: int) -> int:
    return int(_lib.cpu().hc_max_compressed_bytes(n))


def rate_bytes(n: int) -> int:
    return int(_lib.cpu().hc_rate_bytes(n))


def chunk_elems(count: int, world: int) -> int:
    return int(_lib.cpu().hc_chunk_elems(count, world))


def cpu_quantize(x, eb: float) -> np.ndarray:
    x = _f32(x)
    q = np.empty(x.size, dtype=np.int32)
    _lib.check(_lib.cpu().hc_cpu_quantize(_p(x), x.size, eb, _p(q)), "quantize")
    return q


def cpu_dequantize(q, eb: float) -> np.ndarray:
    q = np.ascontiguousarray(np.asarray(q, dtype=np.int32).reshape(-1))
    x = np.empty(q.size, dtype=np.float32)
    _lib.check(_lib.cpu().hc_cpu_dequantize(_p(q), q.size, eb, _p(x)), "dequantize")
    return x


def cpu_quant_pred(x, eb: float, mode="outlier") -> np.ndarray:
    x = _f32(x)
    nb = (x.size + 31) // 32
    d = np.empty(nb * 32, dtype=np.int32)
    _lib.check(_lib.cpu().hc_cpu_quant_pred(_p(x), x.size, eb, _mode(mode), _p(d)), "quant_pred")
    return d


def cpu_compress(x, eb: float, mode="outlier") -> np.ndarray:
    x = _f32(x)
    cap = max_compressed_bytes(x.size)
    out = np.empty(cap, dtype=np.uint8)
    size = C.c_size_t(0)
    _lib.check(_lib.cpu().hc_cpu_compress(_p(x), x.size, eb, _mode(mode), _p(out), cap, C.byref(size)), "compress")
    return out[: size.value].copy()


def cpu_decompress(stream, n: int, eb: float, mode="outlier") -> np.ndarray:
    s = _u8(stream)
    x = np.empty(n, dtype=np.float32)
    _lib.check(_lib.cpu().hc_cpu_decompress(_p(s), s.size, n, eb, _mode(mode), _p(x)), "decompress")
    return x


def cpu_decode_quant(stream, n: int, mode="outlier") -> np.ndarray:
    s = _u8(stream)
    q = np.empty(n, dtype=np.int32)
    _lib.check(_lib.cpu().hc_cpu_decode_quant(_p(s), s.size, n, _mode(mode), _p(q)), "decode_quant")
    return q


def cpu_hom_add(stream, local, eb: float, mode="outlier") -> np.ndarray:
    """stream (+) fp32 values -> stream, added in the quantised delta domain."""
    s, x = _u8(stream), _f32(local)
    cap = max_compressed_bytes(x.size)
    out = np.empty(cap, dtype=np.uint8)
    size = C.c_size_t(0)
    _lib.check(_lib.cpu().hc_cpu_hom_add_f32(_p(s), s.size, _p(x), x.size, eb, _mode(mode), _p(out), cap,
                                             C.byref(size)), "hom_add")
    return out[: size.value].copy()


def cpu_hom_add_deltas(stream, deltas, n: int, mode="outlier") -> np.ndarray:
    s = _u8(stream)
    d = np.ascontiguousarray(np.asarray(deltas, dtype=np.int32).reshape(-1))
    cap = max_compressed_bytes(n)
    out = np.empty(cap, dtype=np.uint8)
    size = C.c_size_t(0)
    _lib.check(_lib.cpu().hc_cpu_hom_add_i32(_p(s), s.size, _p(d), n, _mode(mode), _p(out), cap, C.byref(size)),
               "hom_add_deltas")
    return out[: size.value].copy()


def cpu_hom_add_streams(a, b, n: int, mode="outlier") -> np.ndarray:
    a, b = _u8(a), _u8(b)
    cap = max_compressed_bytes(n)
    out = np.empty(cap, dtype=np.uint8)
    size = C.c_size_t(0)
    _lib.check(_lib.cpu().hc_cpu_hom_add_stream(_p(a), a.size, _p(b), b.size, n, _mode(mode), _p(out), cap,
                                                C.byref(size)), "hom_add_streams")
    return out[: size.value].copy()


def cpu_stream_size(stream, n: int) -> int:
    s = _u8(stream)
    size = C.c_size_t(0)
    _lib.check(_lib.cpu().hc_cpu_stream_size(_p(s), s.size, n, C.byref(size)), "stream_size")
    return int(size.value)


def cpu_ring_allreduce(bufs, eb: float, return_hop_bytes: bool = False):
    """Compressed ring allreduce of ``len(bufs)`` host ranks simulated in this process."""
    arrs = [_f32(b) for b in bufs]
    P, n = len(arrs), arrs[0].size
    assert all(a.size == n for a in arrs)
    outs = [np.zeros(n, dtype=np.float32) for _ in range(P)]
    ins_p = (C.c_void_p * P)(*[a.ctypes.data for a in arrs])
    outs_p = (C.c_void_p * P)(*[o.ctypes.data for o in outs])
    hops = (C.c_size_t * (P * P))()
    _lib.check(_lib.cpu().hc_cpu_ring_allreduce(ins_p, outs_p, P, n, eb, hops), "cpu_ring_allreduce")
    if return_hop_bytes:
        return outs, np.array(list(hops), dtype=np.int64).reshape(P, P)
    return outs
