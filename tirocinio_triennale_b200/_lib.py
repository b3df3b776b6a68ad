"""ctypes bindings of the native libraries.

``cpu()`` always works (g++ build of the portable codec).  ``cuda()`` is the sm_100a library and
raises if it cannot be loaded: on a machine with a GPU nothing in this package falls back to
PyTorch code silently.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from . import _build

_lock = threading.Lock()
_cpu = None
_cuda = None

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int32)
szp = C.POINTER(C.c_size_t)
vp = C.c_void_p


def _declare_cpu(lib):
    sz, f, i = C.c_size_t, C.c_float, C.c_int
    lib.hc_max_compressed_bytes.restype = sz
    lib.hc_max_compressed_bytes.argtypes = [sz]
    lib.hc_rate_bytes.restype = sz
    lib.hc_rate_bytes.argtypes = [sz]
    lib.hc_chunk_elems.restype = sz
    lib.hc_chunk_elems.argtypes = [sz, i]
    sigs = {
        "hc_cpu_quantize": [vp, sz, f, vp],
        "hc_cpu_dequantize": [vp, sz, f, vp],
        "hc_cpu_quant_pred": [vp, sz, f, i, vp],
        "hc_cpu_compress": [vp, sz, f, i, vp, sz, szp],
        "hc_cpu_decompress": [vp, sz, sz, f, i, vp],
        "hc_cpu_decode_quant": [vp, sz, sz, i, vp],
        "hc_cpu_hom_add_f32": [vp, sz, vp, sz, f, i, vp, sz, szp],
        "hc_cpu_hom_add_i32": [vp, sz, vp, sz, i, vp, sz, szp],
        "hc_cpu_hom_add_stream": [vp, sz, vp, sz, sz, i, vp, sz, szp],
        "hc_cpu_stream_size": [vp, sz, sz, szp],
        "hc_cpu_ring_allreduce": [C.POINTER(vp), C.POINTER(vp), i, sz, f, szp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.restype = i
        fn.argtypes = args


def _declare_cuda(lib):
    sz, f, i = C.c_size_t, C.c_float, C.c_int
    lib.hc_codec_workspace_bytes.restype = sz
    lib.hc_codec_workspace_bytes.argtypes = [sz]
    lib.hc_tile_elems.restype = sz
    lib.hc_tile_elems.argtypes = []
    lib.hc_status_string.restype = C.c_char_p
    lib.hc_status_string.argtypes = [i]
    lib.hc_codec_destroy.restype = None
    lib.hc_codec_destroy.argtypes = [vp]
    sigs = {
        "hc_codec_create": [C.POINTER(vp), sz],
        "hc_codec_create_in": [C.POINTER(vp), vp, sz, sz, vp],
        "hc_codec_set_timeout_ms": [vp, C.c_uint],
        "hc_codec_set_prepass": [vp, i],
        "hc_codec_status_site": [vp],
        "hc_codec_status": [vp, i],
        "hc_compress": [vp, vp, sz, f, i, vp, sz, vp, vp],
        "hc_decompress": [vp, vp, sz, sz, f, i, vp, vp],
        "hc_decompress_flagged": [vp, vp, sz, sz, f, i, vp, vp, C.c_uint, vp],
        "hc_decompress_sum": [vp, i, vp, vp, sz, f, vp, vp],
        "hc_hom_add_f32": [vp, vp, sz, vp, sz, f, i, vp, sz, vp, vp],
        "hc_hom_add_i32": [vp, vp, sz, vp, sz, i, vp, sz, vp, vp],
        "hc_hom_add_stream": [vp, vp, sz, vp, sz, sz, i, vp, sz, vp, vp],
        "hc_quant_pred": [vp, sz, f, i, vp, vp],
        "hc_compress_batch": [vp, i, vp, vp, f, i, vp, sz, vp, vp],
        "hc_hom_add_multi": [vp, i, vp, vp, vp, sz, f, i, vp, sz, vp, vp],
        "hc_sum": [vp, vp, vp, vp, vp, sz, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.restype = i
        fn.argtypes = args


def cpu():
    global _cpu
    with _lock:
        if _cpu is None:
            import os

            # HC_CPU_LIB: load this build of the portable library instead (e.g. one compiled with sanitizers)
            path = os.environ.get("HC_CPU_LIB") or _build.build_cpu()
            lib = C.CDLL(str(path))
            _declare_cpu(lib)
            _cpu = lib
    return _cpu


def cuda():
    """The sm_100a library.  Built on demand when nvcc is present; raises otherwise.
    With ``HC_TIMELINE=1`` in the environment the instrumented build is loaded instead
    (``utils/timeline.py``)."""
    global _cuda
    with _lock:
        if _cuda is None:
            import os

            tl = os.environ.get("HC_TIMELINE", "0") not in ("", "0")
            path = Path(_build.LIBDIR / ("libhomcomp_b200_tl.so" if tl else "libhomcomp_b200.so"))
            if os.environ.get("HC_CUDA_LIB"):  # an alternative build of the library (debug, experiment)
                path = Path(os.environ["HC_CUDA_LIB"])
            elif _build.nvcc_path() is not None:
                path = _build.build_cuda(timeline=tl)
            if not path.exists():
                raise RuntimeError("libhomcomp_b200.so is missing and nvcc is not available to build it")
            lib = C.CDLL(str(path))
            _declare_cpu(lib)
            _declare_cuda(lib)
            from . import _lib_ext

            _lib_ext.declare(lib)
            _cuda = lib
    return _cuda


class HomCompError(RuntimeError):
    def __init__(self, status: int, what: str = ""):
        names = {1: "capacity", 2: "truncated", 3: "timeout", 4: "argument", 5: "cuda", 6: "peer"}
        super().__init__("%s failed: status %d (%s)" % (what or "homcomp call", status, names.get(status, "?")))
        self.status = status


def check(status: int, what: str = ""):
    if status != 0:
        raise HomCompError(status, what)
