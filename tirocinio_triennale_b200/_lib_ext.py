"""Signatures of the collective / compatibility entry points of libhomcomp_b200.so."""
from __future__ import annotations

import ctypes as C

vp = C.c_void_p


def declare(lib):
    sz, f, i, u = C.c_size_t, C.c_float, C.c_int, C.c_uint
    sigs = {}
    for name, args in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = i
            fn.argtypes = args
