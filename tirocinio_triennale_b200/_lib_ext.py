"""Signatures of the collective / compatibility entry points of libhomcomp_b200.so."""
from __future__ import annotations

import ctypes as C

vp = C.c_void_p

SEND_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t)
RECV_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t))


class HostTransport(C.Structure):
    _fields_ = [("send", SEND_FN), ("recv", RECV_FN), ("user", C.c_void_p)]


def declare(lib):
    sz, f, i, u = C.c_size_t, C.c_float, C.c_int, C.c_uint
    lib.hc_comm_symmetric_bytes.restype = sz
    lib.hc_comm_symmetric_bytes.argtypes = [i, sz]
    lib.hc_comm_destroy.restype = None
    lib.hc_comm_destroy.argtypes = [vp]
    sigs = {
        "hc_comm_create": [C.POINTER(vp), i, i, sz, C.POINTER(vp), vp],
        "hc_comm_set_timeout_ms": [vp, u],
        "hc_comm_status": [vp, i],
        "hc_comm_status_site": [vp],
        "hc_allreduce": [vp, vp, vp, sz, f, vp],
        "hc_allreduce_raw": [vp, vp, vp, sz, vp],
        "hc_allreduce_mixed": [vp, vp, vp, vp, sz, f, vp],
        "hc_comm_set_inter": [vp, vp],
        "hc_comm_call_numbers": [vp, C.POINTER(C.c_uint32)],
        "hc_comm_resync": [vp, C.c_uint32, C.c_uint32],
        "hc_allreduce_host": [vp, vp, vp, sz, f, i, vp],
        "hc_comm_set_trace": [vp, i],
        "hc_comm_set_algorithm": [vp, i],
        "hc_comm_set_small_count": [vp, sz],
        "hc_comm_last_form": [vp],
        "hc_comm_set_overlap": [vp, i],
        "hc_comm_set_shares": [vp, i, i, i],
        "hc_comm_set_sparse_tiles": [vp, i],
        "hc_comm_last_step_ms": [vp, C.POINTER(C.c_float), i],
        "hc_comm_last_stream_bytes": [vp, C.POINTER(C.c_uint64), i],
        "hc_allreduce_host_staged": [vp, C.POINTER(HostTransport), i, i, vp, vp, sz, f, vp],
        "hc_comm_set_host_transport": [vp, C.POINTER(HostTransport)],
        "hc_comm_allreduce_host_staged": [vp, vp, vp, sz, f, vp],
        "hc_ipc_alloc": [C.POINTER(vp), sz, C.c_char_p],
        "hc_ipc_open": [C.c_char_p, C.POINTER(vp)],
        "hc_ipc_close": [vp],
        "hc_ipc_free": [vp],
    }
    for name, args in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = i
            fn.argtypes = args
