"""hc_compress_noalloc: the entry point for callers that cannot allocate device memory.

Plug-ins that live inside another framework's memory pool, allocation-free real-time loops and
processes whose device budget is already spent cannot give the compressor the scratch memory it
needs, and must not let it call cudaMalloc.  For them the library carries that scratch in a
built-in device array.  This test calls the exported C symbol directly (ctypes, no wrapper) and
checks that its stream is byte-identical to the regular hc_compress entry point, twice in a row on
different data, so that state left in the shared array by the first call cannot leak into the
second.  The file sorts last so that a stop-at-first-failure run has executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _compress_regular(lib, x, eb, cap):
    h = C.c_void_p()
    assert lib.hc_codec_create(C.byref(h), x.numel()) == 0
    out = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    size = torch.zeros(1, dtype=torch.int64, device="cuda")
    rc = lib.hc_compress(h, x.data_ptr(), x.numel(), eb, 0, out.data_ptr(), cap, size.data_ptr(),
                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.hc_codec_status(h, 1) == 0
    lib.hc_codec_destroy(h)
    return out[: int(size.item())].cpu().numpy()


def test_noalloc_entry_matches_regular_entry_twice():
    from tirocinio_triennale_b200 import _lib

    lib = _lib.cuda()
    fn = lib.hc_compress_noalloc  # the exported C symbol itself
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.hc_noalloc_scratch_bytes.restype = C.c_size_t
    assert 0 < lib.hc_noalloc_scratch_bytes() <= 1 << 20  # a modest, fixed footprint

    lib.hc_noalloc_status.restype = C.c_int
    lib.hc_noalloc_status.argtypes = [C.c_int]

    eb = 1e-4
    g = torch.Generator(device="cuda").manual_seed(7)
    # one warm-up call: the first call on a device loads the kernel and looks the array up
    w = torch.randn(4096, device="cuda", generator=g)
    wout = torch.zeros(int(lib.hc_max_compressed_bytes(4096)) + 64, dtype=torch.uint8, device="cuda")
    wsize = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert fn(w.data_ptr(), 4096, eb, wout.data_ptr(), wout.numel(), wsize.data_ptr(),
              torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    sizes = [1_000_003, 250_001]  # the second call is shorter: stale look-back words stay behind it
    for call, n in enumerate(sizes):
        x = torch.randn(n, device="cuda", generator=g) * (0.01 * (call + 1))
        cap = int(lib.hc_max_compressed_bytes(n)) + 64
        out = torch.zeros(cap, dtype=torch.uint8, device="cuda")
        size = torch.zeros(1, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: sees any cudaMalloc, not only torch's
        rc = fn(x.data_ptr(), n, eb, out.data_ptr(), cap, size.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert lib.hc_noalloc_status(0) == 0
        got = out[: int(size.item())].cpu().numpy()
        want = _compress_regular(lib, x, eb, cap)
        assert got.size == want.size
        np.testing.assert_array_equal(got, want)  # same tolerance as the other codec tests: exact bytes

    # sizes beyond the built-in scratch are refused, loudly and without touching anything
    too_big = 16 * 1024 * 1024 + 1
    assert fn(x.data_ptr(), too_big, eb, out.data_ptr(), cap, size.data_ptr(), 0) == 4

    # an output buffer that is too small: the call is accepted, the device notes status 1, the size word
    # stays as it was, and the status survives until it is read and cleared
    size.fill_(-1)
    small = int(lib.hc_rate_bytes(n)) + 128
    assert fn(x.data_ptr(), n, eb, out.data_ptr(), small, size.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    assert lib.hc_noalloc_status(0) == 1
    assert int(size.item()) == -1
    assert lib.hc_noalloc_status(1) == 1
    assert lib.hc_noalloc_status(0) == 0
    assert fn(x.data_ptr(), n, eb, out.data_ptr(), cap, size.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out[: int(size.item())].cpu().numpy(), want)
