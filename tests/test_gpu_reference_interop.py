"""Stream interchange with the reference kernels (compiled by baseline/build_ref.py; the only change
inside the kernels is that the shared variable the first chunk reads uninitialised is set to 0):
streams written by either implementation decode in the other, and for inputs that are whole chunks
the bytes are identical."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm

    lib = reference_arm._load()
    if lib is None:
        pytest.skip("reference library not built")
    return lib


def _data(n, seed, kind):
    from datasets import gradient_like, smooth

    return (gradient_like if kind == "gradient" else smooth)(n, seed)


@pytest.mark.parametrize("kind", ["gradient", "smooth"])
@pytest.mark.parametrize("n", [32768, 5 * 32768])
def test_streams_are_interchangeable(ref, kind, n):
    from tirocinio_triennale_b200 import ops

    eb = 1e-4
    x = _data(n, 3, kind)
    gx = torch.from_numpy(x).cuda()
    codec = ops.Codec(n)
    ours, size = codec.compress(gx, eb)
    ours_n = int(size.item())
    theirs = torch.zeros(4 * n + 65536, dtype=torch.uint8, device="cuda")
    reported = ref.ref_compress(gx.data_ptr(), theirs.data_ptr(), n, eb)
    torch.cuda.synchronize()
    # the reference reports the true length plus one byte per block
    assert reported == ours_n + ops.rate_bytes(n)
    np.testing.assert_array_equal(theirs[:ours_n].cpu().numpy(), ours[:ours_n].cpu().numpy())
    # each decodes the other's stream
    y = codec.decompress(theirs, n, eb, stream_bytes=reported)
    z = torch.zeros(n, device="cuda")
    ref.ref_decompress(z.data_ptr(), ours.data_ptr(), n, ours_n, eb)
    torch.cuda.synchronize()
    want = ops.cpu_decompress(ours[:ours_n].cpu().numpy(), n, eb)
    np.testing.assert_array_equal(y.cpu().numpy(), want)
    np.testing.assert_array_equal(z.cpu().numpy(), want)
    assert codec.status() == 0


def test_homomorphic_sum_matches_reference_on_dense_data(ref):
    from tirocinio_triennale_b200 import ops

    n, eb = 4 * 32768, 1e-4
    x, y = _data(n, 5, "gradient"), _data(n, 6, "gradient")  # no zero blocks: the reference mishandles those
    gx, gy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    codec = ops.Codec(n)
    s, size = codec.compress(gx, eb)
    ours, size2 = codec.hom_add(s, gy, eb, stream_bytes=int(size.item()))
    theirs = torch.zeros(4 * n + 65536, dtype=torch.uint8, device="cuda")
    reported = ref.ref_hom_sum_F(s.data_ptr(), gy.data_ptr(), theirs.data_ptr(), n, eb, int(size.item()))
    torch.cuda.synchronize()
    m = int(size2.item())
    assert reported == m + ops.rate_bytes(n)
    np.testing.assert_array_equal(theirs[:m].cpu().numpy(), ours[:m].cpu().numpy())
