"""Stream invariants of the portable codec (no GPU)."""
import numpy as np
import pytest

from tirocinio_triennale_b200 import ops
from datasets import ALL, SIZES


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("mode", ["outlier", "plain", "vec"])
def test_roundtrip_error_bound(name, n, mode):
    eb = 1e-3
    x = ALL[name](n, seed=n)
    s = ops.cpu_compress(x, eb, mode)
    assert s.size <= ops.max_compressed_bytes(n)
    assert ops.cpu_stream_size(s, n) == s.size
    y = ops.cpu_decompress(s, n, eb, mode)
    q = ops.cpu_quantize(x, eb)
    np.testing.assert_array_equal(y, ops.cpu_dequantize(q, eb))
    # |x - 2 eb q| <= eb up to fp32 rounding of the products
    assert np.abs(x.astype(np.float64) - y).max() <= eb * (1 + 1e-3) + np.abs(x).max() * 2e-7


def test_quantiser_is_round_half_away_from_zero():
    eb = 0.5  # recip = 1: q = round-half-away(x)
    x = np.array([0.0, 0.49, 0.5, 1.5, 2.5, -0.49, -0.5, -0.51, -1.5, -2.5, 1e12], dtype=np.float32)
    q = ops.cpu_quantize(x, eb)
    assert q.tolist() == [0, 0, 1, 2, 3, 0, 0, -1, -2, -3, 2**31 - 1]


def test_stream_layout_plain_block():
    # one block, deltas (+1, 0, ..., 0, +2 at element 9, -2 at element 10, -1 at element 31): plain mode, F = 2
    eb = 0.5
    x = np.ones(32, dtype=np.float32)
    x[9] = 3.0
    x[31] = 0.0
    s = ops.cpu_compress(x, eb)
    assert s.size == 1024 + 4 + 8
    assert s[0] == 2 and not s[1:1024].any()
    body = s[1024:]
    assert body[:4].tolist() == [0, 0x20, 0, 1]        # sign map: elements 10 and 31 negative
    assert body[4:8].tolist() == [0x80, 0, 0, 1]       # plane 0: elements 0 and 31
    assert body[8:12].tolist() == [0, 0x60, 0, 0]      # plane 1: elements 9 and 10


def test_stream_layout_outlier_block():
    eb = 0.5
    x = np.full(32, 1000.0, dtype=np.float32)  # d0 = 1000, the rest 0 -> outlier mode, F = 0, 2 outlier bytes
    s = ops.cpu_compress(x, eb)
    assert s[0] == (0x80 | (1 << 5) | 0)
    assert s.size == 1024 + 2 + 4
    assert s[1024:1026].tolist() == [1000 & 255, 1000 >> 8]
    assert not s[1026:1030].any()
    np.testing.assert_array_equal(ops.cpu_decompress(s, 32, eb), x)
    # plain codec never takes the outlier layout
    sp = ops.cpu_compress(x, eb, "plain")
    assert sp[0] == 10 and sp.size == 1024 + 4 + 40
    np.testing.assert_array_equal(ops.cpu_decompress(sp, 32, eb, "plain"), x)
    # a plain stream is a valid outlier-codec stream
    np.testing.assert_array_equal(ops.cpu_decompress(sp, 32, eb, "outlier"), x)


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("n", [1, 33, 8193, 70001])
def test_hom_add_is_exact_in_the_quantised_domain(name, n):
    eb = 1e-4 if name != "wide" else 1e-2
    x, y = ALL[name](n, seed=1), ALL[name](n, seed=2)
    sx = ops.cpu_compress(x, eb)
    sxy = ops.cpu_hom_add(sx, y, eb)
    q = ops.cpu_decode_quant(sxy, n)
    np.testing.assert_array_equal(q, ops.cpu_quantize(x, eb) + ops.cpu_quantize(y, eb))
    # the three adds agree byte for byte
    np.testing.assert_array_equal(sxy, ops.cpu_hom_add_deltas(sx, ops.cpu_quant_pred(y, eb), n))
    np.testing.assert_array_equal(sxy, ops.cpu_hom_add_streams(sx, ops.cpu_compress(y, eb), n))


def test_hom_add_on_zero_and_outlier_f0_blocks():
    # the two corner cases the reference mishandles: incoming zero block, outlier block with F = 0
    eb = 0.5
    zero = np.zeros(64, dtype=np.float32)
    spike = np.zeros(64, dtype=np.float32)
    spike[:32] = -700.0
    y = np.arange(64, dtype=np.float32)
    for a in (zero, spike):
        s = ops.cpu_hom_add(ops.cpu_compress(a, eb), y, eb)
        np.testing.assert_array_equal(ops.cpu_decompress(s, 64, eb), a + y)


def test_truncated_stream_is_reported():
    from tirocinio_triennale_b200._lib import HomCompError

    x = ALL["gradient"](5000)
    s = ops.cpu_compress(x, 1e-4)
    with pytest.raises(HomCompError):
        ops.cpu_decompress(s[:-10], x.size, 1e-4)


@pytest.mark.parametrize("P", [1, 2, 3, 8])
def test_cpu_ring_allreduce(P):
    n, eb = 50001, 1e-4
    bufs = [ALL["smooth"](n, seed=r) for r in range(P)]
    outs, hops = ops.cpu_ring_allreduce(bufs, eb, return_hop_bytes=True)
    exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
    for o in outs:
        np.testing.assert_array_equal(o, outs[0])  # every rank decodes the same bytes
    assert np.abs(outs[0] - exact).max() <= P * eb * 1.01
    # homomorphic property: result is exactly 2 eb * sum of the quantised inputs
    qsum = sum(ops.cpu_quantize(b, eb).astype(np.int64) for b in bufs).astype(np.int32)
    np.testing.assert_array_equal(outs[0], ops.cpu_dequantize(qsum, eb))
    assert (hops > 0).all()


def test_host_affinity_helper_never_raises():
    """Used by bench.py before pinned buffers are allocated; on a machine without a GPU (or without the
    sysfs entries) it must say so instead of failing."""
    from tirocinio_triennale_b200.utils import timing

    msg = timing.bind_host_thread_near_gpu(0)
    assert isinstance(msg, str) and msg.startswith("gpu 0")
