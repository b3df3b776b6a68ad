"""Property tests of the portable codec (no GPU): for arbitrary finite inputs inside the contract the
stream round trip reproduces the quantiser, the homomorphic adds are exact integer additions in the
quantised domain whatever the grouping, and sizes are what the rate bytes say."""
import numpy as np
from hypothesis import given, settings, strategies as st
from hypothesis.extra import numpy as hnp

from tirocinio_triennale_b200 import ops

MODES = ["outlier", "plain", "vec"]


def _arrays(max_abs=1e4):
    return st.integers(min_value=1, max_value=300).flatmap(
        lambda n: hnp.arrays(np.float32, n, elements=st.floats(-max_abs, max_abs, width=32, allow_nan=False,
                                                               allow_infinity=False)))


@settings(max_examples=60, deadline=None)
@given(x=_arrays(), eb=st.sampled_from([1e-1, 1e-2, 1e-3]), mode=st.sampled_from(MODES))
def test_round_trip_is_the_quantiser(x, eb, mode):
    n = x.size
    s = ops.cpu_compress(x, eb, mode)
    assert s.size == ops.cpu_stream_size(s, n) <= ops.max_compressed_bytes(n)
    q = ops.cpu_quantize(x, eb)
    np.testing.assert_array_equal(ops.cpu_decode_quant(s, n, mode), q)
    np.testing.assert_array_equal(ops.cpu_decompress(s, n, eb, mode), ops.cpu_dequantize(q, eb))
    # the bound itself, with room for the fp32 rounding of x * r and q * 2 eb
    assert np.abs(x.astype(np.float64) - ops.cpu_decompress(s, n, eb, mode)).max() <= eb * (1 + 1e-3) + 1e4 * 3e-7


@settings(max_examples=60, deadline=None)
@given(data=st.data(), eb=st.sampled_from([1e-2, 1e-3]), mode=st.sampled_from(MODES))
def test_homomorphic_adds_are_integer_additions(data, eb, mode):
    x = data.draw(_arrays())
    n = x.size
    elems = st.floats(-1e4, 1e4, width=32, allow_nan=False, allow_infinity=False)
    y = data.draw(hnp.arrays(np.float32, n, elements=elems))
    z = data.draw(hnp.arrays(np.float32, n, elements=elems))
    qx, qy, qz = (ops.cpu_quantize(v, eb).astype(np.int64) for v in (x, y, z))
    sx, sy, sz = (ops.cpu_compress(v, eb, mode) for v in (x, y, z))
    # stream (+) fp32, stream (+) stream, stream (+) int32 deltas: the same integers
    a = ops.cpu_hom_add(sx, y, eb, mode)
    b = ops.cpu_hom_add_streams(sx, sy, n, mode)
    c = ops.cpu_hom_add_deltas(sx, ops.cpu_quant_pred(y, eb, mode), n, mode)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(a, c)
    np.testing.assert_array_equal(ops.cpu_decode_quant(a, n, mode).astype(np.int64), qx + qy)
    # grouping does not matter: (x + y) + z and x + (y + z) give the same bytes
    left = ops.cpu_hom_add_streams(b, sz, n, mode)
    right = ops.cpu_hom_add_streams(sx, ops.cpu_hom_add_streams(sy, sz, n, mode), n, mode)
    np.testing.assert_array_equal(left, right)
    np.testing.assert_array_equal(ops.cpu_decode_quant(left, n, mode).astype(np.int64), qx + qy + qz)


@settings(max_examples=25, deadline=None)
@given(data=st.data(), world=st.integers(min_value=1, max_value=5), eb=st.sampled_from([1e-2, 1e-3]))
def test_ring_allreduce_is_the_sum_of_the_quantised_inputs(data, world, eb):
    n = data.draw(st.integers(min_value=1, max_value=400))
    elems = st.floats(-1e3, 1e3, width=32, allow_nan=False, allow_infinity=False)
    bufs = [data.draw(hnp.arrays(np.float32, n, elements=elems)) for _ in range(world)]
    outs = ops.cpu_ring_allreduce(bufs, eb)
    q = sum(ops.cpu_quantize(b, eb).astype(np.int64) for b in bufs)
    want = ops.cpu_dequantize(q.astype(np.int32), eb)
    for o in outs:  # every rank holds the same bits
        np.testing.assert_array_equal(o, want)
