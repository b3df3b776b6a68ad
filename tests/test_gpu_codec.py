"""sm_100a codec kernels against the CPU oracle: streams must match byte for byte."""
import numpy as np
import pytest
import torch

from tirocinio_triennale_b200 import ops
from datasets import ALL, SIZES

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def codec():
    c = ops.Codec(max_elems=1 << 22)
    yield c
    assert c.status() == 0


def _gpu(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _stream(out, size):
    return out[: int(size.item())].cpu().numpy()


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("n", SIZES)
def test_compress_matches_oracle(codec, name, n):
    eb = 1e-3
    x = ALL[name](n, seed=n)
    out, size = codec.compress(_gpu(x), eb)
    ref = ops.cpu_compress(x, eb)
    got = _stream(out, size)
    assert got.size == ref.size
    np.testing.assert_array_equal(got, ref)
    assert codec.status() == 0


@pytest.mark.parametrize("mode", ["plain", "vec"])
@pytest.mark.parametrize("n", [33, 8193, 100000])
def test_compress_other_modes(codec, mode, n):
    eb = 1e-4
    x = ALL["gradient"](n, seed=3)
    out, size = codec.compress(_gpu(x), eb, mode)
    np.testing.assert_array_equal(_stream(out, size), ops.cpu_compress(x, eb, mode))
    y = codec.decompress(out, n, eb, mode)
    np.testing.assert_array_equal(y.cpu().numpy(), ops.cpu_decompress(ops.cpu_compress(x, eb, mode), n, eb, mode))


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("n", SIZES)
def test_decompress_matches_oracle(codec, name, n):
    eb = 1e-3
    x = ALL[name](n, seed=n + 1)
    s = ops.cpu_compress(x, eb)
    pad = np.concatenate([s, np.zeros(32, np.uint8)])
    y = torch.full((n,), 7.0, device="cuda")  # stale values must be overwritten, zero blocks included
    codec.decompress(_gpu(pad), n, eb, out=y, stream_bytes=s.size)
    np.testing.assert_array_equal(y.cpu().numpy(), ops.cpu_decompress(s, n, eb))
    assert codec.status() == 0


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("n", [1, 33, 8192, 8193, 32769, 262144 + 17])
def test_hom_add_matches_oracle(codec, name, n):
    eb = 1e-4 if name != "wide" else 1e-2
    x, y = ALL[name](n, seed=5), ALL[name](n, seed=6)
    sx = ops.cpu_compress(x, eb)
    ref = ops.cpu_hom_add(sx, y, eb)
    gsx = _gpu(np.concatenate([sx, np.zeros(32, np.uint8)]))
    out, size = codec.hom_add(gsx, _gpu(y), eb, stream_bytes=sx.size)
    np.testing.assert_array_equal(_stream(out, size), ref)
    # two-kernel form: quantise + predict, then add int32 deltas
    d = codec.quant_pred(_gpu(y), eb)
    np.testing.assert_array_equal(d.cpu().numpy(), ops.cpu_quant_pred(y, eb))
    out2, size2 = codec.hom_add_deltas(gsx, d, n, stream_bytes=sx.size)
    np.testing.assert_array_equal(_stream(out2, size2), ref)
    # stream (+) stream
    sy = ops.cpu_compress(y, eb)
    gsy = _gpu(np.concatenate([sy, np.zeros(32, np.uint8)]))
    out3, size3 = codec.hom_add_streams(gsx, gsy, n, a_bytes=sx.size, b_bytes=sy.size)
    np.testing.assert_array_equal(_stream(out3, size3), ref)
    assert codec.status() == 0


def test_unaligned_pointers(codec):
    n, eb = 20000, 1e-3
    x = ALL["smooth"](n + 1)
    gx = _gpu(x)[1:]  # 4-byte aligned only: the plain-load path
    ref = ops.cpu_compress(x[1:], eb)
    buf = torch.zeros(ops.max_compressed_bytes(n) + 64, dtype=torch.uint8, device="cuda")
    out, size = codec.compress(gx.contiguous() if False else gx, eb, out=buf[3:])
    np.testing.assert_array_equal(out[: int(size.item())].cpu().numpy(), ref)
    y = torch.zeros(n + 1, device="cuda")
    codec.decompress(buf[3:], n, eb, out=y[1:], stream_bytes=ref.size)
    np.testing.assert_array_equal(y[1:].cpu().numpy(), ops.cpu_decompress(ref, n, eb))


def test_capacity_and_truncation_are_reported_not_fatal(codec):
    n, eb = 50000, 1e-4
    x = ALL["gradient"](n)
    small = torch.zeros(ops.rate_bytes(n) + 100, dtype=torch.uint8, device="cuda")
    codec.compress(_gpu(x), eb, out=small)
    assert codec.status() == 1  # capacity
    s = ops.cpu_compress(x, eb)
    y = codec.decompress(_gpu(s), n, eb, stream_bytes=s.size - 1000)
    assert codec.status() == 2  # truncated
    assert torch.isfinite(y).all()
    # the handle keeps working afterwards
    out, size = codec.compress(_gpu(x), eb)
    np.testing.assert_array_equal(_stream(out, size), s)
    assert codec.status() == 0


def test_many_launches_reuse_workspace(codec):
    n, eb = 300000, 1e-4
    x = ALL["gradient"](n)
    gx = _gpu(x)
    ref = ops.cpu_compress(x, eb)
    for _ in range(50):
        out, size = codec.compress(gx, eb)
    np.testing.assert_array_equal(_stream(out, size), ref)


def test_large_roundtrip_error_bound(codec):
    n, eb = (1 << 22) - 5, 1e-4
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, device="cuda", generator=g) * 0.01
    out, size = codec.compress(x, eb)
    y = codec.decompress(out, n, eb)
    assert (x - y).abs().max().item() <= eb * 1.001 + 1e-9
    ratio = 4 * n / int(size.item())
    assert 1.5 < ratio < 20
    # against the oracle on the same data
    np.testing.assert_array_equal(_stream(out, size), ops.cpu_compress(x.cpu().numpy(), eb))


def test_sum_kernel(codec):
    a, b, c, d = (torch.randn(100003, device="cuda") for _ in range(4))
    dst = torch.empty_like(a)
    codec.sum(dst, a, b)
    torch.testing.assert_close(dst, a + b, rtol=0, atol=0)
    codec.sum(dst, a, b, c, d)
    torch.testing.assert_close(dst, ((a + b) + c) + d, rtol=0, atol=0)


@pytest.mark.parametrize("lens", [[1000, 1000], [70000, 33, 8193], [32768 * 3, 5, 32768 * 3 - 1, 100, 200000, 1, 4096, 8192]])
def test_batched_compress_matches_oracle(lens):
    eb = 1e-4
    codec = ops.Codec(max_elems=1 << 22)
    xs = [ALL["gradient" if i % 2 else "smooth"](n, seed=i) for i, n in enumerate(lens)]
    outs, sizes = codec.compress_batch([_gpu(x) for x in xs], eb)
    assert codec.status() == 0
    for x, o, sz in zip(xs, outs, sizes.tolist()):
        np.testing.assert_array_equal(o[:sz].cpu().numpy(), ops.cpu_compress(x, eb))


@pytest.mark.parametrize("k", [1, 3, 7])
@pytest.mark.parametrize("n", [33, 8193, 300000])
def test_multi_stream_add_matches_oracle(k, n):
    eb = 1e-4
    codec = ops.Codec(max_elems=1 << 22)
    xs = [ALL["gradient"](n, seed=10 + i) for i in range(k)]
    y = ALL["smooth"](n, seed=99)
    streams = [ops.cpu_compress(x, eb) for x in xs]
    want = ops.cpu_compress(y, eb)
    for s in streams:  # the oracle adds stream by stream; integer sums do not care about the order
        want = ops.cpu_hom_add_streams(want, s, n)
    gs = [_gpu(np.concatenate([s, np.zeros(32, np.uint8)])) for s in streams]
    out, size = codec.hom_add_multi(gs, _gpu(y), eb, stream_bytes=[s.size for s in streams])
    assert codec.status() == 0
    np.testing.assert_array_equal(_stream(out, size), want)


@pytest.mark.parametrize("k", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [1, 33, 8193, 300000, 1100 * 4096 + 7])
def test_decode_and_sum_of_streams_matches_oracle(k, n):
    """One kernel decodes k streams and adds their quantised values: the oracle's chain of stream adds
    followed by one decompress, bit for bit (1100 tiles and more go through the offsets pre-pass)."""
    eb = 1e-4
    codec = ops.Codec(max_elems=8 * n + 8 * 32768)  # room for eight look-back chains of whole chunks
    xs = [ALL["gradient" if i % 2 else "smooth"](n, seed=40 + i) for i in range(k)]
    streams = [ops.cpu_compress(x, eb) for x in xs]
    acc = streams[0]
    for s in streams[1:]:
        acc = ops.cpu_hom_add_streams(acc, s, n)
    want = ops.cpu_decompress(acc, n, eb)
    gs = [_gpu(np.concatenate([s, np.zeros(32, np.uint8)])) for s in streams]
    for _ in range(2):
        out = torch.full((n,), -7.0, device="cuda")
        codec.decompress_sum(gs, n, eb, out=out, stream_bytes=[s.size for s in streams])
        assert codec.status() == 0
        np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("k,n", [(1, 500 * 4096 + 77), (3, 520 * 4096), (7, 1000 * 4096 + 5)])
def test_multi_stream_add_about_one_tile_per_cta(k, n):
    """Tile counts for which the launcher picks the single-stage, four-CTAs-per-SM variant of the
    add kernel (one round of tiles fewer than with three CTAs per SM)."""
    eb = 1e-4
    codec = ops.Codec(max_elems=8 * n)
    xs = [ALL["gradient"](n, seed=20 + i) for i in range(k)]
    y = ALL["gradient"](n, seed=98)
    streams = [ops.cpu_compress(x, eb) for x in xs]
    want = ops.cpu_compress(y, eb)
    for s in streams:
        want = ops.cpu_hom_add_streams(want, s, n)
    gs = [_gpu(np.concatenate([s, np.zeros(32, np.uint8)])) for s in streams]
    for _ in range(2):
        out, size = codec.hom_add_multi(gs, _gpu(y), eb, stream_bytes=[s.size for s in streams])
        assert codec.status() == 0
        np.testing.assert_array_equal(_stream(out, size), want)


@pytest.mark.parametrize("world,n", [(1, 5000), (2, 100_003), (3, 300_000), (4, 33)])
def test_native_host_staged_ring_between_threads(world, n):
    """hc_allreduce_host_staged with queues between threads as the transport: every rank is a host
    thread with its own codec handle on the one GPU (no kernel waits for another one here: all
    waiting is done by the host threads)."""
    import queue
    import threading

    from tirocinio_triennale_b200.parallel import collectives

    eb = 1e-4
    bufs = [ALL["gradient" if r % 2 else "smooth"](n, seed=40 + r) for r in range(world)]
    want = ops.cpu_ring_allreduce(bufs, eb)
    xs = [_gpu(b) for b in bufs]
    outs = [torch.full_like(x, -7.0) for x in xs]
    codecs = [ops.Codec(ops.chunk_elems(n, world) + 64) for _ in range(world)]
    streams = [torch.cuda.Stream() for _ in range(world)]
    links = {(a, b): queue.Queue() for a in range(world) for b in range(world)}
    errors = []

    def rank_main(r):
        try:
            with torch.cuda.stream(streams[r]):
                collectives.host_staged_allreduce_native(
                    codecs[r], r, world, lambda dst, data: links[(r, dst)].put(data),
                    lambda src: links[(src, r)].get(timeout=20), xs[r], outs[r], eb)
        except Exception as e:  # noqa: BLE001
            errors.append((r, repr(e)))

    torch.cuda.synchronize()
    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors and not any(t.is_alive() for t in threads), errors
    torch.cuda.synchronize()
    for r in range(world):
        np.testing.assert_array_equal(outs[r].cpu().numpy(), want[r])


def test_stream_files_cross_between_device_and_host(tmp_path):
    """A tensor written from the GPU reads back on the CPU and the other way round: same bytes."""
    from tirocinio_triennale_b200.ops import stream_io

    eb = 1e-4
    t = torch.from_numpy(ALL["gradient"](70_000, seed=7)).reshape(7, 10_000)
    stream_io.save_tensor(tmp_path / "gpu.hcz", t.cuda(), eb)
    stream_io.save_tensor(tmp_path / "cpu.hcz", t, eb)
    assert (tmp_path / "gpu.hcz").read_bytes() == (tmp_path / "cpu.hcz").read_bytes()
    on_cpu = stream_io.load_tensor(tmp_path / "gpu.hcz")
    on_gpu = stream_io.load_tensor(tmp_path / "cpu.hcz", device="cuda")
    assert on_gpu.is_cuda and on_gpu.shape == t.shape
    assert torch.equal(on_gpu.cpu(), on_cpu)
    assert (on_cpu - t).abs().max().item() <= eb * 1.0001


@pytest.mark.parametrize("name", ["gradient", "sparse"])
def test_prepass_offsets_give_the_same_bytes(name):
    """Streams of 1024 tiles and more get their tile offsets from the pre-pass kernel: decode and all
    homomorphic adds must give the bytes of the look-back path and of the oracle, ragged tail included."""
    n, eb = 1024 * 4096 + 4096 * 3 + 77, 1e-4
    c = ops.Codec(max_elems=2 * n + 65536)  # two input streams, each rounded up to whole chunks
    x, y = ALL[name](n, seed=11), ALL[name](n, seed=12)
    sx, sy = ops.cpu_compress(x, eb), ops.cpu_compress(y, eb)
    gsx = _gpu(np.concatenate([sx, np.zeros(32, np.uint8)]))
    gsy = _gpu(np.concatenate([sy, np.zeros(32, np.uint8)]))
    ref_add = ops.cpu_hom_add(sx, y, eb)
    ref_dec = ops.cpu_decompress(sx, n, eb)
    for on in (True, False):
        c.set_prepass(on)
        d = torch.full((n,), 3.0, device="cuda")
        c.decompress(gsx, n, eb, out=d, stream_bytes=sx.size)
        np.testing.assert_array_equal(d.cpu().numpy(), ref_dec)
        out, size = c.hom_add(gsx, _gpu(y), eb, stream_bytes=sx.size)
        np.testing.assert_array_equal(_stream(out, size), ref_add)
        out, size = c.hom_add_streams(gsx, gsy, n, a_bytes=sx.size, b_bytes=sy.size)
        np.testing.assert_array_equal(_stream(out, size), ref_add)
        out, size = c.hom_add_multi([gsx, gsy], torch.zeros(n, device="cuda"), eb, stream_bytes=[sx.size, sy.size])
        np.testing.assert_array_equal(_stream(out, size), ref_add)
        assert c.status() == 0
    # a truncated stream is still reported, not read past its end
    c.set_prepass(True)
    c.decompress(gsx, n, eb, stream_bytes=sx.size - 5000)
    assert c.status() == 2
