"""Failure detection on the device without faulting it: every wait is bounded, a wait that runs
out ends in a status word that the host reads, and the context stays usable."""
import time

import numpy as np
import pytest
import torch

from tirocinio_triennale_b200 import ops

pytestmark = pytest.mark.gpu


def test_flag_that_never_rises_times_out_with_status():
    n, eb = 100_000, 1e-4
    x = np.random.default_rng(0).normal(0, 0.01, n).astype(np.float32)
    s = ops.cpu_compress(x, eb)
    gs = torch.from_numpy(np.concatenate([s, np.zeros(64, np.uint8)])).cuda()
    codec = ops.Codec(n, timeout_ms=300)
    tiles = (ops.rate_bytes(n) * 32) // codec.tile_elems
    # what a producer would publish: tag << 40 | byte offset of the tile's payload
    rate = s[: ops.rate_bytes(n)].astype(np.int64)
    F, outl = rate & 31, rate >> 7
    plen = np.where(outl == 1, 4 + 4 * F + ((rate >> 5) & 3) + 1, np.where(F > 0, 4 + 4 * F, 0))
    per_tile = plen.reshape(tiles, -1).sum(axis=1)
    offs = ops.rate_bytes(n) + np.concatenate([[0], np.cumsum(per_tile)[:-1]])

    def flags_for(tag, upto):
        f = np.zeros(tiles, dtype=np.int64)
        f[:upto] = (tag << 40) | offs[:upto]
        return torch.from_numpy(f).cuda()

    # the producer "arrived" for the first tiles only; nothing ever sets the rest
    t0 = time.time()
    y = codec.decompress_flagged(gs, n, eb, flags_for(7, 3), want=7, stream_bytes=s.size)
    status = codec.status()
    assert status == 6  # peer never delivered
    assert time.time() - t0 < 20  # bounded, not a hang
    want = ops.cpu_decompress(s, n, eb)
    done = 3 * codec.tile_elems
    np.testing.assert_array_equal(y[:done].cpu().numpy(), want[:done])  # delivered tiles were decoded
    # all flags up: the same handle works again
    y = codec.decompress_flagged(gs, n, eb, flags_for(9, tiles), want=9, stream_bytes=s.size)
    assert codec.status() == 0
    np.testing.assert_array_equal(y.cpu().numpy(), want)


def test_corrupted_rate_bytes_are_contained():
    n, eb = 50_000, 1e-4
    x = np.random.default_rng(1).normal(0, 0.01, n).astype(np.float32)
    s = ops.cpu_compress(x, eb).copy()
    s[10:200] = 0xFF  # claims 31 planes + 4 outlier bytes per block: far more payload than exists
    codec = ops.Codec(n)
    y = codec.decompress(torch.from_numpy(s).cuda(), n, eb)
    assert codec.status() == 2  # truncated: rate bytes imply more bytes than the stream has
    assert y.numel() == n
    out, size = codec.compress(torch.from_numpy(x).cuda(), eb)  # still usable
    assert codec.status() == 0


def _missing_peer(rank, world):
    """A rank that is alive but sits one call out.  Host-made failure: no kernel faults or hangs; the
    other rank's bounded waits run out, it reads status 6, the ranks realign their call numbers over
    the host channel and the next call is an ordinary one.  Peer stores over CUDA IPC only (no
    multicast), short time-out, nobody leaves before close()."""
    import numpy as np
    import torch.distributed as dist

    from datasets import gradient_like
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import CompressedAllreduce

    n, eb = 600_000, 1e-4
    ar = CompressedAllreduce(n, timeout_ms=300, transport="ipc")
    bufs = [gradient_like(n, seed=40 + r) for r in range(world)]
    want = ops.cpu_ring_allreduce(bufs, eb)[rank]
    x = torch.from_numpy(bufs[rank]).cuda()
    out = torch.empty_like(x)
    for algorithm in ("direct", "onestep", "ring"):
        ar.set_algorithm(algorithm)
        ar.set_small_count(0)  # "direct" means the three-step form here, whatever the size
        ar.allreduce(x, out, eb)
        assert ar.status() == 0
        np.testing.assert_array_equal(out.cpu().numpy(), want)
        dist.barrier()
        # the broken call: rank 1 skips it on the host
        if rank != 1:
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            ar.allreduce(x, out, eb)
            t1.record()
            torch.cuda.synchronize()
            assert ar.status(clear=False) == 6  # a peer never arrived
            assert t0.elapsed_time(t1) < 5000.0  # the waits gave up, one time-out deep per step at most
        dist.barrier()
        cleared = ar.resync()
        assert cleared == (6 if rank != 1 else 0)
        for _ in range(2):  # both all-gather buffer sets
            out.fill_(-1.0)
            ar.allreduce(x, out, eb)
            assert ar.status() == 0
            np.testing.assert_array_equal(out.cpu().numpy(), want)
    dist.barrier()
    ar.close()


@pytest.mark.multigpu
def test_peer_that_skips_a_call_then_resync():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mp_util import run_ranks

    run_ranks(_missing_peer, 2)
