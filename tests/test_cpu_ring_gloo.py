"""Host-rank compressed ring over gloo: real processes, the configuration of the CPU reference
path (2 ranks, 1 Mi floats of 3 sinusoids + noise, eb 1e-4), plus host-side fault injection."""
import numpy as np
import pytest

from mp_util import run_ranks


def _field(n, seed):
    rng = np.random.default_rng(seed)
    t = np.arange(n, dtype=np.float64) / n
    x = sum(np.sin(2 * np.pi * rng.uniform(1, 50) * t + rng.uniform(0, 6.28)) for _ in range(3))
    return (x + rng.normal(0, 1e-3, n)).astype(np.float32)


def _worker(rank, world, n, eb):
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import cpu_compressed_allreduce

    bufs = [_field(n, seed=r) for r in range(world)]
    log = []
    out = cpu_compressed_allreduce(bufs[rank], eb, hop_log=log)
    want = ops.cpu_ring_allreduce(bufs, eb)[rank]
    np.testing.assert_array_equal(out, want)  # same bytes as the in-process oracle
    exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
    assert np.abs(out - exact).max() <= world * eb * 1.01
    # byte-exact stream round trip of this rank's own chunk
    B = ops.chunk_elems(n, world)
    mine = bufs[rank][rank * B: (rank + 1) * B]
    s = ops.cpu_compress(mine, eb)
    assert ops.cpu_stream_size(s, mine.size) == s.size == log[0]
    np.testing.assert_array_equal(ops.cpu_compress(ops.cpu_decompress(s, mine.size, eb), eb), s)


@pytest.mark.parametrize("world,n", [(2, 1 << 20), (3, 100_003), (4, 70_000)])
def test_gloo_ring_matches_oracle(world, n):
    run_ranks(_worker, world, args=(n, 1e-4))


def _faulty(rank, world):
    import torch.distributed as dist

    from tirocinio_triennale_b200.parallel import PeerTimeout, cpu_compressed_allreduce

    x = _field(40_000, rank)
    if rank == 1:
        # rank 1 never sends its first hop; its successor must time out, not hang
        try:
            cpu_compressed_allreduce(x, 1e-4, drop_hop=(1, 0))
        except PeerTimeout:
            pass
        return
    with pytest.raises(PeerTimeout):
        cpu_compressed_allreduce(x, 1e-4)


def test_dropped_message_times_out_instead_of_hanging():
    # a short group timeout makes the missed message surface within seconds
    run_ranks(_faulty_entry, 2, args=(), timeout=120)


def _faulty_entry(rank, world):
    import datetime

    import torch.distributed as dist

    # re-create the group with a short timeout (run_ranks made one with the default)
    dist.destroy_process_group()
    import os

    dist.init_process_group("gloo", rank=rank, world_size=world,
                            init_method="tcp://127.0.0.1:%d" % (int(os.environ["MASTER_PORT"]) + 1),
                            timeout=datetime.timedelta(seconds=5))
    _faulty(rank, world)


def test_hierarchy_oracle_composition():
    """Host restatement of the hierarchical allreduce: one group is the plain fp32 sum in rank order; with
    two groups every value is within (groups * eb) of the exact sum and every slice is what the compressed
    ring gives for the group sums."""
    import numpy as np

    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import collectives

    rng = np.random.default_rng(3)
    n, eb = 10_007, 1e-4
    bufs = [rng.normal(0, 0.01, n).astype(np.float32) for _ in range(4)]
    one = collectives.hierarchy_oracle(bufs, 4, eb)
    acc = np.zeros(n, np.float32)
    for b in bufs:
        acc = acc + b
    np.testing.assert_array_equal(one, acc)
    two = collectives.hierarchy_oracle(bufs, 2, eb)
    exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
    assert np.abs(two - exact).max() <= 2 * eb * 1.01 + 1e-6
    B = ops.chunk_elems(n, 2)
    s0, s1 = bufs[0] + bufs[1], bufs[2] + bufs[3]
    np.testing.assert_array_equal(two[:B], ops.cpu_ring_allreduce([s0[:B], s1[:B]], eb)[0])
