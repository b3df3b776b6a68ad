"""Compressed ring allreduce on 2+ GPUs against the host-rank oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, counts, eb, algorithm="direct"):
    import torch.distributed as dist

    from datasets import gradient_like, smooth
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import CompressedAllreduce

    ar = CompressedAllreduce(max(counts), timeout_ms=5000, algorithm=algorithm)
    ar.set_small_count(0)  # the direct form at every size here; the one-step form has a test of its own
    for it, n in enumerate(counts):
        gen = smooth if it % 2 == 0 else gradient_like
        bufs = [gen(n, seed=100 * it + r) for r in range(world)]
        x = torch.from_numpy(bufs[rank]).cuda()
        out = torch.full_like(x, -3.0)
        ar.allreduce(x, out, eb)
        got = out.cpu().numpy()
        want = ops.cpu_ring_allreduce(bufs, eb)[rank]
        assert ar.status() == 0, "device status"
        np.testing.assert_array_equal(got, want)
        exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
        assert np.abs(got - exact).max() <= world * eb * 1.01 + 1e-6
        # in place, and again (flags and slots are reused without any reset); with the steps of the
        # direct algorithm strictly one after the other this time
        y = x.clone()
        ar.set_overlap(False)
        ar.allreduce(y, None, eb)
        ar.set_overlap(True)
        np.testing.assert_array_equal(y.cpu().numpy(), want)
        if algorithm == "direct" and it >= 3:
            # packed transport buffers instead of tiles at fixed offsets, and the steps sharing the GPU
            ar.set_sparse_tiles(False)
            ar.set_shares(2, 1, 0)
            z = torch.full_like(x, 5.0)
            ar.allreduce(x, z, eb)
            ar.set_sparse_tiles(True)
            ar.set_shares(0, 0, 0)
            assert ar.status() == 0
            np.testing.assert_array_equal(z.cpu().numpy(), want)
            # host buffers in, host buffers out: same values, whatever the number of pieces
            hx = x.cpu().pin_memory()
            for pieces in (0, 1, 3):
                hy = torch.empty_like(hx).pin_memory()
                ar.allreduce_host(hx, hy, eb, pieces=pieces)
                torch.cuda.current_stream().synchronize()
                assert ar.status() == 0
                np.testing.assert_array_equal(hy.numpy(), want)
    ar.allreduce(x, out, eb)  # so that the statistics below are those of a device-buffer call
    sizes = ar.last_stream_bytes()
    assert all(s > 0 for s in sizes)
    st = ar.stats()
    assert st["status"] == 0 and st["count"] == counts[-1] and st["stream_bytes"] == sizes
    assert st["compression_ratio"] > 1.0 and st["algorithm"] == algorithm
    dist.barrier()
    ar.close()


@pytest.mark.parametrize("algorithm", ["direct", "ring"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_matches_host_oracle(world, algorithm):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    # 1048589: at 2 ranks the chunks are 524320 and 524269 values, one 32768-value chunk apart in their
    # rate bytes, so the shorter stream has tile tickets past its own end in the shared decode launch
    counts = [1, 33, 4097, 100000, 1 << 20, 1048589, (1 << 22) + 12345]
    run_ranks(_worker, world, args=(counts, 1e-4, algorithm))


def _onestep_worker(rank, world, counts, eb):
    import torch.distributed as dist

    from datasets import gradient_like, smooth
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import CompressedAllreduce

    max_count = world * (1 << 20)
    ar = CompressedAllreduce(max_count, timeout_ms=5000, algorithm="onestep")
    bad = []
    for it, n in enumerate(counts):
        gen = smooth if it % 2 == 0 else gradient_like
        bufs = [gen(n, seed=300 * it + r) for r in range(world)]
        want = ops.cpu_ring_allreduce(bufs, eb)[rank]
        x = torch.from_numpy(bufs[rank]).cuda()
        out = torch.full_like(x, -3.0)
        ar.allreduce(x, out, eb)
        if ar.status() != 0 or not np.array_equal(out.cpu().numpy(), want):
            bad.append(("onestep", n))
        # twice more in place: both sets of slots and flags are reused without a reset
        y = x.clone()
        ar.allreduce(y, None, eb)
        z = x.clone()
        ar.allreduce(z, None, eb)
        if not (np.array_equal(y.cpu().numpy(), want) and np.array_equal(z.cpu().numpy(), want)):
            bad.append(("onestep in place", n))
    sizes = ar.last_stream_bytes()
    if not (sizes[0] > 0 and all(s == 0 for s in sizes[1:])):
        bad.append(("sizes", sizes))
    # the direct form with a small-message limit: calls of both kinds share slots, flags and counters
    ar.set_algorithm("direct")
    ar.set_small_count(100_000)
    for it, n in enumerate([4097, 200_000, 33, 150_000, 100_000]):
        bufs = [gradient_like(n, seed=500 + 10 * it + r) for r in range(world)]
        want = ops.cpu_ring_allreduce(bufs, eb)[rank]
        x = torch.from_numpy(bufs[rank]).cuda()
        ar.allreduce(x, None, eb)
        if ar.status() != 0 or not np.array_equal(x.cpu().numpy(), want):
            bad.append(("mixed", n))
    # a message too large for one slot falls back to the direct form
    ar.set_algorithm("onestep")
    n = (1 << 20) + 4096 * world
    bufs = [smooth(n, seed=700 + r) for r in range(world)]
    x = torch.from_numpy(bufs[rank]).cuda()
    ar.allreduce(x, None, eb)
    if ar.status() != 0 or not np.array_equal(x.cpu().numpy(), ops.cpu_ring_allreduce(bufs, eb)[rank]):
        bad.append(("fallback", n))
    dist.barrier()
    ar.close()
    assert not bad, bad


@pytest.mark.parametrize("world", [2, 4, 8])
def test_one_step_allreduce_matches_host_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    run_ranks(_onestep_worker, world, args=([1, 33, 4097, 100000, 1 << 20], 1e-4))


def _raw_worker(rank, world):
    import torch.distributed as dist

    from datasets import gradient_like
    from tirocinio_triennale_b200.parallel import CompressedAllreduce, collectives

    n = 300_003
    ar = CompressedAllreduce(n, timeout_ms=5000)
    bufs = [gradient_like(n, seed=r) for r in range(world)]
    x = torch.from_numpy(bufs[rank]).cuda()
    for it in range(3):
        out = torch.zeros_like(x)
        collectives.allreduce_ring_gpu(ar, x, out)
        want = torch.zeros(n)
        for b in bufs:  # rank order, fp32: the kernel's summation order
            want += torch.from_numpy(b)
        assert ar.status() == 0
        torch.testing.assert_close(out.cpu(), want, rtol=0, atol=0)
    out2 = torch.zeros_like(x)
    collectives.mixed_compressed_allreduce(ar, x, out2, 1e-4)  # one group: nothing is compressed
    torch.testing.assert_close(out2.cpu(), want, rtol=0, atol=0)
    # host-staged variant: same numbers as the device ring
    out3 = torch.zeros_like(x)
    collectives.cpuCopy_allreduce_ring_comprs_hom_sum_F(x, out3, 1e-4)
    out4 = torch.zeros_like(x)
    collectives.allreduce_ring_comprs_hom_sum_F_opt(ar, x, out4, 1e-4)
    torch.testing.assert_close(out3, out4, rtol=0, atol=0)
    dist.barrier()
    ar.close()


def test_uncompressed_and_named_variants():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_raw_worker, 2)


def _nvls_worker(rank, world, counts, eb, note_path, transport="nvls"):
    """Same check over the multicast transport.  Mismatches are collected and raised only after
    every rank has left the collective and unmapped its region together."""
    import torch.distributed as dist

    from datasets import gradient_like, smooth
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.parallel import CompressedAllreduce

    ar = CompressedAllreduce(max(counts), timeout_ms=5000, transport=transport)
    problems = []
    for algorithm in ("direct", "ring"):
        ar.set_algorithm(algorithm)
        for it, n in enumerate(counts):
            gen = smooth if it % 2 == 0 else gradient_like
            bufs = [gen(n, seed=100 * it + r) for r in range(world)]
            x = torch.from_numpy(bufs[rank]).cuda()
            for rep in range(2):  # both all-gather buffer sets
                out = torch.full_like(x, -3.0)
                ar.allreduce(x, out, eb)
                status = ar.status()
                want = ops.cpu_ring_allreduce(bufs, eb)[rank]
                if status != 0 or not np.array_equal(out.cpu().numpy(), want):
                    problems.append((algorithm, n, rep, status))
    # uncompressed sum: formed inside the switch when there is a multicast mapping (its own order of
    # additions, the same bits on every rank), by peer loads in rank order otherwise
    n = 300_003
    bufs = [gradient_like(n, seed=r) for r in range(world)]
    x = torch.from_numpy(bufs[rank]).cuda()
    for rep in range(3):
        out = torch.zeros_like(x)
        ar.allreduce_raw(x, out)
        status = ar.status()
        exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
        err = np.abs(out.cpu().numpy().astype(np.float64) - exact).max()
        everyone = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(everyone, out)
        if status != 0 or err > 1e-5 or not all(torch.equal(e, out) for e in everyone):
            problems.append(("raw", rep, status, float(err)))
    multicast = ar.multicast
    dist.barrier()
    ar.close()
    if rank == 0:
        with open(note_path, "w") as f:
            f.write("1" if multicast else "0")
    assert not problems, problems


@pytest.mark.parametrize("transport", ["nvls", "mc"])
def test_allreduce_over_multicast_transport(tmp_path, transport):
    """``nvls``: region and multicast mapping from torch's symmetric memory; ``mc``: from the library's
    own bootstrap (driver virtual-memory API, file descriptors over a unix socket)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    note = tmp_path / "multicast"
    run_ranks(_nvls_worker, world, args=([1, 4097, 100000, (1 << 22) + 12345], 1e-4, str(note), transport),
              backend="nccl")
    if note.read_text() != "1":
        pytest.skip("the fabric offers no multicast mapping: ran over peer stores on symmetric memory")


def _hier_worker(rank, world, group_size, counts, eb):
    """mixed_compressed_allreduce with the ranks split into groups: raw inside a group, compressed
    between the groups; compared with the host oracle composed the same way, bit for bit on every rank."""
    import torch.distributed as dist

    from datasets import gradient_like, smooth
    from tirocinio_triennale_b200.parallel import collectives

    local, inter = collectives.make_hierarchy(max(counts), group_size, timeout_ms=5000)
    for it, n in enumerate(counts):
        gen = smooth if it % 2 == 0 else gradient_like
        bufs = [gen(n, seed=300 * it + r) for r in range(world)]
        want = collectives.hierarchy_oracle(bufs, group_size, eb)
        x = torch.from_numpy(bufs[rank]).cuda()
        for rep in range(2):  # twice: flags, slots and the result area are reused without any reset
            out = torch.full_like(x, -3.0)
            collectives.mixed_compressed_allreduce(local, x, out, eb, inter_comm=inter)
            assert local.status() == 0 and (inter is None or inter.status() == 0)
            np.testing.assert_array_equal(out.cpu().numpy(), want)
        exact = np.sum(np.stack(bufs).astype(np.float64), axis=0)
        n_groups = world // group_size
        assert np.abs(want - exact).max() <= n_groups * eb * 1.01 + 1e-5
        # the flat uncompressed call of the same handle still works in between (shared call counter)
        out2 = torch.zeros_like(x)
        local.allreduce_raw(x, out2)
        assert local.status() == 0
    dist.barrier()
    if inter is not None:
        inter.close()
    local.close()


@pytest.mark.parametrize("world,group_size", [(2, 1), (2, 2), (4, 2), (8, 4), (8, 2)])
def test_hierarchical_allreduce_matches_composed_oracle(world, group_size):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    run_ranks(_hier_worker, world, args=(group_size, [33, 100_003, (1 << 21) + 77], 1e-4))
