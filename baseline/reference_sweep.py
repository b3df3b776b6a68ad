"""The reference's allreduce (``allreduce_ring_comprs_hom_sum_F`` over the single-host MPI of
csrc/mpi_shim) at a few message sizes of the sweep, for the comparison column of the sweep tables.

    HCREF_SLOT_BYTES=700000000 python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        baseline/reference_sweep.py --mbs 1 16 256 1024 --eb 1e-3

Smooth sinusoid field (the sweep's data), CUDA events around each call, median over ``--iters``
calls, max over ranks.  One JSON line per size on rank 0.  ``--host-staged`` times the host-staged
variants of both libraries instead (``cpuCopy_allreduce_ring_comprs_hom_sum_F``).  The mailbox of the stand-in MPI must
hold one compressed chunk buffer (count / ranks * 4 bytes): set HCREF_SLOT_BYTES accordingly.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbs", type=int, nargs="+", default=[1, 16, 256, 1024])
    ap.add_argument("--eb", type=float, default=1e-3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--host-staged", action="store_true",
                    help="time the variants for GPUs that cannot address each other instead: the reference's "
                         "cpuCopy_allreduce_ring_comprs_hom_sum_F (chunks through host memory and MPI) and this "
                         "library's function of the same name (chunks through pinned host memory and gloo)")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist

    import bench as B
    import reference_arm
    from tirocinio_triennale_b200.utils import datagen

    lib = reference_arm._load()
    if lib is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference library could not be built here"}))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, world, local = B.init_dist(world)
    try:
        if world > 1 and lib.ref_init() != 0:
            raise SystemExit("MPI shim failed to initialise")
        max_n = max(a.mbs) * 1024 * 1024 // 4
        full = datagen.sinusoid_field(max_n, seed=rank, device="cuda")
        out = torch.empty_like(full)
        for mb in a.mbs:
            n = mb * 1024 * 1024 // 4
            x, y = full[:n].clone(), out[:n]
            ts = []
            for it in range(a.iters + 1):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if world > 1 and a.host_staged:
                    assert lib.ref_allreduce_cpucopy_F(x.data_ptr(), y.data_ptr(), n, a.eb) == 0
                elif world > 1:
                    assert lib.ref_allreduce_F(x.data_ptr(), y.data_ptr(), n, a.eb) == 0
                else:
                    sz = lib.ref_compress(x.data_ptr(), y.data_ptr(), n, a.eb)
                e1.record()
                e1.synchronize()
                if it:
                    ts.append(e0.elapsed_time(e1))
            ms = B.max_over_ranks(sorted(ts)[len(ts) // 2])
            row = {"impl": "reference", "bytes": mb * 1024 * 1024, "eb": a.eb, "world": world, "ms": ms,
                   "effective_GBps": mb * 1024 * 1024 / ms / 1e6}
            if world > 1 and a.host_staged:
                from tirocinio_triennale_b200.parallel import collectives

                row["call"] = "cpuCopy_allreduce_ring_comprs_hom_sum_F"
                z = torch.empty_like(y)
                ts = []
                for it in range(a.iters + 1):
                    dist.barrier()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    collectives.cpuCopy_allreduce_ring_comprs_hom_sum_F(x, z, a.eb)
                    e1.record()
                    e1.synchronize()
                    if it:
                        ts.append(e0.elapsed_time(e1))
                row["ours_ms"] = B.max_over_ranks(sorted(ts)[len(ts) // 2])
                row["max_abs_diff_ours_vs_reference"] = float((z - y).abs().max())
            if rank == 0:
                print(json.dumps(row), flush=True)
        if world > 1:
            lib.ref_finalize()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
