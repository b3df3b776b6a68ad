"""Reference arm of bench.py.

Runs the reference library (built by baseline/build_ref.py from the reference sources with the
three fixes it needs to compile and to run without faulting on B200, listed there) through its own
public API on the configuration bench.py measures: 64 MiB of float32 per rank,
gradient-like values, error bound 1e-4.

* N >= 2: ``allreduce_ring_comprs_hom_sum_F`` (the variant the reference benchmarks, its stock code
  path: per-call cudaMalloc/cudaFree, blocking size read-backs, MPI point-to-point per hop).  MPI is
  the single-host shim in baseline/mpi_shim, which moves device buffers GPU to GPU through
  IPC-mapped mailboxes, as a CUDA-aware MPI does inside one node.
* N == 1: the reference's allreduce returns without doing anything for one rank, so the arm times
  what one rank's share of the pipeline is made of: ``GSZ_compress_deviceptr_outlier`` followed by
  ``GSZ_decompress_deviceptr_outlier`` on the 64 MiB buffer (the same work our N = 1 line does).

None of this package's kernels, models or engine is on this path.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
COUNT = 16 * 1024 * 1024
EB = 1e-4
NBUF = 4


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _load():
    sys.path.insert(0, HERE)
    import build_ref

    lib_path = build_ref.build()
    if lib_path is None or not os.path.exists(lib_path):
        return None
    lib = C.CDLL(str(lib_path))
    vp, sz, f = C.c_void_p, C.c_size_t, C.c_float
    lib.ref_init.restype = C.c_int
    lib.ref_finalize.restype = C.c_int
    lib.ref_barrier.restype = C.c_int
    lib.ref_allreduce_F.restype = C.c_int
    lib.ref_allreduce_F.argtypes = [vp, vp, sz, f]
    if hasattr(lib, "ref_allreduce_cpucopy_F"):
        lib.ref_allreduce_cpucopy_F.restype = C.c_int
        lib.ref_allreduce_cpucopy_F.argtypes = [vp, vp, sz, f]
    lib.ref_compress.restype = sz
    lib.ref_compress.argtypes = [vp, vp, sz, f]
    lib.ref_decompress.restype = None
    lib.ref_decompress.argtypes = [vp, vp, sz, sz, f]
    lib.ref_hom_sum_F.restype = sz
    lib.ref_hom_sum_F.argtypes = [vp, vp, vp, sz, f, sz]
    return lib


def main(args):
    try:
        lib = _load()
    except Exception as e:  # build or load problem: say so in one line
        return _unavailable("reference build failed: %s" % str(e).splitlines()[0][:160])
    if lib is None:
        return _unavailable("reference library could not be built here (no nvcc or no reference sources)")

    import torch
    import torch.distributed as dist

    root = os.path.dirname(HERE)
    sys.path.insert(0, root)
    import bench as B
    from tirocinio_triennale_b200.utils import datagen, timing

    rank, world, local = B.init_dist(args.gpus)
    try:
        if world > 1 and lib.ref_init() != 0:
            return _unavailable("MPI shim failed to initialise")
        xs = [datagen.gradient_like(COUNT, seed=1000 * b + rank, device="cuda") for b in range(NBUF)]
        outs = [torch.empty_like(xs[0]) for _ in range(NBUF)]
        cmp_buf = torch.empty(COUNT * 4 + 65536, dtype=torch.uint8, device="cuda")
        flush = timing.L2Flusher()
        sizes = []

        def step(i):
            b = i % NBUF
            if world == 1:
                sz = lib.ref_compress(xs[b].data_ptr(), cmp_buf.data_ptr(), COUNT, EB)
                outs[b].zero_()  # the reference decoder leaves zero blocks untouched
                lib.ref_decompress(outs[b].data_ptr(), cmp_buf.data_ptr(), COUNT, sz, EB)
                sizes.append(sz)
            else:
                rc = lib.ref_allreduce_F(xs[b].data_ptr(), outs[b].data_ptr(), COUNT, EB)
                assert rc == 0

        warm = max(args.warmup, 3)
        for i in range(warm):
            step(i)
        flush()
        with timing.ClockSampler(local) as clk:
            ms = B.timed_loop(step, args.steps)
        clocks = clk.summary()

        exact = xs[0].double()
        dist.all_reduce(exact)
        step(0)
        torch.cuda.synchronize()
        max_err = float((outs[0].double() - exact).abs().max().item())

        host_in = [torch.empty(COUNT, dtype=torch.float32).pin_memory() for _ in range(NBUF)]
        for b in range(NBUF):
            host_in[b].copy_(xs[b])
        host_out = [torch.empty(COUNT, dtype=torch.float32).pin_memory() for _ in range(NBUF)]

        def e2e_step(i):  # the reference has no host-buffer collective: copy up, its call, copy down
            b = i % NBUF
            xs[b].copy_(host_in[b], non_blocking=True)
            step(i)
            host_out[b].copy_(outs[b], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(host_out[b][0])

        for i in range(3):
            e2e_step(i)
        e2e_ms = B.timed_loop(e2e_step, args.steps)

        total_bytes = 4.0 * COUNT * world
        per_step = ms / args.steps
        value = total_bytes / (per_step * 1e-3) / 1e9
        out = {
            "impl": "reference",
            "metric": "compressed_allreduce_effective_GBps_aggregate", "value": value,
            "unit": "GB/s (N ranks x 64 MiB uncompressed input per call / device time, max over ranks)",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / world / B.PUBLISHED_PER_RANK_GBS,
            "dtype": "fp32 data, int32 quantised domain", "data": "synthetic",
            "config": B.bench_config(world),
            "implementation": {
                "algorithm_timed": "reference allreduce_ring_comprs_hom_sum_F (host-driven ring over MPI point to point)"
                                   if world > 1 else
                                   "reference GSZ_compress_deviceptr_outlier + GSZ_decompress_deviceptr_outlier "
                                   "(its allreduce is a no-op for one rank)",
                "transport": "single-host MPI shim: IPC-mapped device mailboxes (GPU to GPU copies)",
                "build": "nvcc -arch sm_100 -O3 of the reference sources; not byte-for-byte unmodified: stand-in "
                         "comprs_test.cuh, declaration fix in intra_node_allgather, and the __shared__ excl_sum "
                         "that the first chunk reads uninitialised is set to 0 (as shipped the kernels store out "
                         "of bounds on B200)",
                "e2e_call": "torch copy of the input to the device, the reference's call, torch copy of the result back",
            },
            "per_rank_gbs": value / world, "max_abs_err": max_err, "err_bound_world_x_eb": world * EB,
            "e2e": {"value": total_bytes / (e2e_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s aggregate",
                    "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": 4 * COUNT, "d2h_bytes_per_step": 4 * COUNT},
            "gpu_launches": args.steps * (2 if world == 1 else 2 * world),
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
        }
        if world == 1 and sizes:
            out["compression_ratio_reported"] = 4.0 * COUNT / sizes[-1]
        if world > 1:
            lib.ref_finalize()
        if rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        dist.destroy_process_group()
