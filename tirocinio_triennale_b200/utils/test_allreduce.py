"""Allreduce benchmark driver with the reference's command line
(HomComp/src/test_allreduce.cu:39-357): ``--iter N --file F --mode M --eb E [--nccl]``.

Every rank loads the same float32 file (or generates ``--data`` of ``--count`` values), runs the
chosen collective ``--iter`` times after ``--warmup`` untimed calls, and rank 0 prints min / max /
avg latency over ranks, then the same for the uncompressed NCCL allreduce (the reference compares
against ``MPI_Allreduce``; NCCL takes that place here).  Times are CUDA events on the device, not
host wall clock.  ``--out`` writes the result of rank 0 as text for the checker.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m tirocinio_triennale_b200.utils.test_allreduce --iter 10 --data normal --count 250000000 --eb 1e-4
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import datagen


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-i", "--iter", type=int, default=10)
    ap.add_argument("-f", "--file", default=None)
    ap.add_argument("-m", "--mode", default="normal", choices=["normal", "mixed", "opt", "seg", "raw"],
                    help="normal/opt/seg: compressed ring (one engine); mixed: hierarchical; raw: uncompressed P2P")
    ap.add_argument("--eb", type=float, default=1e-4)
    ap.add_argument("--nccl", "--MPI", dest="nccl", action="store_true", help="also time the library allreduce")
    ap.add_argument("--data", default="normal")
    ap.add_argument("--count", type=int, default=16 * 1024 * 1024)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    ap.add_argument("--algorithm", default="direct", choices=["direct", "ring", "onestep"])
    ap.add_argument("--trace", action="store_true",
                    help="afterwards: device time of every step of the collective (CUDA events between the launches, "
                         "which also serialises the steps), median over --iter calls, maximum over ranks")
    a = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from ..parallel import CompressedAllreduce, collectives

    if a.file:
        x = torch.from_numpy(np.fromfile(a.file, dtype=np.float32)).cuda()
    elif a.data in ("sinusoid", "gradient"):
        x = getattr(datagen, "sinusoid_field" if a.data == "sinusoid" else "gradient_like")(a.count, 0, "cuda")
    else:
        x = datagen.from_distribution(a.count, a.data, 0, "cuda")
    n = x.numel()
    out = torch.empty_like(x)
    ar = CompressedAllreduce(n, algorithm=a.algorithm)

    def call():
        if a.mode == "mixed":
            collectives.mixed_compressed_allreduce(ar, x, out, a.eb)
        elif a.mode == "raw":
            collectives.allreduce_ring_gpu(ar, x, out)
        else:
            ar.allreduce(x, out, a.eb)

    def bench(fn):
        for _ in range(a.warmup):
            fn()
        times = []
        for _ in range(a.iter):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e-3)
        mean = torch.tensor([sum(times) / len(times)], dtype=torch.float64, device="cuda")
        lo, hi, s = mean.clone(), mean.clone(), mean.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(s)
        return float(lo), float(hi), float(s) / world

    res = {"mode": a.mode, "count": n, "iterations": a.iter, "eb": a.eb, "world": world}
    lo, hi, avg = bench(call)
    res["collective_s"] = {"min": lo, "max": hi, "avg": avg}
    res["effective_GBps"] = 4 * n / hi / 1e9
    res["device_status"] = ar.status()
    if a.nccl:
        y = x.clone()
        lo, hi, avg = bench(lambda: dist.all_reduce(y))
        res["nccl_s"] = {"min": lo, "max": hi, "avg": avg}
    if a.trace and a.mode not in ("mixed", "raw"):
        ar.set_trace(True)
        steps = []
        for it in range(a.iter + a.warmup):
            dist.barrier()
            ar.allreduce(x, out, a.eb)
            ms = ar.last_step_ms()
            if it >= a.warmup:
                steps.append(ms)
        ar.set_trace(False)
        med = torch.tensor(np.median(np.array(steps), axis=0), dtype=torch.float64, device="cuda")
        dist.all_reduce(med, op=dist.ReduceOp.MAX)
        res["form"] = ar.stats()["form"]
        res["step_ms"] = [round(float(v), 4) for v in med]
    if rank == 0:
        print(json.dumps(res), flush=True)
        if a.out:
            np.savetxt(a.out, out.cpu().numpy(), fmt="%.9g")
    ar.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
