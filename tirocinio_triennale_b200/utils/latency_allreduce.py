"""Small-message latency of the compressed allreduce: back-to-back calls (no host synchronisation
between them, four rotating buffer pairs), the direct form, the one-step form and NCCL's fp32
``all_reduce`` side by side, and a check that the two forms return the same bits.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m tirocinio_triennale_b200.utils.latency_allreduce --counts 1024 65536 1048576 --eb 1e-4

Times are CUDA events around ``--calls`` calls, best of ``--repeats`` loops, maximum over ranks,
microseconds per call.  Messages of these sizes stay in L2 in any real use, so nothing is flushed
here; the message-size sweep (``sweep_allreduce``) times isolated calls behind an L2 flush.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import datagen


def _loop_us(fn, calls: int, repeats: int) -> float:
    best = None
    for _ in range(repeats):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(calls):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t) * 1e3 / calls
        best = us if best is None else min(best, us)
    return best


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--counts", type=int, nargs="+", default=[1024, 65536, 262144, 1 << 20, 1 << 21, 1 << 22])
    ap.add_argument("--eb", type=float, default=1e-4)
    ap.add_argument("--calls", type=int, default=30)
    ap.add_argument("--repeats", type=int, default=3)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29538")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from ..parallel import CompressedAllreduce

    for n in a.counts:
        ar = CompressedAllreduce(n * world)  # every size fits one stream slot, so both forms can run
        xs = [datagen.gradient_like(n, 1000 * b + rank, "cuda") for b in range(4)]
        outs = [torch.empty_like(xs[0]) for _ in range(4)]
        row = {"values": n, "bytes": 4 * n, "world": world, "eb": a.eb}
        first = None
        for form in ("direct", "onestep"):
            ar.set_algorithm(form)
            ar.set_small_count(0)
            for i in range(6):
                ar.allreduce(xs[i % 4], outs[i % 4], a.eb)
            row[form + "_us"] = _loop_us(lambda i: ar.allreduce(xs[i % 4], outs[i % 4], a.eb), a.calls, a.repeats)
            ar.allreduce(xs[0], outs[0], a.eb)
            torch.cuda.synchronize()
            if first is None:
                first = outs[0].clone()
            else:
                row["same_bits"] = bool(torch.equal(first, outs[0]))
        row["status"] = ar.status()
        ys = [x.clone() for x in xs]
        for i in range(6):
            dist.all_reduce(ys[i % 4])
        row["nccl_us"] = _loop_us(lambda i: dist.all_reduce(ys[i % 4]), a.calls, a.repeats)
        ar.close()
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
