"""Message-size sweep of the compressed allreduce: 4 KB - 1 GB (powers of two) on the smooth
sinusoid field, error bounds 1e-3 and 1e-5; effective GB/s (message bytes / device time, max over
ranks), compression ratio, NCCL uncompressed time, and the fraction of the roofline
max(HBM bytes / measured copy bandwidth, NVLink bytes / 770 GB/s); `form` says which form of the
allreduce a size took (small messages take the one-step form unless `--small-count 0`).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m tirocinio_triennale_b200.utils.sweep_allreduce --max-mb 1024 --out sweep8.jsonl
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import datagen, timing

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction between two B200s on one NVSwitch (GB/s)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-kb", type=int, default=4)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--ebs", type=float, nargs="+", default=[1e-3, 1e-5])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--algorithm", default="direct", choices=["direct", "ring", "onestep"])
    ap.add_argument("--small-count", type=int, default=None,
                    help="direct: values up to which a message takes the one-step form (0: never; default: the library's)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29537")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from ..parallel import CompressedAllreduce

    peaks = timing.measured_peaks()
    max_n = a.max_mb * 1024 * 1024 // 4
    ar = CompressedAllreduce(max_n, algorithm=a.algorithm)
    if a.small_count is not None:
        ar.set_small_count(a.small_count)
    full = datagen.sinusoid_field(max_n, seed=rank, device="cuda")
    out = torch.empty_like(full)
    flush = timing.L2Flusher()
    rows = []
    nbytes = a.min_kb * 1024
    while nbytes <= a.max_mb * 1024 * 1024:
        n = nbytes // 4
        x, y = full[:n], out[:n]
        ncc = x.clone()

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(a.iters):
                flush()
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                e1.synchronize()
                ts.append(e0.elapsed_time(e1))
            t = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        nccl_ms = timed(lambda: dist.all_reduce(ncc))
        for eb in a.ebs:
            ms = timed(lambda: ar.allreduce(x, y, eb))
            st = ar.stats()
            cr = st["compression_ratio"] or 1.0
            exact = x.double()
            dist.all_reduce(exact)
            err = float((y.double() - exact).abs().max())
            # bytes this rank's kernels must move: read input, write result, streams in and out
            comp = 4 * n / cr
            if st["form"] == "onestep":  # the whole stream to every rank, every rank's stream read once
                hbm = 4 * n + 4 * n + comp * (1 + world)
                link = comp * (world - 1)
            else:
                hbm = 4 * n + 4 * n + 4 * comp * (world - 1) / max(world, 1) + 2 * comp
                link = 2 * comp * (world - 1) / max(world, 1)
            roof_ms = max(hbm / (peaks["hbm_gbs"] * 1e9), link / (NVLINK_GBS * 1e9)) * 1e3
            rows.append({"bytes": nbytes, "eb": eb, "world": world, "ms": ms, "effective_GBps": nbytes / ms / 1e6,
                         "nccl_ms": nccl_ms, "speedup_vs_nccl": nccl_ms / ms, "compression_ratio": cr, "form": st["form"],
                         "max_abs_err": err, "err_bound": world * eb, "roofline_ms": roof_ms,
                         "roofline_fraction_of_%s" % peaks["source"]: roof_ms / ms, "status": ar.status()})
            if rank == 0:
                print(json.dumps(rows[-1]), flush=True)
        nbytes *= 2
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    ar.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
