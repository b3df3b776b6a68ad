"""Runs a function on N ranks as child processes (one GPU each when the ranks use CUDA)."""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, backend, fn, args, errq):
    try:
        import torch.distributed as dist

        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        if backend != "gloo" or torch.cuda.is_available() and args and args[0] == "cuda":
            pass
        if torch.cuda.is_available() and torch.cuda.device_count() >= world:
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world, init_method="tcp://127.0.0.1:%d" % port)
        try:
            fn(rank, world, *args)
        finally:
            dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world, args=(), backend="gloo", timeout=240):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errors.append((-1, "rank process timed out"))
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    assert not errors and not bad, "rank failures: %s %s" % (errors, bad)
