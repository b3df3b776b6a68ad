"""Data-parallel training of a GPT-2-shaped model with compressed gradient allreduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m tirocinio_triennale_b200.models.train_dp --steps 200 --batch 8 --eb 1e-5

Runs the same seeded training twice: fp32 gradient buckets of 25 MB averaged (a) with this
library's compressed allreduce through the DDP communication hook, overlapped with backward on a
side stream, and (b) with plain NCCL.  Prints one JSON line with tokens/s of both runs and the loss
gap after the last step.  Random-init weights, uniform random token ids (no dataset, no download).

``--save PATH`` writes model, optimiser, step count and the data generator's state after the last
step (rank 0; one file per arm: PATH.compressed / PATH.nccl); ``--resume PATH`` continues from such
files, bit for bit the run that was never interrupted.  ``--save-compressed-eb EB`` additionally
writes the model weights as error-bounded streams (PATH.*.hcz, ``ops.stream_io.save_state``).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from ..parallel import CompressedHookState, compressed_allreduce_hook
from .gpt2 import GPT2, GPT2Config


def run(args, compressed: bool, rank: int, world: int, device):
    torch.manual_seed(1234)
    cfg = GPT2Config.small() if args.model == "small" else GPT2Config.tiny()
    cfg.seq_len = args.seq
    model = GPT2(cfg).to(device)
    ddp = DDP(model, device_ids=[device.index] if device.type == "cuda" else None, bucket_cap_mb=args.bucket_mb,
              gradient_as_bucket_view=True)
    state = None
    if compressed:
        state = CompressedHookState(eb=args.eb, max_bucket_elems=int(args.bucket_mb * 1.5 * 1024 * 1024 / 4) + (1 << 20))
        ddp.register_comm_hook(state, compressed_allreduce_hook)
    opt = torch.optim.AdamW(ddp.parameters(), lr=args.lr, weight_decay=0.0, fused=device.type == "cuda")
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    arm = "compressed" if compressed else "nccl"
    start = 0
    if getattr(args, "resume", None):
        ck = torch.load("%s.%s.rank%d" % (args.resume, arm, rank), map_location=device, weights_only=False)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["opt"])
        g.set_state(ck["gen"])
        start = int(ck["step"])
    losses = []
    t0 = None
    for step in range(args.steps + args.warmup):
        if step == args.warmup:
            if device.type == "cuda":
                torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
        tokens = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=g).to(device, non_blocking=True)
        with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=device.type == "cuda"):
            loss = ddp(tokens[:, :-1], tokens[:, 1:])
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(loss.detach())
    if device.type == "cuda":
        torch.cuda.synchronize()
    dist.barrier()
    dt = time.perf_counter() - t0
    last = torch.stack(losses[-5:]).float().mean()
    dist.all_reduce(last)
    out = {"tokens_per_s": args.steps * args.batch * args.seq * world / dt, "final_loss": float(last) / world,
           "first_loss": float(losses[0]), "last_loss_rank0": float(losses[-1]), "steps_done": start + len(losses)}
    if getattr(args, "save", None):
        # every rank keeps its own data generator state; the weights are identical on all ranks
        torch.save({"model": model.state_dict(), "opt": opt.state_dict(), "gen": g.get_state(),
                    "step": start + len(losses)}, "%s.%s.rank%d" % (args.save, arm, rank))
        if rank == 0 and getattr(args, "save_compressed_eb", 0.0):
            from ..ops import stream_io

            out["compressed_checkpoint"] = stream_io.save_state("%s.%s.hcz" % (args.save, arm), model.state_dict(),
                                                                args.save_compressed_eb)
    if state is not None:
        state.check()  # a time-out or a missing peer in any bucket's collective surfaces here, not as silent garbage
        out["hook_calls"] = state.calls
        out["compressed_calls"] = state.compressed_calls
        state.close()
    del ddp, opt, model
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="small", choices=["small", "tiny"])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--eb", type=float, default=1e-5)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--cpu", action="store_true", help="gloo + host-rank ring (functional check without GPUs)")
    ap.add_argument("--save", default=None, help="checkpoint prefix written after the last step")
    ap.add_argument("--resume", default=None, help="checkpoint prefix to continue from")
    ap.add_argument("--save-compressed-eb", type=float, default=0.0,
                    help="also write the weights as error-bounded streams with this absolute bound")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    if args.cpu:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        a = run(args, True, rank, world, device)
        b = run(args, False, rank, world, device)
        if rank == 0:
            print(json.dumps({"model": args.model, "n_gpus": world, "batch_per_gpu": args.batch, "seq": args.seq,
                              "eb": args.eb, "bucket_mb": args.bucket_mb, "steps": args.steps,
                              "compressed": a, "nccl": b,
                              "loss_gap": a["final_loss"] - b["final_loss"],
                              "speedup_vs_nccl": a["tokens_per_s"] / b["tokens_per_s"]}), flush=True)
        return {"compressed": a, "nccl": b}
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
