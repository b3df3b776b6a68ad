"""Per-CTA timeline of the codec kernels (instrumented build, ``-DHC_TIMELINE``).

    HC_TIMELINE=1 python -m tirocinio_triennale_b200.utils.timeline --n 16777216 --ops compress,decompress,hom_add,reduce7

The instrumented library (``_build.build_cuda(timeline=True)`` -> ``libhomcomp_b200_tl.so``) makes
every CTA write, for the last four launches, nanosecond stamps of its first tile's way through the
loader / compute / scanner warps (slots 0-15) and, for its first compute warp, the SM-clock cycles
spent in each phase of the tile loop (slots 16-30) plus the number of tiles it handled (slot 31).
``hc_debug_timeline`` copies them to the host.  This module runs one operation at a time and prints
the device span of the launch (first CTA in to last CTA out) and the share of each phase.
The reference has no tracing of any kind (its thesis used Nsight Compute by hand).
"""
from __future__ import annotations

import argparse
import ctypes as C
import os

import numpy as np

SLOTS = 32
ENCODE_PHASES = ["wait input stream", "decode input", "wait fp32 tile", "load+quantise+lorenzo", "analyse",
                 "(unused)", "copy out (+wait for ring space)", "pack", "scan (barrier)", "rate store+transpose",
                 "S: wait tile total", "S: look-back"]
N_COMPUTE_PHASES = 10  # "S:" entries are the scanner warp's
DECODE_PHASES = ["wait input stream", "decode", "dequantise", "wait tma store+barrier", "store tile+barrier"]


def read(lib) -> np.ndarray:
    """(4 launches, 1024 CTAs, 32 slots) int64; clears the device copy."""
    lib.hc_debug_timeline.restype = C.c_int
    lib.hc_debug_timeline.argtypes = [C.c_void_p]
    a = np.zeros((4, 1024, SLOTS), dtype=np.uint64)
    if lib.hc_debug_timeline(a.ctypes.data) != 0:
        raise RuntimeError("hc_debug_timeline failed")
    return a.astype(np.int64)


def summarise(a: np.ndarray, phases):
    """One dict per launch that left stamps: device span in microseconds, CTAs, tiles, phase shares."""
    out = []
    for e in range(a.shape[0]):
        g = a[e]
        g = g[g[:, 0] > 0]
        if not len(g):
            continue
        cyc = g[:, 16:16 + len(phases)].sum(axis=0).astype(np.float64)
        nc = N_COMPUTE_PHASES if len(phases) > N_COMPUTE_PHASES else len(phases)
        tot = cyc[:nc].sum()
        out.append({
            "span_us": (g[:, 7].max() - g[:, 0].min()) / 1e3,
            "start_spread_us": (g[:, 0].max() - g[:, 0].min()) / 1e3,
            "ctas": int(len(g)), "tiles_first_warp": int(g[:, SLOTS - 1].sum()),
            "cycles_per_tile": tot / max(1, int(g[:, SLOTS - 1].sum())),
            "phase_share": {p: (c / tot if tot else 0.0) for p, c in zip(phases, cyc)},
        })
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=16 * 1024 * 1024)
    ap.add_argument("--eb", type=float, default=1e-4)
    ap.add_argument("--ops", default="compress,decompress,hom_add")
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if os.environ.get("HC_TIMELINE", "0") in ("", "0"):
        raise SystemExit("set HC_TIMELINE=1 so that the instrumented library is loaded")
    import torch

    from .. import _lib, ops
    from . import datagen

    lib = _lib.cuda()
    n = args.n
    x = datagen.gradient_like(n, 0, "cuda")
    y = datagen.gradient_like(n, 1, "cuda")
    codec = ops.Codec(n)
    stream, size = codec.compress(x, args.eb)
    nbytes = int(size.item())
    out = torch.empty_like(stream)
    dec = torch.empty_like(x)
    size2 = torch.zeros_like(size)
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.int32, device="cuda")
    read(lib)
    parts = None
    for op in args.ops.split(","):
        for rep in range(args.reps):
            flush.add_(1)
            torch.cuda.synchronize()
            if op == "compress":
                codec.compress(x, args.eb, out=out, size=size2)
                phases = ENCODE_PHASES
            elif op == "decompress":
                codec.decompress(stream, n, args.eb, out=dec, stream_bytes=nbytes)
                phases = DECODE_PHASES
            elif op == "hom_add":
                codec.hom_add(stream, y, args.eb, out=out, size=size2, stream_bytes=nbytes)
                phases = ENCODE_PHASES
            elif op == "reduce7":
                # the reduce step of an 8-rank allreduce on one GPU: 7 streams (+) fp32 of n / 8 values
                if parts is None:
                    chunk = n // 8 // 4096 * 4096
                    parts = codec.compress_batch([x[(k + 1) * chunk: (k + 2) * chunk] for k in range(7)], args.eb)
                    part_bytes = [int(v) for v in parts[1].tolist()]
                    read(lib)
                codec.hom_add_multi(parts[0], y[:chunk], args.eb, stream_bytes=part_bytes)
                phases = ENCODE_PHASES
            else:
                raise SystemExit("unknown op " + op)
            for s in summarise(read(lib), phases):
                shares = ", ".join("%s %.0f%%" % (k, 100 * v) for k, v in s["phase_share"].items())
                print("%s rep %d: span %.1f us, %d CTAs (start spread %.1f us), %.0f cycles/tile of the first compute "
                      "warp: %s" % (op, rep, s["span_us"], s["ctas"], s["start_spread_us"], s["cycles_per_tile"],
                                    shares), flush=True)
    assert codec.status() == 0


if __name__ == "__main__":
    main()
