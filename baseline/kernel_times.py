"""Kernel against kernel on the same GPU: the reference's three hot kernels alone (scratch allocated
once, clearing outside the timed region: ``ref_kernel_times`` in ref_driver.cu) next to this
library's compress / decompress / fused add on the same input, CUDA events, median.

    python baseline/kernel_times.py [--n 16777216] [--eb 1e-4] [--data gradient|blob] [--iters 9]

Prints one JSON line.  Input larger than L2 by default (64 MiB in, rotating is not needed: every
launch streams through the whole buffer).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=16 * 1024 * 1024)
    ap.add_argument("--eb", type=float, default=1e-4)
    ap.add_argument("--data", default="gradient", choices=["gradient", "blob", "sinusoid"])
    ap.add_argument("--iters", type=int, default=9)
    args = ap.parse_args()
    import torch

    import build_ref
    from tirocinio_triennale_b200 import ops
    from tirocinio_triennale_b200.utils import datagen, timing

    n = args.n
    if args.data == "blob":
        x = datagen.blob_field_3d((512, 512, 256), seed=0, device="cuda").reshape(-1)
        n = x.numel()
    elif args.data == "sinusoid":
        x = datagen.sinusoid_field(n, 0, "cuda")
    else:
        x = datagen.gradient_like(n, 0, "cuda")
    n_pad = (n + 32767) // 32768 * 32768  # the reference kernels process whole chunks
    xp = torch.zeros(n_pad, device="cuda")
    xp[:n] = x
    out = {"n": n, "eb": args.eb, "data": args.data, "iters": args.iters}

    lib_path = build_ref.build()
    if lib_path is not None and os.path.exists(lib_path):
        lib = C.CDLL(str(lib_path))
        lib.ref_kernel_times.restype = C.c_int
        lib.ref_kernel_times.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_int,
                                         C.POINTER(C.c_float)]
        cmp1 = torch.zeros(n_pad * 4 + n_pad // 32 + 65536, dtype=torch.uint8, device="cuda")
        cmp2 = torch.zeros_like(cmp1)
        dec = torch.zeros(n_pad, device="cuda")
        ms = (C.c_float * 3)()
        rc = lib.ref_kernel_times(xp.data_ptr(), cmp1.data_ptr(), cmp2.data_ptr(), dec.data_ptr(), n_pad, args.eb,
                                  args.iters, ms)
        torch.cuda.synchronize()
        out["reference_ms"] = {"compress": ms[0], "decompress": ms[1], "hom_sum_F": ms[2], "rc": rc}
        del cmp1, cmp2, dec
    else:
        out["reference_ms"] = None

    codec = ops.Codec(n_pad)
    stream, size = codec.compress(xp, args.eb)
    nbytes = int(size.item())
    out["compressed_bytes"] = nbytes
    out["compression_ratio"] = 4.0 * n_pad / nbytes
    dec = torch.empty_like(xp)
    out2 = torch.empty_like(stream)
    size2 = torch.zeros_like(size)
    flush = timing.L2Flusher()
    med = lambda v: statistics.median(v)
    ours = {
        "compress": med(timing.time_cuda(lambda: codec.compress(xp, args.eb, out=out2, size=size2), args.iters, 3, flush)),
        "decompress": med(timing.time_cuda(lambda: codec.decompress(stream, n_pad, args.eb, out=dec, stream_bytes=nbytes),
                                           args.iters, 3, flush)),
        "hom_add": med(timing.time_cuda(lambda: codec.hom_add(stream, xp, args.eb, out=out2, size=size2, stream_bytes=nbytes),
                                        args.iters, 3, flush)),
    }
    assert codec.status() == 0
    out["ours_ms"] = ours
    peaks = timing.measured_peaks()
    raw = 4.0 * n_pad
    out["ours_fraction_of_hbm"] = {
        "compress": (raw + nbytes) / (ours["compress"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "decompress": (raw + nbytes) / (ours["decompress"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "hom_add": (raw + 2 * nbytes) / (ours["hom_add"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
    }
    out["ours_gbs_of_fp32"] = {k: raw / (v * 1e-3) / 1e9 for k, v in ours.items()}
    if out["reference_ms"]:
        r = out["reference_ms"]
        out["speedup"] = {"compress": r["compress"] / ours["compress"], "decompress": r["decompress"] / ours["decompress"],
                          "hom_add": r["hom_sum_F"] / ours["hom_add"]}
        out["reference_gbs_of_fp32"] = {k: raw / (r[k] * 1e-3) / 1e9 for k in ("compress", "decompress", "hom_sum_F")}
    out["peaks"] = peaks["source"]
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
