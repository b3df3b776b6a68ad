"""Single-GPU codec evaluation: throughput of compress / decompress / fused homomorphic add, the
decompress-operate-compress (DOC) alternative it replaces, compression ratio and error metrics.

Counterpart of the reference's homcomp_eval tool (HomComp/src/homcomp_eval.cu:135-236), timed with
CUDA events and an L2 flush between iterations instead of gettimeofday.

    python -m tirocinio_triennale_b200.utils.eval_codec --data blob --eb 1e-3 --iters 10
    python -m tirocinio_triennale_b200.utils.eval_codec --file field.bin --eb 1e-4 --rel
"""
from __future__ import annotations

import argparse
import json
import statistics

import numpy as np
import torch

from .. import ops
from . import datagen, metrics, timing


def make_data(args) -> torch.Tensor:
    if args.file:
        return torch.from_numpy(np.fromfile(args.file, dtype=np.float32)).cuda()
    if args.data == "blob":
        return datagen.blob_field_3d(tuple(args.shape), args.seed, "cuda")
    if args.data == "sinusoid":
        return datagen.sinusoid_field(args.n, args.seed, "cuda")
    if args.data == "gradient":
        return datagen.gradient_like(args.n, args.seed, "cuda")
    return datagen.from_distribution(args.n, args.data, args.seed, "cuda", smooth=args.smooth)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data", default="blob",
                    choices=["blob", "sinusoid", "gradient", "uniform", "normal", "exponential", "randomwalk"])
    ap.add_argument("--file", default=None, help="raw float32 file (as written by the dataset generator)")
    ap.add_argument("--n", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--shape", type=int, nargs=3, default=[512, 512, 256])
    ap.add_argument("--eb", type=float, default=1e-3)
    ap.add_argument("--rel", action="store_true", help="error bound relative to the value range")
    ap.add_argument("--mode", default="outlier", choices=["outlier", "plain", "vec"])
    ap.add_argument("--smooth", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ops", default="compress,decompress,hom_add,doc",
                    help="comma list of compress,decompress,hom_add,doc,scatter7,reduce7,sum4 (scatter7, reduce7: the "
                         "shapes of an 8-rank allreduce on one GPU: 7-segment compress of 7/8 of the data, 7 streams "
                         "(+) fp32 of 1/8 of it; sum4: four streams of a quarter of the data decoded and summed by "
                         "one kernel, step 2 of the one-step allreduce at 4 ranks)")
    args = ap.parse_args(argv)

    x = make_data(args)
    n = x.numel()
    eb = args.eb * float(x.max() - x.min()) if args.rel else args.eb
    codec = ops.Codec(n)
    flush = timing.L2Flusher()
    peaks = timing.measured_peaks()
    out, size = codec.compress(x, eb, args.mode)
    nbytes = int(size.item())
    y = codec.decompress(out, n, eb, args.mode)
    res = {"n": n, "eb": eb, "mode": args.mode, "compressed_bytes": nbytes,
           **metrics.error_metrics(x, y, nbytes), "peaks": peaks["source"]}
    out2, size2 = codec.hom_add(out, x, eb, args.mode, stream_bytes=nbytes)
    z = codec.decompress(out2, n, eb, args.mode)
    res["hom_add_max_abs_err_vs_2x"] = float((z.double() - 2 * x.double()).abs().max())
    gb = n * 4 / 1e9
    want = set(args.ops.split(","))

    def report(name, fn, bytes_moved):
        t = timing.time_cuda(fn, args.iters, args.warmup, flush)
        ms = statistics.median(t)
        res[name] = {"ms": ms, "GBps_of_fp32": gb / ms * 1e3, "hbm_fraction_of_%s" % peaks["source"]:
                     bytes_moved / 1e9 / ms * 1e3 / peaks["hbm_gbs"]}

    if "compress" in want:
        report("compress", lambda: codec.compress(x, eb, args.mode, out=out, size=size), 4 * n + nbytes)
    if "decompress" in want:
        report("decompress", lambda: codec.decompress(out, n, eb, args.mode, out=y, stream_bytes=nbytes), 4 * n + nbytes)
    if "hom_add" in want:
        report("hom_add", lambda: codec.hom_add(out, x, eb, args.mode, out=out2, size=size2, stream_bytes=nbytes),
               4 * n + 2 * nbytes)
    if "doc" in want:
        tmp = torch.empty_like(x)

        def doc():  # decompress, add in fp32, compress again
            codec.decompress(out, n, eb, args.mode, out=tmp, stream_bytes=nbytes)
            codec.sum(tmp, tmp, x)
            codec.compress(tmp, eb, args.mode, out=out2, size=size2)

        report("doc", doc, 4 * n * 5 + 2 * nbytes)
    if "scatter7" in want or "reduce7" in want:
        # what rank 0 of 8 does in the direct algorithm, without the peers: chunk = n / 8
        chunk = n // 8 // 4096 * 4096
        parts = [x[(k + 1) * chunk: (k + 2) * chunk] for k in range(7)]
        if "scatter7" in want:
            report("scatter7", lambda: codec.compress_batch(parts, eb, args.mode), 7 * 4 * chunk + 7 * nbytes // 8)
        if "reduce7" in want:
            outs, sizes = codec.compress_batch(parts, eb, args.mode)
            nb = [int(v) for v in sizes.tolist()]
            report("reduce7", lambda: codec.hom_add_multi(outs, x[:chunk], eb, args.mode, stream_bytes=nb),
                   4 * chunk + 8 * nbytes // 8)
    if "sum4" in want:
        # what a rank of 4 does in step 2 of the one-step allreduce, without the peers: four streams of
        # n / 4 values decoded and summed by one kernel
        part = n // 4 // 4096 * 4096
        outs, sizes = codec.compress_batch([x[k * part: (k + 1) * part] for k in range(4)], eb, args.mode)
        nb = [int(v) for v in sizes.tolist()]
        dst = torch.empty(part, dtype=torch.float32, device="cuda")
        report("sum4", lambda: codec.decompress_sum(outs, part, eb, out=dst, stream_bytes=nb), 4 * part + sum(nb))
    res["status"] = codec.status()
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
