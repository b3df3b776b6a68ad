"""Writes synthetic float datasets as raw binary or CSV files.

Same distributions, flags and file naming as the reference's generator
(HomComp/src/utils/dataset_generator.py:9-66): ``<dist>_smooth-<bool>_idx-<nnn>_<size>MB.<ext>``,
plus the three fields this project's benchmarks use (``sinusoid``, ``blob``, ``gradient``).

    python -m tirocinio_triennale_b200.utils.dataset_generator --dist normal --size 250000000 --format bin
"""
from __future__ import annotations

import argparse
import os

import numpy as np
import torch

from . import datagen


def main(argv=None):
    ap = argparse.ArgumentParser(description="Generate/save float datasets as CSV or binary")
    ap.add_argument("--outdir", default="datasets")
    ap.add_argument("--size", type=int, default=1000, help="number of elements per file")
    ap.add_argument("--dtype", default="float32", choices=["float32", "float64"])
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--dist", default="uniform",
                    choices=["uniform", "normal", "exponential", "randomwalk", "sinusoid", "blob", "gradient"])
    ap.add_argument("--files", type=int, default=1)
    ap.add_argument("--mean", type=float, default=0.0)
    ap.add_argument("--std", type=float, default=1.0)
    ap.add_argument("--low", type=float, default=0.0)
    ap.add_argument("--high", type=float, default=1.0)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--smooth", action="store_true")
    ap.add_argument("--kernel-size", type=int, default=5)
    ap.add_argument("--format", default="csv", choices=["csv", "bin"])
    ap.add_argument("--rw-mean", type=float, default=0.0)
    ap.add_argument("--rw-std", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    os.makedirs(a.outdir, exist_ok=True)
    paths = []
    for idx in range(a.files):
        seed = a.seed + idx
        if a.dist == "sinusoid":
            x = datagen.sinusoid_field(a.size, seed, a.device)
        elif a.dist == "blob":
            side = max(8, round(a.size ** (1 / 3)))
            x = datagen.blob_field_3d((side, side, max(1, a.size // (side * side))), seed, a.device)
        elif a.dist == "gradient":
            x = datagen.gradient_like(a.size, seed, a.device)
        else:
            x = datagen.from_distribution(a.size, a.dist, seed, a.device, a.mean, a.std, a.low, a.high, a.scale,
                                          a.rw_mean, a.rw_std, a.smooth, a.kernel_size)
        arr = x.cpu().numpy().astype(np.float32 if a.dtype == "float32" else np.float64)
        base = "%s_smooth-%s_idx-%03d" % (a.dist, a.smooth, idx)
        tmp = os.path.join(a.outdir, base + "." + a.format)
        if a.format == "csv":
            np.savetxt(tmp, arr, header="value", comments="", fmt="%.9g")
        else:
            arr.tofile(tmp)
        mb = os.path.getsize(tmp) / (1024 * 1024)
        final = os.path.join(a.outdir, "%s_%.2fMB.%s" % (base, mb, a.format))
        os.replace(tmp, final)
        print("Saved: %s (%.2f MB)" % (final, mb))
        paths.append(final)
    return paths


if __name__ == "__main__":
    main()
