"""Error metrics of a lossy reconstruction: the set printed by the reference's evaluation tool
(max abs / max rel error, PSNR, NRMSE, Pearson correlation, compression ratio;
HomComp/src/homcomp_eval.cu:72-133)."""
from __future__ import annotations

import math

import torch


def error_metrics(ref: torch.Tensor, rec: torch.Tensor, compressed_bytes: int | None = None) -> dict:
    a = ref.reshape(-1).double()
    b = rec.reshape(-1).double()
    diff = (a - b).abs()
    rng = float(a.max() - a.min())
    mse = float((diff * diff).mean())
    max_abs = float(diff.max())
    denom = a.abs().clamp_min(1e-300)
    max_rel = float((diff / denom)[a != 0].max()) if bool((a != 0).any()) else 0.0
    nrmse = math.sqrt(mse) / rng if rng > 0 else float("nan")
    psnr = 20 * math.log10(rng) - 10 * math.log10(mse) if mse > 0 and rng > 0 else float("inf")
    am, bm = a - a.mean(), b - b.mean()
    den = float(am.norm() * bm.norm())
    pearson = float((am * bm).sum()) / den if den > 0 else float("nan")
    out = {"max_abs_err": max_abs, "max_rel_err": max_rel, "psnr_db": psnr, "nrmse": nrmse, "pearson": pearson,
           "value_range": rng}
    if compressed_bytes:
        out["compression_ratio"] = a.numel() * 4 / compressed_bytes
    return out
