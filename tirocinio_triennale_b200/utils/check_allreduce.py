"""Checks an allreduce result against its input when every rank held the same data.

Counterpart of the reference's checker (HomComp/src/utils/checksmooth.c:42-63): expected value
is ``world * input``; a value passes when ``|world * in - out| <= 2 * eb * (world + world / 10)``;
values that came back exactly zero while the expectation is not are listed, because that is the
symptom of a dropped block.  Accepts the text files the reference's drivers write
(one value per line) or raw float32 files.

    python -m tirocinio_triennale_b200.utils.check_allreduce smooth.in smooth.out --world 4 --eb 1e-4
"""
from __future__ import annotations

import argparse
import sys

import numpy as np


def load(path: str) -> np.ndarray:
    if path.endswith((".bin", ".f32", ".dat")):
        return np.fromfile(path, dtype=np.float32)
    return np.loadtxt(path, dtype=np.float64, ndmin=1)


def check(inp: np.ndarray, out: np.ndarray, world: int, eb: float, strict: bool = False) -> dict:
    n = min(inp.size, out.size)
    exp = inp[:n].astype(np.float64) * world
    diff = np.abs(exp - out[:n].astype(np.float64))
    tol = world * eb * 1.0001 if strict else 2 * eb * (world + world / 10)
    bad = np.nonzero(diff > tol)[0]
    zeros = np.nonzero((out[:n] == 0) & (np.abs(exp) > tol))[0]
    return {"n": int(n), "tolerance": tol, "max_abs_err": float(diff.max()) if n else 0.0,
            "violations": int(bad.size), "first_violations": bad[:10].tolist(),
            "unexpected_zeros": int(zeros.size), "first_zeros": zeros[:10].tolist(),
            "ok": bad.size == 0 and zeros.size == 0}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("input")
    ap.add_argument("output")
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--eb", type=float, default=1e-4)
    ap.add_argument("--strict", action="store_true", help="tolerance world * eb (this library's guarantee)")
    a = ap.parse_args(argv)
    r = check(load(a.input), load(a.output), a.world, a.eb, a.strict)
    print(r)
    return 0 if r["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
