"""Builds the reference library (cornflexxx/Tirocinio-Triennale, HomComp) under baseline/_ref.

The sources are copied unmodified from the reference tree, with the two things the shipped tree
cannot compile without: a stand-in ``include/comprs_test.cuh`` that only includes ``homcomp.cuh`` (the header is included
but absent, HomComp/src/GSZ_entry.cu:3) and the declaration fix in ``intra_node_allgather``
(HomComp/src/cuda_awareallreduce.cu:648-658: ``send_count`` declared twice, ``recv_count`` never).
That function is not on the benchmarked path.  One more change is needed to RUN the kernels on
B200 at all: the shared variable ``excl_sum`` is read uninitialised by the first chunk of every
kernel (see the comment in ``build``); it is set to 0 here.  ``mpi.h`` comes from csrc/mpi_shim (the single-host MPI of
this repository) because no MPI exists on the image.  Nothing of this library is used by the product.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# where the reference checkout lives: HC_REFERENCE_ROOT, the first argument of the command line, or a
# directory called "reference" beside this repository
REF = Path(os.environ.get("HC_REFERENCE_ROOT") or (HERE.parent.parent / "reference")) / "HomComp"
SHIM = HERE.parent / "csrc" / "mpi_shim"
OUT = HERE / "_ref"
LIB = OUT / "libhomcomp_ref.so"


def build(force: bool = False) -> Path | None:
    if LIB.exists() and not force:
        return LIB
    if not REF.exists():
        return LIB if LIB.exists() else None
    src, inc = OUT / "src", OUT / "include"
    src.mkdir(parents=True, exist_ok=True)
    inc.mkdir(parents=True, exist_ok=True)
    for f in ("GSZ.cu", "homcomp.cu", "GSZ_entry.cu", "cuda_awareallreduce.cu", "nca_allreduce.cu"):
        shutil.copyfile(REF / "src" / f, src / f)
    for f in (REF / "include").iterdir():
        shutil.copyfile(f, inc / f.name)
    # the absent header evidently declared the hom-sum kernels for GSZ_entry.cu (it calls them without
    # including homcomp.cuh), so the stand-in forwards to that header and adds nothing else
    (inc / "comprs_test.cuh").write_text('#pragma once\n#include "homcomp.cuh"\n')
    p = src / "cuda_awareallreduce.cu"
    text = p.read_text()
    first = text.find("size_t send_count;")
    second = text.find("size_t send_count =", first)
    if first >= 0 and second >= 0:
        text = text[:second] + "size_t recv_count;\n  send_count =" + text[second + len("size_t send_count ="):]
    p.write_text(text)
    # Undefined behaviour that faults on B200: in every kernel the __shared__ variable `excl_sum` is
    # only written by chunks with index > 0 (HomComp/src/GSZ.cu:196-222) but read by all of them
    # (`base_idx = excl_sum + rate_ofs`, GSZ.cu:237), so the first chunk's payload goes to whatever
    # offset the previous kernel left in shared memory.  On A100 that happened to read as 0; here it
    # does not, and the stores leave the buffer.  The build therefore initialises it to 0, the value
    # the code relies on; nothing else in the kernels is touched.
    for f in ("GSZ.cu", "homcomp.cu"):
        q = src / f
        t = q.read_text()
        decl = "  __shared__ unsigned int excl_sum;\n"
        t = t.replace(decl, decl + "  if (threadIdx.x == 0) excl_sum = 0; /* build_ref.py: see above */\n")
        q.write_text(t)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100,code=sm_100", "-O3", "-shared", "-Xcompiler", "-fPIC",
           "-w", "-I", str(SHIM), "-I", str(inc),
           str(src / "GSZ.cu"), str(src / "homcomp.cu"), str(src / "GSZ_entry.cu"), str(src / "cuda_awareallreduce.cu"),
           str(src / "nca_allreduce.cu"), str(HERE / "ref_driver.cu"), str(SHIM / "mpi_shim.cpp"), "-o", str(LIB), "-lcudart", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        (OUT / "build.log").write_text(r.stdout + r.stderr)
        print("reference build failed, see %s" % (OUT / "build.log"), file=sys.stderr)
        return None
    log = OUT / "build.log"
    if log.exists():
        log.unlink()
    return LIB


if __name__ == "__main__":
    if len(sys.argv) > 1:
        REF = Path(sys.argv[1]) / "HomComp"
    print(build(force=True))
