"""Builds the native libraries in-tree.

``libhomcomp_cpu.so``   g++ only: the portable codec, the host-rank ring (the oracle).
``libhomcomp_b200.so``  nvcc, ``-gencode arch=compute_100a,code=sm_100a``: everything above plus the
                        sm_100a kernels, the device codec API and the collectives.

The reference builds with a Makefile that passes no ``-arch`` at all (HomComp/src/Makefile:1-4).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

CPU_SOURCES = ["cpu/hc_cpu_codec.cpp", "cpu/hc_cpu_ring.cpp"]
CUDA_SOURCES = ["cuda/hc_kernels.cu", "cuda/hc_api.cu", "cuda/hc_ring.cu", "cuda/hc_compat.cu", "cuda/hc_noalloc.cu",
                "cuda/hc_host_staged.cu", "cuda/hc_multicast.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off", "--fmad=false",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off"]


def _existing(sources):
    return [s for s in sources if (CSRC / s).exists()]


def _newest_source_mtime() -> float:
    m = 0.0
    for p in CSRC.rglob("*"):
        if p.suffix in (".cu", ".cuh", ".h", ".cpp"):
            m = max(m, p.stat().st_mtime)
    return m


def _stale(lib: Path) -> bool:
    return (not lib.exists()) or lib.stat().st_mtime < _newest_source_mtime()


def nvcc_path() -> str | None:
    for cand in (os.environ.get("HC_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def build_cpu(force: bool = False) -> Path:
    lib = LIBDIR / "libhomcomp_cpu.so"
    if force or _stale(lib):
        LIBDIR.mkdir(parents=True, exist_ok=True)
        tmp = lib.with_suffix(".so.tmp%d" % os.getpid())
        _run(["g++", *CXX_FLAGS, "-shared", "-I", str(CSRC / "include"),
              *[str(CSRC / s) for s in CPU_SOURCES], "-o", str(tmp)])
        os.replace(tmp, lib)
    return lib


def build_cuda(force: bool = False, verbose: bool = False, timeline: bool = False) -> Path:
    """``timeline=True`` builds a second library, ``libhomcomp_b200_tl.so``, whose kernels stamp a
    per-CTA timeline (``-DHC_TIMELINE``; read it with ``utils/timeline.py``).  Slower; never the default."""
    lib = LIBDIR / ("libhomcomp_b200_tl.so" if timeline else "libhomcomp_b200.so")
    if not (force or _stale(lib)):
        return lib
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a library")
    LIBDIR.mkdir(parents=True, exist_ok=True)
    # the ranks of a job import the package at the same time: one of them builds, the others wait
    # for it and find the library fresh (they share the object files, so two builds at once would
    # link each other's half-written objects)
    import fcntl

    with open(LIBDIR / (".build_tl.lock" if timeline else ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not _stale(lib):
            return lib
        return _build_cuda_locked(lib, nvcc, verbose, timeline)


def _build_cuda_locked(lib: Path, nvcc: str, verbose: bool, timeline: bool) -> Path:
    objdir = OBJDIR / "tl" if timeline else OBJDIR
    objdir.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(CSRC / "include"), "-I", str(CSRC / "cuda")]

    def compile_one(src: str) -> str:
        obj = objdir / (Path(src).name + ".o")
        s = CSRC / src
        if src.endswith(".cu"):
            extra = (["-Xptxas", "-v"] if verbose else []) + (["-DHC_TIMELINE"] if timeline else [])
            out = _run([nvcc, *NVCC_FLAGS, *extra, *inc, "-c", str(s), "-o", str(obj)])
        else:
            out = _run(["g++", *CXX_FLAGS, *inc, "-c", str(s), "-o", str(obj)])
        if verbose and out.strip():
            print(out, file=sys.stderr)
        return str(obj)

    sources = _existing(CUDA_SOURCES) + CPU_SOURCES
    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    tmp = lib.with_suffix(".so.tmp%d" % os.getpid())
    _run([nvcc, "-shared", "-o", str(tmp), *objs, "-lcudart", "-ldl"])
    os.replace(tmp, lib)
    return lib


def build_mpi(mpi_include: str | None = None, mpi_sources=(), mpi_link=(), force: bool = False) -> Path:
    """``libhomcomp_b200_mpi.so``: the MPI front door (csrc/cuda/hc_mpi.cu, ``-DHC_WITH_MPI``) next to the
    main library.  ``mpi_include`` is the directory of ``mpi.h``, ``mpi_link`` extra linker arguments
    (e.g. ``["-lmpi"]``), ``mpi_sources`` extra sources to compile in.  With no arguments the single-host
    MPI of csrc/mpi_shim is compiled in, which is all a machine without MPI needs."""
    base = build_cuda()
    lib = LIBDIR / "libhomcomp_b200_mpi.so"
    if mpi_include is None:
        mpi_include = str(CSRC / "mpi_shim")
        mpi_sources = [str(CSRC / "mpi_shim" / "mpi_shim.cpp")]
        mpi_link = ["-lrt"]
    if not (force or _stale(lib) or lib.stat().st_mtime < base.stat().st_mtime):
        return lib
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found")
    tmp = lib.with_suffix(".so.tmp%d" % os.getpid())
    _run([nvcc, *NVCC_FLAGS, "-DHC_WITH_MPI", "-shared", "-I", mpi_include, "-I", str(CSRC / "include"),
          "-I", str(CSRC / "cuda"), str(CSRC / "cuda" / "hc_mpi.cu"), *mpi_sources, "-o", str(tmp), "-L", str(LIBDIR),
          "-lhomcomp_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lcudart", *mpi_link])
    os.replace(tmp, lib)
    return lib


CLI_SOURCES = ["cli/homcomp_eval.cu", "cli/allreduce_threads.cu", "cli/compat_check.cu"]
BINDIR = Path(__file__).resolve().parent / "bin"


def build_cli(force: bool = False):
    """Native command-line tools linked against libhomcomp_b200.so (rpath to the in-tree lib)."""
    lib = build_cuda()
    nvcc = nvcc_path()
    BINDIR.mkdir(parents=True, exist_ok=True)
    outs = []
    for src in CLI_SOURCES:
        exe = BINDIR / Path(src).stem
        s = CSRC / src
        if force or not exe.exists() or exe.stat().st_mtime < max(s.stat().st_mtime, lib.stat().st_mtime):
            _run([nvcc, *NVCC_FLAGS, "-I", str(CSRC / "include"), str(s), "-o", str(exe), "-L", str(LIBDIR),
                  "-lhomcomp_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib", "-lpthread"])
        outs.append(exe)
    return outs


if __name__ == "__main__":
    print(build_cpu(force="--force" in sys.argv))
    print(build_cuda(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--timeline" in sys.argv:
        print(build_cuda(force="--force" in sys.argv, timeline=True))
    print(build_cli(force="--force" in sys.argv))
    print(build_mpi(force="--force" in sys.argv))
