"""Device-side timing helpers: CUDA events on the launching stream, L2 flush between iterations,
clock sampling through nvidia-smi while the timed region runs."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import tempfile
import time
from pathlib import Path

import torch

L2_BYTES = 126 * 1024 * 1024


class L2Flusher:
    """Writes a buffer larger than L2 so the next timed launch starts from DRAM."""

    def __init__(self, device=None, nbytes: int = 2 * L2_BYTES):
        self.buf = torch.empty(nbytes // 4, dtype=torch.int32, device=device or "cuda")

    def __call__(self):
        self.buf.add_(1)


def time_cuda(fn, iters: int = 20, warmup: int = 3, flush: L2Flusher | None = None):
    """Times ``fn`` with CUDA events, one event pair per iteration; returns milliseconds per call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return times


def measured_peaks() -> dict:
    """The pool's measured copy bandwidth and GEMM rate; fallback values when the file is absent."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            t0 = time.time()
            while os.path.getsize(self.path) == 0 and time.time() - t0 < 5.0:  # first sample is in
                time.sleep(0.05)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(2.5 * self.period_ms / 1000.0)  # at least one more sample after the region
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def bind_host_thread_near_gpu(device_index: int) -> str:
    """Pins the calling process to the CPUs of the NUMA node that the GPU hangs off (sysfs
    ``local_cpulist`` of its PCI device), so that pinned host buffers allocated afterwards are local to
    the GPU's PCIe root and the copy engines do not cross the socket interconnect.  Returns a short
    description of what was done; never raises (containers may hide sysfs)."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        addr = "%04x:%02x:%02x.0" % (getattr(props, "pci_domain_id", 0), props.pci_bus_id, props.pci_device_id)
        base = Path("/sys/bus/pci/devices") / addr
        cpus = (base / "local_cpulist").read_text().strip()
        node = (base / "numa_node").read_text().strip()
        ids = set()
        for part in cpus.split(","):
            if "-" in part:
                a, b = part.split("-")
                ids.update(range(int(a), int(b) + 1))
            elif part:
                ids.add(int(part))
        allowed = ids & set(os.sched_getaffinity(0))
        if not allowed:
            return "gpu %d: numa node %s, no allowed cpu in %s" % (device_index, node, cpus)
        os.sched_setaffinity(0, allowed)
        return "gpu %d: numa node %s, bound to %d cpus" % (device_index, node, len(allowed))
    except Exception as e:  # noqa: BLE001
        return "gpu %d: not bound (%s)" % (device_index, str(e)[:80])
