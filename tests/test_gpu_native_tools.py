"""The native command-line tools (C++ against the reference-named API, no Python in the data path)."""
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tools():
    from tirocinio_triennale_b200 import _build

    return {p.name: p for p in _build.build_cli()}


def test_homcomp_eval_tool():
    exe = _tools()["homcomp_eval"]
    r = subprocess.run([str(exe), "gen:3000000", "1e-4", "ABS", "3"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("max abs err")][0]
    err = float(line.split()[3])
    assert err <= 2e-4 * 1.01  # two quantisation errors
    assert "status no error" in r.stdout


def test_reference_named_entry_points_and_their_capacity_rule():
    """compat_check: round trips through the GSZ_* / homomorphic_sum_F names, and incompressible input
    (31 bit planes in every block) with a canary behind the output buffer under both capacity rules."""
    exe = _tools()["compat_check"]
    r = subprocess.run([str(exe), "1000003"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("ok") and "FAIL" not in r.stdout


@pytest.mark.multigpu
def test_allreduce_threads_tool():
    n = min(torch.cuda.device_count(), 8)
    exe = _tools()["allreduce_threads"]
    r = subprocess.run([str(exe), str(n), "2000000", "1e-4", "3"], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("ok")
    # the same run over regions built by the library's own multicast bootstrap (driver VMM API): the
    # compressed result must be the same bits (the line carries a checksum of rank 0's output)
    m = subprocess.run([str(exe), str(n), "2000000", "1e-4", "3", "nvls"], capture_output=True, text=True, timeout=180)
    assert m.returncode == 0, m.stdout + m.stderr
    assert m.stdout.strip().endswith("ok")
    checksum = lambda text: text.split("checksum")[1].split()[0]
    assert checksum(m.stdout) == checksum(r.stdout)
