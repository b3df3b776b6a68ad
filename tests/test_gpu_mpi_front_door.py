"""The MPI front door (homcomp_mpi.h): a communicator bootstrapped from an MPI communicator and the
reference's collective called with its exact signature,
``allreduce_ring_comprs_hom_sum_F(d_sbuf, d_rbuf, count, MPI_COMM_WORLD, eb)``
(HomComp/include/cuda_awareallreduce.cuh:4-17).  No MPI is installed here, so the library is built
against the single-host MPI of csrc/mpi_shim, whose MPI_Comm is an int: the C++ symbols below are
the mangled names for that type."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

CREATE = "_Z18hc_comm_create_mpiimPP7hc_comm"          # hc_comm_create_mpi(int, unsigned long, hc_comm**)
FREE = "_Z16hc_comm_free_mpii"                         # hc_comm_free_mpi(int)
ALLREDUCE_F = "_Z31allreduce_ring_comprs_hom_sum_FPKfPfmif"  # (const float*, float*, unsigned long, int, float)
RING_GPU = "_Z18allreduce_ring_gpuPKfPfmi"             # allreduce_ring_gpu(const float*, float*, unsigned long, int)
MPI_COMM_WORLD = 0


def _worker(rank, world):
    from datasets import gradient_like
    from tirocinio_triennale_b200 import _build, ops

    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["HCREF_SLOT_BYTES"] = str(1 << 20)  # mailbox size of the stand-in MPI: handles only
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    lib = C.CDLL(str(_build.build_mpi()), mode=C.RTLD_GLOBAL)
    assert lib.MPI_Init(None, None) == 0
    n, eb = 700_001, 1e-4
    create = getattr(lib, CREATE)
    create.argtypes = [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
    handle = C.c_void_p()
    assert create(MPI_COMM_WORLD, n, C.byref(handle)) == 0 and handle.value
    allreduce = getattr(lib, ALLREDUCE_F)
    allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_float]
    ring_gpu = getattr(lib, RING_GPU)
    ring_gpu.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    bufs = [gradient_like(n, seed=60 + r) for r in range(world)]
    want = ops.cpu_ring_allreduce(bufs, eb)[rank]
    x = torch.from_numpy(bufs[rank]).cuda()
    for _ in range(2):
        out = torch.full_like(x, -1.0)
        assert allreduce(x.data_ptr(), out.data_ptr(), n, MPI_COMM_WORLD, eb) == 0
        torch.cuda.synchronize()
        np.testing.assert_array_equal(out.cpu().numpy(), want)
    out = torch.zeros_like(x)
    assert ring_gpu(x.data_ptr(), out.data_ptr(), n, MPI_COMM_WORLD) == 0
    torch.cuda.synchronize()
    raw = torch.zeros(n)
    for b in bufs:
        raw += torch.from_numpy(b)
    assert torch.equal(out.cpu(), raw)
    # a communicator nobody created a handle for is an argument error, not a crash
    assert allreduce(x.data_ptr(), out.data_ptr(), n, 12345, eb) == 4
    assert getattr(lib, FREE)(MPI_COMM_WORLD) == 0
    assert lib.MPI_Finalize() == 0


def test_reference_signature_with_an_mpi_communicator():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_worker, 2)
