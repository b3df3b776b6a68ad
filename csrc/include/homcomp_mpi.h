// MPI front door: the reference's collective entry points with their exact signatures, taking a real
// MPI_Comm (HomComp/include/cuda_awareallreduce.cuh:4-17, nca_allreduce.cuh:3-15).
//
// Compile with -DHC_WITH_MPI and your MPI's <mpi.h> on the include path, and link hc_mpi.cu (or
// libhomcomp_b200_mpi.so) next to libhomcomp_b200.so.  MPI is used for the bootstrap only, as host
// MPI is in the reference's CUDA-aware build only for moving the bytes: hc_comm_create_mpi reads
// rank and size, allocates this rank's symmetric region, passes its 64-byte CUDA IPC handle round
// the communicator with MPI_Sendrecv, maps the peers' regions and creates the hc_comm.  After that
// no call of this library touches MPI: every collective is kernels storing into peer memory.
//
// The collectives look their hc_comm up by communicator, so call hc_comm_create_mpi once per
// communicator first (the reference needs no such step; its functions take whatever communicator
// they are given and allocate per call).  Ranks of one communicator must be able to map each other's
// memory (one node, or one NVLink domain).
//
// Where no MPI is installed, csrc/mpi_shim provides a single-host one (processes started by any
// launcher that sets RANK / WORLD_SIZE / MASTER_PORT), enough for this header and its tests.
#pragma once
#ifdef HC_WITH_MPI
#include <mpi.h>
#include <stddef.h>

#include "homcomp_b200.h"

// Collective over `comm`.  max_count: largest message (values) of later calls.  Returns 0 or a
// hc::Status code; *out (optional) receives the handle, which hc_comm_free_mpi releases.
int hc_comm_create_mpi(MPI_Comm comm, size_t max_count, hc_comm** out);
// The handle created for `comm`, or NULL.
hc_comm* hc_comm_from_mpi(MPI_Comm comm);
// Collective: waits for the device, meets the other ranks, unmaps and frees.
int hc_comm_free_mpi(MPI_Comm comm);

int allreduce_ring_comprs_hom_sum(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F_opt(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int mixed_compressed_allreduce(float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_gpu(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm);
#endif  // HC_WITH_MPI
