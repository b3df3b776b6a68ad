// extern "C" doorway into the reference library for the Python benchmark arm: it only forwards to
// the reference's own public functions (HomComp/include/GSZ_entry.h, cuda_awareallreduce.cuh).
#include <cuda_runtime.h>
#include <mpi.h>
#include <stddef.h>

#include "GSZ_entry.h"
#include "cuda_awareallreduce.cuh"

extern "C" {

int ref_init(void) { return MPI_Init(nullptr, nullptr); }
int ref_finalize(void) { return MPI_Finalize(); }
int ref_barrier(void) { return MPI_Barrier(MPI_COMM_WORLD); }
int ref_current_device(void) {
  int d = -1;
  cudaGetDevice(&d);
  return d;
}

int ref_allreduce_F(const float* d_sbuf, float* d_rbuf, size_t count, float eb) {
  return allreduce_ring_comprs_hom_sum_F(d_sbuf, d_rbuf, count, MPI_COMM_WORLD, eb);
}
int ref_allreduce_F_opt(const float* d_sbuf, float* d_rbuf, size_t count, float eb) {
  return allreduce_ring_comprs_hom_sum_F_opt(d_sbuf, d_rbuf, count, MPI_COMM_WORLD, eb);
}
int ref_allreduce_gpu(const float* d_sbuf, float* d_rbuf, size_t count) {
  return allreduce_ring_gpu(d_sbuf, d_rbuf, count, MPI_COMM_WORLD);
}
size_t ref_compress(float* d_x, unsigned char* d_out, size_t n, float eb) {
  size_t sz = 0;
  GSZ_compress_deviceptr_outlier(d_x, d_out, n, &sz, eb, 0);
  return sz;
}
void ref_decompress(float* d_x, unsigned char* d_in, size_t n, size_t sz, float eb) {
  GSZ_decompress_deviceptr_outlier(d_x, d_in, n, sz, eb, 0);
}
size_t ref_hom_sum_F(unsigned char* d_in, float* d_local, unsigned char* d_out, size_t n, float eb, size_t in_size) {
  size_t sz = 0;
  homomorphic_sum_F(d_in, d_local, d_out, n, eb, &sz, in_size, 0);
  return sz;
}

}  // extern "C"
