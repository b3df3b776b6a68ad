// The reference library's C++ entry points by name, as thin calls into the handle-based engine
// (signatures of HomComp/include/GSZ_entry.h:4-37, homcomp.cuh:2-5, cuda_awareallreduce.cuh:4-17,
// nca_allreduce.cuh:3-15, readFile.h:4).
//
// Differences a caller can see:
//   * *cmpSize is the exact stream length (the reference adds one byte per block);
//   * functions that return a size through a host pointer synchronise the stream, as they did;
//   * scratch memory is kept per device between calls instead of cudaMalloc / cudaFree per call;
//   * `MPI_Comm` is this library's communicator handle unless <mpi.h> was included first: no MPI
//     is needed, ranks are bootstrapped with hc_comm_create (any host channel for the handles);
//   * errors come back as a non-zero status instead of exit() / MPI_Abort(); the void functions print
//     a line to stderr and leave the code in hc_compat_last_status.
//
// Output buffers.  The signatures carry no capacity, so it is assumed.  By default a compressed
// output buffer (d_cmpBytes, d_cmpByteOut, cmpBytes) is taken to hold nbEle * 4 bytes, which is
// what every caller in the reference allocates; a stream that would not fit (incompressible
// data needs up to 129 bytes per 128) is cut off at that size, status 1 is reported, *cmpSize is 0,
// and nothing is written past nbEle * 4 bytes.  A caller that allocates
// hc_max_compressed_bytes(nbEle) bytes, which always suffices, says so once with
// hc_compat_set_capacity_rule(1).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "homcomp_b200.h"

#ifndef MPI_VERSION
typedef hc_comm* MPI_Comm;
#define HC_COMPAT_OWN_MPI_COMM 1
#endif

// 0 (default): output buffers hold nbEle * 4 bytes; 1: they hold hc_max_compressed_bytes(nbEle)
void hc_compat_set_capacity_rule(int rule);
extern int hc_compat_last_status;  // last non-zero status of a void entry point (0: none so far)

void GSZ_compress_hostptr(float* oriData, unsigned char* cmpBytes, size_t nbEle, size_t* cmpSize, float errorBound);
void GSZ_decompress_hostptr(float* decData, unsigned char* cmpBytes, size_t nbEle, size_t cmpSize, float errorBound);
void GSZ_compress_deviceptr_plain(float* d_oriData, unsigned char* d_cmpBytes, size_t nbEle, size_t* cmpSize,
                                  float errorBound, cudaStream_t stream = 0);
void GSZ_decompress_deviceptr_plain(float* d_decData, unsigned char* d_cmpBytes, size_t nbEle, size_t cmpSize,
                                    float errorBound, cudaStream_t stream = 0);
void GSZ_compress_deviceptr_outlier(float* d_oriData, unsigned char* d_cmpBytes, size_t nbEle, size_t* cmpSize,
                                    float errorBound, cudaStream_t stream = 0);
void GSZ_decompress_deviceptr_outlier(float* d_decData, unsigned char* d_cmpBytes, size_t nbEle, size_t cmpSize,
                                      float errorBound, cudaStream_t stream = 0);
void GSZ_compress_deviceptr_outlier_vec(float* d_oriData, unsigned char* d_cmpBytes, size_t nbEle, size_t* cmpSize,
                                        float errorBound, cudaStream_t stream = 0);
void GSZ_decompress_deviceptr_outlier_vec(float* d_decData, unsigned char* d_cmpBytes, size_t nbEle, size_t cmpSize,
                                          float errorBound, cudaStream_t stream = 0);
// d_quantPredLoc: output of quant_prediction (whole 32-element blocks)
void homomorphic_sum(unsigned char* d_cmpBytesIn, int* d_quantPredLoc, unsigned char* d_cmpByteOut, size_t nbEle,
                     float errorBound, size_t* cmpSize, size_t cmpSizeCmpBlock, cudaStream_t stream = 0);
void homomorphic_sum_F(unsigned char* d_cmpBytesIn, float* d_localChunk, unsigned char* d_cmpByteOut, size_t nbEle,
                       float errorBound, size_t* cmpSize, size_t cmpSizeCmpBlock, cudaStream_t stream = 0);
// host launcher of the quantise + predict kernel (the reference exposes the __global__ function
// kernel_quant_prediction itself)
void quant_prediction(const float* d_localData, int* d_quantPredData, float errorBound, size_t nbEle,
                      cudaStream_t stream = 0);

#ifdef HC_COMPAT_OWN_MPI_COMM
int allreduce_ring_comprs_hom_sum(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_comprs_hom_sum_F_opt(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int mixed_compressed_allreduce(float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int allreduce_ring_gpu(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm);
// host-staged variants (HomComp/include/nca_allreduce.cuh:3-15): one engine, see
// hc_allreduce_host_staged; the communicator needs a transport (hc_comm_set_host_transport)
int cpuCopy_allreduce_ring_comprs_hom_sum(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int cpuCopy_allreduce_ring_comprs_hom_sum_F(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int cpuCopy_allreduce_ring_comprs_hom_sum_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm, float eb);
int cpuCopy_allreduce_ring_comprs_hom_sum_F_seg(const float* d_sbuf, float* d_rbuf, size_t count, MPI_Comm comm,
                                                float eb);
#endif

// whole-file read of raw float32 values into malloc'd memory (caller frees)
float* read_binary_floats(const char* filename, size_t* out_size);
