// Reference-named entry points on top of the handle-based engine (see homcomp_compat.h).
#include "homcomp_compat.h"

#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "hc_format.h"

namespace {

struct DeviceState {
  hc_codec* codec = nullptr;
  size_t max_elems = 0;
  uint64_t* d_size = nullptr;
};
DeviceState g_state[64];
std::mutex g_mu;

// one codec handle per device, grown when a larger call comes in (set-up cost, not per call)
DeviceState* state_for(size_t n) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& s = g_state[dev];
  if (!s.codec || s.max_elems < n) {
    if (s.codec) {
      cudaDeviceSynchronize();
      hc_codec_destroy(s.codec);
      s.codec = nullptr;
    }
    size_t want = n < (1u << 20) ? (1u << 20) : n + n / 4;
    if (hc_codec_create(&s.codec, want) != 0) return nullptr;
    s.max_elems = want;
    if (!s.d_size && cudaMalloc(&s.d_size, sizeof(uint64_t)) != cudaSuccess) return nullptr;
  }
  return &s;
}

// What the caller's output buffer is taken to hold (the reference's signatures carry no capacity):
// nbEle * 4 bytes as every caller in the reference allocates (HomComp/src/cuda_awareallreduce.cu:191-194),
// or hc_max_compressed_bytes(nbEle) once the caller has said so.
int g_capacity_rule = 0;
size_t assumed_capacity(size_t n) { return g_capacity_rule == 1 ? hc_max_compressed_bytes(n) : n * sizeof(float); }

void report(const char* what, int rc);

void read_size(DeviceState* s, size_t* cmpSize, cudaStream_t stream) {
  uint64_t v = 0;
  cudaMemcpyAsync(&v, s->d_size, sizeof(v), cudaMemcpyDeviceToHost, stream);
  cudaStreamSynchronize(stream);
  if (cmpSize) *cmpSize = (size_t)v;
}

void compress_mode(int mode, float* d_x, unsigned char* d_out, size_t n, size_t* cmpSize, float eb, cudaStream_t st) {
  DeviceState* s = state_for(n);
  if (!s) return report("compress", hc::kErrCuda);
  cudaMemsetAsync(s->d_size, 0, sizeof(uint64_t), st);  // stays 0 when the stream does not fit
  report("compress", hc_compress(s->codec, d_x, n, eb, mode, d_out, assumed_capacity(n), s->d_size, st));
  read_size(s, cmpSize, st);
  report("compress (device)", hc_codec_status(s->codec, 1));
}

void decompress_mode(int mode, float* d_x, unsigned char* d_in, size_t n, size_t cmpSize, float eb, cudaStream_t st) {
  DeviceState* s = state_for(n);
  if (!s) return report("decompress", hc::kErrCuda);
  report("decompress", hc_decompress(s->codec, d_in, cmpSize, n, eb, mode, d_x, st));
}

}  // namespace

int hc_compat_last_status = 0;
namespace {
void report(const char* what, int rc) {
  if (rc) {
    hc_compat_last_status = rc;
    fprintf(stderr, "homcomp: %s failed: %s\n", what, hc_status_string(rc));
  }
}
}  // namespace
void hc_compat_set_capacity_rule(int rule) { g_capacity_rule = rule == 1 ? 1 : 0; }

void GSZ_compress_deviceptr_plain(float* d, unsigned char* c, size_t n, size_t* sz, float eb, cudaStream_t st) {
  compress_mode(hc::kModePlain, d, c, n, sz, eb, st);
}
void GSZ_decompress_deviceptr_plain(float* d, unsigned char* c, size_t n, size_t sz, float eb, cudaStream_t st) {
  decompress_mode(hc::kModePlain, d, c, n, sz, eb, st);
}
void GSZ_compress_deviceptr_outlier(float* d, unsigned char* c, size_t n, size_t* sz, float eb, cudaStream_t st) {
  compress_mode(hc::kModeOutlier, d, c, n, sz, eb, st);
}
void GSZ_decompress_deviceptr_outlier(float* d, unsigned char* c, size_t n, size_t sz, float eb, cudaStream_t st) {
  decompress_mode(hc::kModeOutlier, d, c, n, sz, eb, st);
}
void GSZ_compress_deviceptr_outlier_vec(float* d, unsigned char* c, size_t n, size_t* sz, float eb, cudaStream_t st) {
  compress_mode(hc::kModeVec, d, c, n, sz, eb, st);
}
void GSZ_decompress_deviceptr_outlier_vec(float* d, unsigned char* c, size_t n, size_t sz, float eb, cudaStream_t st) {
  decompress_mode(hc::kModeVec, d, c, n, sz, eb, st);
}

// host-pointer variants use the plain codec, as in the reference (HomComp/src/GSZ_entry.cu:28-148)
void GSZ_compress_hostptr(float* oriData, unsigned char* cmpBytes, size_t nbEle, size_t* cmpSize, float errorBound) {
  float* d_x = nullptr;
  unsigned char* d_c = nullptr;
  const size_t cap = hc_max_compressed_bytes(nbEle);
  if (cudaMalloc(&d_x, nbEle * sizeof(float)) != cudaSuccess || cudaMalloc(&d_c, cap) != cudaSuccess) {
    cudaFree(d_x);
    return report("compress_hostptr", hc::kErrCuda);
  }
  cudaMemcpy(d_x, oriData, nbEle * sizeof(float), cudaMemcpyHostToDevice);
  size_t sz = 0;
  compress_mode(hc::kModePlain, d_x, d_c, nbEle, &sz, errorBound, 0);
  if (sz > assumed_capacity(nbEle)) sz = 0;  // never more than the caller's buffer is taken to hold
  cudaMemcpy(cmpBytes, d_c, sz, cudaMemcpyDeviceToHost);
  if (cmpSize) *cmpSize = sz;
  cudaFree(d_x);
  cudaFree(d_c);
}
void GSZ_decompress_hostptr(float* decData, unsigned char* cmpBytes, size_t nbEle, size_t cmpSize, float errorBound) {
  float* d_x = nullptr;
  unsigned char* d_c = nullptr;
  if (cudaMalloc(&d_x, nbEle * sizeof(float)) != cudaSuccess || cudaMalloc(&d_c, cmpSize + 16) != cudaSuccess) {
    cudaFree(d_x);
    return report("decompress_hostptr", hc::kErrCuda);
  }
  cudaMemcpy(d_c, cmpBytes, cmpSize, cudaMemcpyHostToDevice);
  decompress_mode(hc::kModePlain, d_x, d_c, nbEle, cmpSize, errorBound, 0);
  cudaMemcpy(decData, d_x, nbEle * sizeof(float), cudaMemcpyDeviceToHost);
  cudaFree(d_x);
  cudaFree(d_c);
}

void homomorphic_sum(unsigned char* d_in, int* d_deltas, unsigned char* d_out, size_t n, float eb, size_t* cmpSize,
                     size_t in_size, cudaStream_t st) {
  (void)eb;
  DeviceState* s = state_for(n);
  if (!s) return report("homomorphic_sum", hc::kErrCuda);
  cudaMemsetAsync(s->d_size, 0, sizeof(uint64_t), st);
  report("homomorphic_sum", hc_hom_add_i32(s->codec, d_in, in_size, d_deltas, n, hc::kModeOutlier, d_out,
                                           assumed_capacity(n), s->d_size, st));
  read_size(s, cmpSize, st);
  report("homomorphic_sum (device)", hc_codec_status(s->codec, 1));
}
void homomorphic_sum_F(unsigned char* d_in, float* d_local, unsigned char* d_out, size_t n, float eb, size_t* cmpSize,
                       size_t in_size, cudaStream_t st) {
  DeviceState* s = state_for(n);
  if (!s) return report("homomorphic_sum_F", hc::kErrCuda);
  cudaMemsetAsync(s->d_size, 0, sizeof(uint64_t), st);
  report("homomorphic_sum_F", hc_hom_add_f32(s->codec, d_in, in_size, d_local, n, eb, hc::kModeOutlier, d_out,
                                             assumed_capacity(n), s->d_size, st));
  read_size(s, cmpSize, st);
  report("homomorphic_sum_F (device)", hc_codec_status(s->codec, 1));
}
void quant_prediction(const float* d_x, int* d_deltas, float eb, size_t n, cudaStream_t st) {
  report("quant_prediction", hc_quant_pred(d_x, n, eb, hc::kModeOutlier, d_deltas, st));
}

// The five compressed ring variants of the reference differ only in host orchestration (two
// kernels or one per hop, even or uneven chunks, scratch per call or hoisted); here they are one
// fused, allocation-free engine.  They run on the default stream and return when enqueued.
int allreduce_ring_comprs_hom_sum_F(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return hc_allreduce(comm, s, r, count, eb, 0);
}
int allreduce_ring_comprs_hom_sum(const float* s, float* r, size_t c, MPI_Comm comm, float eb) {
  return allreduce_ring_comprs_hom_sum_F(s, r, c, comm, eb);
}
int allreduce_ring_comprs_hom_sum_seg(const float* s, float* r, size_t c, MPI_Comm comm, float eb) {
  return allreduce_ring_comprs_hom_sum_F(s, r, c, comm, eb);
}
int allreduce_ring_comprs_hom_sum_F_seg(const float* s, float* r, size_t c, MPI_Comm comm, float eb) {
  return allreduce_ring_comprs_hom_sum_F(s, r, c, comm, eb);
}
int allreduce_ring_comprs_hom_sum_F_opt(const float* s, float* r, size_t c, MPI_Comm comm, float eb) {
  return allreduce_ring_comprs_hom_sum_F(s, r, c, comm, eb);
}
// Hierarchical allreduce: `comm` spans the ranks of one group (the reference takes the ranks that share
// a node, HomComp/src/cuda_awareallreduce.cu:678-683); the communicator of the ranks with the same
// local index in the other groups is attached to it with hc_comm_set_inter.  Raw fp32 reduce-scatter
// inside the group, compressed allreduce (error bound eb) of this rank's slice between the groups, raw
// all-gather inside the group.  Without an attached communicator there is one group and nothing is
// compressed, as in the reference when every rank shares a node.
int mixed_compressed_allreduce(float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return hc_allreduce_mixed(comm, hc_comm_get_inter(comm), s, r, count, eb, 0);
}
int allreduce_ring_gpu(const float* s, float* r, size_t count, MPI_Comm comm) { return hc_allreduce_raw(comm, s, r, count, 0); }

int cpuCopy_allreduce_ring_comprs_hom_sum_F(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return hc_comm_allreduce_host_staged(comm, s, r, count, eb, 0);
}
int cpuCopy_allreduce_ring_comprs_hom_sum(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return cpuCopy_allreduce_ring_comprs_hom_sum_F(s, r, count, comm, eb);
}
int cpuCopy_allreduce_ring_comprs_hom_sum_seg(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return cpuCopy_allreduce_ring_comprs_hom_sum_F(s, r, count, comm, eb);
}
int cpuCopy_allreduce_ring_comprs_hom_sum_F_seg(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  return cpuCopy_allreduce_ring_comprs_hom_sum_F(s, r, count, comm, eb);
}

float* read_binary_floats(const char* filename, size_t* out_size) {
  if (out_size) *out_size = 0;
  FILE* f = fopen(filename, "rb");
  if (!f) return nullptr;
  if (fseek(f, 0, SEEK_END) != 0) { fclose(f); return nullptr; }
  long bytes = ftell(f);
  rewind(f);
  if (bytes < 0) { fclose(f); return nullptr; }
  size_t n = (size_t)bytes / sizeof(float);
  float* data = static_cast<float*>(malloc(n ? n * sizeof(float) : sizeof(float)));
  if (!data) { fclose(f); return nullptr; }
  size_t got = fread(data, sizeof(float), n, f);
  fclose(f);
  if (got != n) { free(data); return nullptr; }
  if (out_size) *out_size = n;
  return data;
}
