// Host-staged compressed ring allreduce: for GPUs that cannot address each other.
//
// The codec and the fused homomorphic add run on the device; every compressed chunk is copied to
// pinned host memory, handed to a caller-supplied transport (send / receive of byte messages:
// sockets, MPI, shared memory, a queue between threads) and copied back up on the other side.
// Counterpart of the reference's non-CUDA-aware variants (cpuCopy_allreduce_ring_comprs_hom_sum*,
// HomComp/src/nca_allreduce.cu:195-324), which do the same around MPI_Send / MPI_Recv.  Partition,
// hop order and arithmetic are those of the device ring and of hc_cpu_ring_allreduce, so the three
// produce the same bits.  Like the reference's version it synchronises the host once per hop (the
// message length has to be known on the host); unlike it, the bounce buffers (two device, three
// pinned) are kept per codec handle between calls and only grow.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <map>
#include <mutex>

#include "hc_format.h"
#include "homcomp_b200.h"

namespace {

struct Buffers {
  uint8_t* d_in = nullptr;   // incoming stream on the device
  uint8_t* d_out = nullptr;  // stream produced by the current hop
  uint64_t* d_size = nullptr;
  uint8_t* h_out = nullptr;  // pinned: what this rank sends
  uint8_t* h_in = nullptr;   // pinned: what this rank receives
  uint64_t* h_size = nullptr;
  size_t cap = 0;
  ~Buffers() {
    if (d_in) cudaFree(d_in);
    if (d_out) cudaFree(d_out);
    if (d_size) cudaFree(d_size);
    if (h_out) cudaFreeHost(h_out);
    if (h_in) cudaFreeHost(h_in);
    if (h_size) cudaFreeHost(h_size);
  }
};

// bounce buffers of every codec handle that has used this path; released by hc_codec_destroy
std::map<const hc_codec*, Buffers*> g_buffers;
std::mutex g_buffers_mu;

Buffers* buffers_for(const hc_codec* codec, size_t cap) {
  std::lock_guard<std::mutex> lock(g_buffers_mu);
  Buffers*& b = g_buffers[codec];
  if (b && b->cap >= cap) return b;
  if (b) {
    cudaDeviceSynchronize();
    delete b;
    b = nullptr;
  }
  Buffers* n = new Buffers();
  if (cudaMalloc(&n->d_in, cap) != cudaSuccess || cudaMalloc(&n->d_out, cap) != cudaSuccess ||
      cudaMalloc(&n->d_size, sizeof(uint64_t)) != cudaSuccess || cudaMallocHost(&n->h_out, cap) != cudaSuccess ||
      cudaMallocHost(&n->h_in, cap) != cudaSuccess || cudaMallocHost(&n->h_size, sizeof(uint64_t)) != cudaSuccess) {
    delete n;
    g_buffers.erase(codec);
    return nullptr;
  }
  n->cap = cap;
  b = n;
  return b;
}

}  // namespace

// called by hc_codec_destroy
void hc_host_staged_release(const hc_codec* codec) {
  std::lock_guard<std::mutex> lock(g_buffers_mu);
  auto it = g_buffers.find(codec);
  if (it == g_buffers.end()) return;
  delete it->second;
  g_buffers.erase(it);
}

extern "C" int hc_allreduce_host_staged(hc_codec* codec, const hc_host_transport* t, int rank, int world,
                                        const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
  if (!codec || !t || !t->send || !t->recv || world < 1 || rank < 0 || rank >= world || !d_sbuf || !d_rbuf ||
      !(eb > 0.0f))
    return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  const int P = world, r = rank;
  const size_t B = hc_chunk_elems(count, P);
  auto chunk_len = [&](int c) -> size_t {
    const size_t lo = (size_t)c * B;
    if (lo >= count) return 0;
    const size_t hi = lo + B;
    return (hi > count ? count : hi) - lo;
  };
  const size_t cap = hc_max_compressed_bytes(B) + 64;  // + what a bulk copy may read past the end
  Buffers* kept = buffers_for(codec, cap);  // allocated on the handle's first call (or when a larger one comes)
  if (!kept) return hc::kErrCuda;
  Buffers& b = *kept;
  if (cudaMemsetAsync(b.d_in, 0, cap, stream) != cudaSuccess) return hc::kErrCuda;
  const int next = (r + 1) % P, prev = (r - 1 + P) % P;

  // device stream -> pinned host bytes; returns the stream length (the one host sync of a hop)
  auto bring_down = [&](size_t* bytes) -> int {
    if (cudaMemcpyAsync(b.h_size, b.d_size, sizeof(uint64_t), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
      return hc::kErrCuda;
    *bytes = (size_t)*b.h_size;
    if (*bytes > cap) return hc::kErrCapacity;
    if (*bytes && (cudaMemcpyAsync(b.h_out, b.d_out, *bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                   cudaStreamSynchronize(stream) != cudaSuccess))
      return hc::kErrCuda;
    return hc::kOk;
  };
  // even ranks send first, odd ranks receive first: no deadlock with a blocking transport
  auto exchange = [&](size_t out_bytes, size_t* in_bytes) -> int {
    *in_bytes = 0;
    if (P == 1) return hc::kOk;
    int rc;
    if (r % 2 == 0) {
      if ((rc = t->send(t->user, next, b.h_out, out_bytes)) != 0) return hc::kErrPeer;
      if ((rc = t->recv(t->user, prev, b.h_in, cap, in_bytes)) != 0) return hc::kErrPeer;
    } else {
      if ((rc = t->recv(t->user, prev, b.h_in, cap, in_bytes)) != 0) return hc::kErrPeer;
      if ((rc = t->send(t->user, next, b.h_out, out_bytes)) != 0) return hc::kErrPeer;
    }
    if (*in_bytes > cap) return hc::kErrCapacity;
    return hc::kOk;
  };
  auto bring_up = [&](size_t bytes) -> int {
    if (bytes && cudaMemcpyAsync(b.d_in, b.h_in, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return hc::kErrCuda;
    return hc::kOk;
  };

  int rc;
  size_t held = 0;  // bytes in h_out
  // ---- reduce-scatter ----------------------------------------------------------------------------
  if (size_t n = chunk_len(r)) {
    if ((rc = hc_compress(codec, d_sbuf + (size_t)r * B, n, eb, 0, b.d_out, cap, b.d_size, stream)) != hc::kOk) return rc;
    if ((rc = bring_down(&held)) != hc::kOk) return rc;
  }
  for (int s = 1; s < P; ++s) {
    size_t got = 0;
    if ((rc = exchange(held, &got)) != hc::kOk) return rc;
    const int c = ((r - s) % P + P) % P;
    const size_t n = chunk_len(c);
    held = 0;
    if (n == 0) continue;
    if ((rc = bring_up(got)) != hc::kOk) return rc;
    rc = got ? hc_hom_add_f32(codec, b.d_in, got, d_sbuf + (size_t)c * B, n, eb, 0, b.d_out, cap, b.d_size, stream)
             : hc_compress(codec, d_sbuf + (size_t)c * B, n, eb, 0, b.d_out, cap, b.d_size, stream);
    if (rc != hc::kOk) return rc;
    if ((rc = bring_down(&held)) != hc::kOk) return rc;
  }
  // ---- all-gather: rank r holds the reduced stream of chunk (r + 1) mod P ------------------------
  int held_c = (r + 1) % P;
  for (int s = 0; s < P; ++s) {
    // decode what is held (it is in h_out after a hop of the reduce-scatter, in h_in afterwards)
    const size_t n = chunk_len(held_c);
    if (n && held) {
      const uint8_t* src = s == 0 ? b.h_out : b.h_in;
      if (cudaMemcpyAsync(b.d_in, src, held, cudaMemcpyHostToDevice, stream) != cudaSuccess) return hc::kErrCuda;
      if ((rc = hc_decompress(codec, b.d_in, held, n, eb, 0, d_rbuf + (size_t)held_c * B, stream)) != hc::kOk) return rc;
    }
    if (s == P - 1) break;
    // pass it on; the bytes to send must sit in h_out
    if (s > 0 && held) {
      if (cudaStreamSynchronize(stream) != cudaSuccess) return hc::kErrCuda;  // the upload above reads h_in
      memcpy(b.h_out, b.h_in, held);
    }
    size_t got = 0;
    if (s == 0 && cudaStreamSynchronize(stream) != cudaSuccess) return hc::kErrCuda;
    if ((rc = exchange(held, &got)) != hc::kOk) return rc;
    held = got;
    held_c = (held_c - 1 + P) % P;
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return hc::kErrCuda;
  return hc_codec_status(codec, 0);
}
