// Multi-GPU allreduce driver without Python, MPI or NCCL: one host thread per GPU of this machine,
// peer access between all of them, the reference-named collective API (homcomp_compat.h).  Every
// rank holds the same data, so the expected result is world * input; the check is the
// reference checker's rule |world * in - out| <= 2 eb (world + world / 10)
// (HomComp/src/utils/checksmooth.c:50-51).  Prints device-timed latency per mode: compressed over
// peer memory, uncompressed, host-staged (cpuCopy_* names) with mailboxes between the threads
// standing in for the host network, and, for an even number of GPUs, the hierarchical form
// (mixed_compressed_allreduce) with the GPUs split into two groups: raw inside a group, compressed
// between the two.
//
// With `nvls` as the fifth argument the symmetric regions come from hc_mc_create_local (driver virtual
// memory API + multicast object) instead of cudaMalloc + peer access: the reduced chunks then leave
// with one multimem.st for all GPUs and the uncompressed sum is formed inside the switch.  The line
// ends with a checksum of rank 0's compressed-allreduce result, which must not depend on the transport.
//
//   allreduce_threads [gpus] [count] [eb] [iterations] [ipc|nvls]
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <string.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "homcomp_compat.h"

struct Barrier {
  std::atomic<int> count{0}, sense{0};
  int n;
  explicit Barrier(int n_) : n(n_) {}
  void wait(int& local) {
    local ^= 1;
    if (count.fetch_add(1) == n - 1) {
      count.store(0);
      sense.store(local);
    } else {
      while (sense.load() != local) std::this_thread::yield();
    }
  }
};

// one mailbox per (source, destination) pair: the "host network" of the host-staged mode
struct Mailbox {
  std::mutex m;
  std::condition_variable cv;
  std::deque<std::vector<unsigned char>> q;
};
struct Net {
  int P, rank;
  std::vector<Mailbox>* boxes;  // [src * P + dst]
};
static int net_send(void* user, int dst, const void* buf, size_t bytes) {
  Net* n = static_cast<Net*>(user);
  Mailbox& b = (*n->boxes)[(size_t)n->rank * n->P + dst];
  std::vector<unsigned char> msg(bytes);
  if (bytes) memcpy(msg.data(), buf, bytes);
  {
    std::lock_guard<std::mutex> g(b.m);
    b.q.push_back(std::move(msg));
  }
  b.cv.notify_one();
  return 0;
}
static int net_recv(void* user, int src, void* buf, size_t cap, size_t* bytes) {
  Net* n = static_cast<Net*>(user);
  Mailbox& b = (*n->boxes)[(size_t)src * n->P + n->rank];
  std::unique_lock<std::mutex> g(b.m);
  if (!b.cv.wait_for(g, std::chrono::seconds(20), [&] { return !b.q.empty(); })) return 1;  // the peer never sent
  std::vector<unsigned char> msg = std::move(b.q.front());
  b.q.pop_front();
  if (msg.size() > cap) return 2;
  if (!msg.empty()) memcpy(buf, msg.data(), msg.size());
  *bytes = msg.size();
  return 0;
}

int main(int argc, char** argv) {
  int ndev = 0;
  cudaGetDeviceCount(&ndev);
  int P = argc > 1 ? atoi(argv[1]) : ndev;
  const size_t count = argc > 2 ? (size_t)atoll(argv[2]) : (size_t)1 << 22;
  const float eb = argc > 3 ? (float)atof(argv[3]) : 1e-4f;
  const int iters = argc > 4 ? atoi(argv[4]) : 10;
  const bool nvls = argc > 5 && strcmp(argv[5], "nvls") == 0;
  if (P < 1 || P > ndev || P > 8) {
    fprintf(stderr, "need 1..%d GPUs\n", ndev < 8 ? ndev : 8);
    return 2;
  }
  std::vector<float> host(count);
  for (size_t i = 0; i < count; ++i) host[i] = (float)(sin(i * 3e-5) + 0.1 * sin(i * 7e-3));
  const size_t sym = hc_comm_symmetric_bytes(P, count);
  std::vector<void*> region(P, nullptr);
  std::vector<int> failures(P, 0);
  std::vector<float> lat_c(P, 0), lat_r(P, 0), lat_h(P, 0), lat_m(P, 0);
  // hierarchical mode: two groups of P / 2 ranks; rank r is local rank r % L of group r / L
  const bool mixed = P >= 2 && P % 2 == 0;
  const int L = mixed ? P / 2 : P;
  const size_t slice = hc_chunk_elems(count, L);
  const size_t sym_local = hc_comm_symmetric_bytes(L, count), sym_inter = hc_comm_symmetric_bytes(2, slice);
  std::vector<void*> region_local(P, nullptr), region_inter(P, nullptr);
  std::vector<Mailbox> boxes((size_t)P * P);
  Barrier bar(P);
  unsigned long long checksum = 0;
  hc_mc_region* mc_region = nullptr;
  void* mc_base = nullptr;
  if (nvls) {
    std::vector<int> devs(P);
    for (int r = 0; r < P; ++r) devs[r] = r;
    if (hc_mc_create_local(&mc_region, P, devs.data(), sym) != 0) {
      fprintf(stderr, "hc_mc_create_local failed\n");
      return 2;
    }
    for (int r = 0; r < P; ++r) region[r] = hc_mc_unicast_ptr(mc_region, r);
    mc_base = hc_mc_multicast_ptr(mc_region);
  }
  auto worker = [&](int r) {
    int sense = 0;
    cudaSetDevice(r);
    for (int q = 0; q < P; ++q)
      if (q != r) cudaDeviceEnablePeerAccess(q, 0);
    if (!nvls) {
      cudaMalloc(&region[r], sym);
      cudaMemset(region[r], 0, sym);
    }
    if (mixed) {
      cudaMalloc(&region_local[r], sym_local);
      cudaMemset(region_local[r], 0, sym_local);
      cudaMalloc(&region_inter[r], sym_inter);
      cudaMemset(region_inter[r], 0, sym_inter);
    }
    cudaDeviceSynchronize();
    bar.wait(sense);
    hc_comm* comm = nullptr;
    if (hc_comm_create(&comm, r, P, count, region.data(), mc_base) != 0) { failures[r] = 1; return; }
    hc_comm *local = nullptr, *inter = nullptr;
    if (mixed) {
      const int g = r / L, l = r % L;
      std::vector<void*> lb(L), ib(2);
      for (int q = 0; q < L; ++q) lb[q] = region_local[g * L + q];
      for (int q = 0; q < 2; ++q) ib[q] = region_inter[q * L + l];
      if (hc_comm_create(&local, l, L, count, lb.data(), nullptr) != 0 ||
          hc_comm_create(&inter, g, 2, slice, ib.data(), nullptr) != 0 || hc_comm_set_inter(local, inter) != 0) {
        failures[r] = 1;
        return;
      }
    }
    Net net{P, r, &boxes};
    hc_host_transport tp{net_send, net_recv, &net};
    if (hc_comm_set_host_transport(comm, &tp) != 0) failures[r] = 1;
    float *d_in, *d_out;
    cudaMalloc(&d_in, count * 4);
    cudaMalloc(&d_out, count * 4);
    cudaMemcpy(d_in, host.data(), count * 4, cudaMemcpyHostToDevice);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    std::vector<float> out(count);
    for (int mode = 0; mode < (mixed ? 4 : 3); ++mode) {
      float total = 0, ms;
      for (int it = 0; it < iters + 2; ++it) {
        bar.wait(sense);
        cudaEventRecord(e0);
        int rc = mode == 0   ? allreduce_ring_comprs_hom_sum_F(d_in, d_out, count, comm, eb)
                 : mode == 1 ? allreduce_ring_gpu(d_in, d_out, count, comm)
                 : mode == 2 ? cpuCopy_allreduce_ring_comprs_hom_sum_F(d_in, d_out, count, comm, eb)
                             : mixed_compressed_allreduce(d_in, d_out, count, local, eb);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&ms, e0, e1);
        if (rc) failures[r] = 1;
        if (it >= 2) total += ms;
      }
      (mode == 0 ? lat_c : mode == 1 ? lat_r : mode == 2 ? lat_h : lat_m)[r] = total / iters;
      cudaMemcpy(out.data(), d_out, count * 4, cudaMemcpyDeviceToHost);
      const double tol = mode != 1 ? 2.0 * eb * (P + P / 10.0) : 1e-5 * P;
      size_t bad = 0;
      for (size_t i = 0; i < count; ++i)
        if (fabs((double)host[i] * P - out[i]) > tol) ++bad;
      if (bad || hc_comm_status(comm, 1) != 0) failures[r] = 1;
      if (mode == 3 && (hc_comm_status(local, 1) != 0 || hc_comm_status(inter, 1) != 0)) failures[r] = 1;
      if (bad) fprintf(stderr, "rank %d mode %d: %zu values out of tolerance\n", r, mode, bad);
      if (r == 0 && mode == 0) {  // FNV-1a over the result bytes
        unsigned long long h = 1469598103934665603ull;
        const unsigned char* b = reinterpret_cast<const unsigned char*>(out.data());
        for (size_t i = 0; i < count * 4; ++i) h = (h ^ b[i]) * 1099511628211ull;
        checksum = h;
      }
    }
    bar.wait(sense);
    hc_comm_destroy(comm);
    if (local) hc_comm_destroy(local);
    if (inter) hc_comm_destroy(inter);
    cudaFree(d_in);
    cudaFree(d_out);
    bar.wait(sense);
    if (!nvls) cudaFree(region[r]);
    if (mixed) {
      cudaFree(region_local[r]);
      cudaFree(region_inter[r]);
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back(worker, r);
  for (auto& t : th) t.join();
  if (mc_region) hc_mc_destroy(mc_region);
  float mc = 0, mr = 0, mh = 0, mm = 0;
  int fail = 0;
  for (int r = 0; r < P; ++r) {
    mc = lat_c[r] > mc ? lat_c[r] : mc;
    mr = lat_r[r] > mr ? lat_r[r] : mr;
    mh = lat_h[r] > mh ? lat_h[r] : mh;
    mm = lat_m[r] > mm ? lat_m[r] : mm;
    fail |= failures[r];
  }
  printf("gpus %d count %zu eb %g | compressed allreduce %.3f ms (%.1f GB/s) | uncompressed %.3f ms (%.1f GB/s) | "
         "host-staged %.3f ms | hierarchical (2 groups of %d) %.3f ms | transport %s | checksum %016llx | %s\n",
         P, count, eb, mc, 4e-6 * count / mc, mr, 4e-6 * count / mr, mh, mixed ? L : 0, mm,
         nvls ? (mc_base ? "nvls (multicast)" : "nvls asked, no multicast support: peer stores") : "ipc", checksum,
         fail ? "FAILED" : "ok");
  return fail;
}
