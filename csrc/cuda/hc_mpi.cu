// MPI front door (see homcomp_mpi.h): bootstrap of a hc_comm from an MPI communicator and the
// reference-named collectives with a real MPI_Comm.  Built only with -DHC_WITH_MPI.
#ifdef HC_WITH_MPI
#include "homcomp_mpi.h"

#include <cuda_runtime.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "hc_format.h"

namespace {

struct Entry {
  MPI_Comm mpi;
  hc_comm* comm;
  void* own = nullptr;            // this rank's region (hc_ipc_alloc)
  std::vector<void*> mapped;      // the peers' regions as mapped here
};
std::vector<Entry> g_entries;
std::mutex g_mu;

// MPI_Comm is an int in some MPIs and a pointer in others: compare the bytes
bool same_comm(const MPI_Comm& a, const MPI_Comm& b) { return memcmp(&a, &b, sizeof(MPI_Comm)) == 0; }

Entry* find(MPI_Comm comm) {
  for (auto& e : g_entries)
    if (same_comm(e.mpi, comm)) return &e;
  return nullptr;
}

}  // namespace

int hc_comm_create_mpi(MPI_Comm comm, size_t max_count, hc_comm** out) {
  int rank = 0, size = 1;
  if (MPI_Comm_rank(comm, &rank) != MPI_SUCCESS || MPI_Comm_size(comm, &size) != MPI_SUCCESS) return hc::kErrArgument;
  if (size < 1 || size > 8) return hc::kErrArgument;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (find(comm)) return hc::kErrArgument;  // one handle per communicator
  }
  Entry e;
  e.mpi = comm;
  e.comm = nullptr;
  const size_t bytes = hc_comm_symmetric_bytes(size, max_count);
  unsigned char mine[64];
  if (int rc = hc_ipc_alloc(&e.own, bytes, mine)) return rc;
  std::vector<void*> bases((size_t)size, nullptr);
  bases[(size_t)rank] = e.own;
  int failed = 0;
  // round k: my handle goes k ranks up, the handle of the rank k below comes in
  for (int k = 1; k < size; ++k) {
    const int up = (rank + k) % size, down = (rank - k + size) % size;
    unsigned char theirs[64];
    if (MPI_Sendrecv(mine, 64, MPI_BYTE, up, 0, theirs, 64, MPI_BYTE, down, 0, comm, MPI_STATUS_IGNORE) != MPI_SUCCESS) {
      failed = 1;
      continue;
    }
    void* p = nullptr;
    if (hc_ipc_open(theirs, &p) != 0) failed = 1;
    bases[(size_t)down] = p;
    if (p) e.mapped.push_back(p);
  }
  int rc = failed ? (int)hc::kErrCuda : hc_comm_create(&e.comm, rank, size, max_count, bases.data(), nullptr);
  // every region is zeroed and mapped everywhere before anybody's first store
  if (MPI_Barrier(comm) != MPI_SUCCESS && rc == 0) rc = hc::kErrPeer;
  if (rc != 0) {
    if (e.comm) hc_comm_destroy(e.comm);
    for (void* p : e.mapped) hc_ipc_close(p);
    hc_ipc_free(e.own);
    return rc;
  }
  if (out) *out = e.comm;
  std::lock_guard<std::mutex> lock(g_mu);
  g_entries.push_back(e);
  return hc::kOk;
}

hc_comm* hc_comm_from_mpi(MPI_Comm comm) {
  std::lock_guard<std::mutex> lock(g_mu);
  Entry* e = find(comm);
  return e ? e->comm : nullptr;
}

int hc_comm_free_mpi(MPI_Comm comm) {
  Entry e;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    Entry* f = find(comm);
    if (!f) return hc::kErrArgument;
    e = *f;
    g_entries.erase(g_entries.begin() + (f - g_entries.data()));
  }
  cudaDeviceSynchronize();
  MPI_Barrier(comm);  // nobody may still be storing into a region that is about to go away
  hc_comm_destroy(e.comm);
  for (void* p : e.mapped) hc_ipc_close(p);
  hc_ipc_free(e.own);
  return hc::kOk;
}

// The five compressed variants of the reference differ in host orchestration only; here they are one
// engine (see homcomp_compat.h).  All run on the default stream and return when enqueued.
int allreduce_ring_comprs_hom_sum_F(const float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  hc_comm* c = hc_comm_from_mpi(comm);
  return c ? hc_allreduce(c, s, r, count, eb, 0) : (int)hc::kErrArgument;
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
int mixed_compressed_allreduce(float* s, float* r, size_t count, MPI_Comm comm, float eb) {
  hc_comm* c = hc_comm_from_mpi(comm);
  return c ? hc_allreduce_mixed(c, hc_comm_get_inter(c), s, r, count, eb, 0) : (int)hc::kErrArgument;
}
int allreduce_ring_gpu(const float* s, float* r, size_t count, MPI_Comm comm) {
  hc_comm* c = hc_comm_from_mpi(comm);
  return c ? hc_allreduce_raw(c, s, r, count, 0) : (int)hc::kErrArgument;
}
#endif  // HC_WITH_MPI
