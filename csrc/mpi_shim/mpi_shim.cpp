// Single-host MPI shim (see mpi.h).  Host-side control through a POSIX shared-memory segment,
// payloads through device mailboxes mapped into every rank with CUDA IPC.
#include "mpi.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>

namespace {

constexpr int kMaxRanks = 16;
constexpr int kSlots = 2;

struct Channel {  // one per ordered pair (src, dst)
  std::atomic<unsigned long long> sent;   // messages published by src
  std::atomic<unsigned long long> taken;  // messages consumed by dst
  long long nbytes[kSlots];
  char pad[24];
};

struct Shared {
  std::atomic<int> ready;
  std::atomic<int> attached;
  std::atomic<int> barrier_count;
  std::atomic<int> barrier_sense;
  cudaIpcMemHandle_t mailbox[kMaxRanks];
  std::atomic<int> mailbox_ready[kMaxRanks];
  Channel chan[kMaxRanks][kMaxRanks];
};

struct State {
  bool up = false;
  int rank = 0, size = 1;
  size_t slot_bytes = 0;
  Shared* sh = nullptr;
  char shm_name[64];
  unsigned char* my_box = nullptr;            // kMaxRanks destinations x kSlots slots
  unsigned char* peer_box[kMaxRanks] = {};    // other ranks' mailboxes
  int local_sense = 0;
} g;

unsigned char* out_slot(int dst, unsigned long long seq) {
  return g.my_box + ((size_t)dst * kSlots + (seq % kSlots)) * g.slot_bytes;
}
const unsigned char* in_slot(int src, unsigned long long seq) {
  return g.peer_box[src] + ((size_t)g.rank * kSlots + (seq % kSlots)) * g.slot_bytes;
}

void fail(const char* what) {
  fprintf(stderr, "[mpi shim rank %d] %s\n", g.rank, what);
  fflush(stderr);
  _exit(3);
}

void spin_until(std::atomic<unsigned long long>& v, unsigned long long want_at_least) {
  const double t0 = MPI_Wtime();
  unsigned long spins = 0;
  while (v.load(std::memory_order_acquire) < want_at_least) {
    if ((++spins & 1023) == 0) {
      sched_yield();
      if (MPI_Wtime() - t0 > 120.0) fail("timed out waiting for a peer");
    }
  }
}

int type_bytes(MPI_Datatype dt) { return dt == MPI_BYTE ? 1 : (dt == MPI_DOUBLE ? 8 : 4); }

}  // namespace

struct hcref_request {
  int kind;  // 0 recv, 1 send (already complete)
  void* buf;
  long long cap;
  int peer;
};

extern "C" {

double MPI_Wtime(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

int MPI_Init(int*, char***) {
  if (g.up) return MPI_SUCCESS;
  const char* r = getenv("RANK");
  const char* w = getenv("WORLD_SIZE");
  const char* port = getenv("MASTER_PORT");
  g.rank = r ? atoi(r) : 0;
  g.size = w ? atoi(w) : 1;
  if (g.size > kMaxRanks) fail("too many ranks");
  const char* sb = getenv("HCREF_SLOT_BYTES");
  g.slot_bytes = sb ? (size_t)atoll(sb) : ((size_t)96 << 20);
  snprintf(g.shm_name, sizeof(g.shm_name), "/hcref_%s_%d", port ? port : "0", (int)getuid());
  int fd = -1;
  if (g.rank == 0) {
    shm_unlink(g.shm_name);
    fd = shm_open(g.shm_name, O_CREAT | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, sizeof(Shared)) != 0) fail("shm_open/ftruncate");
  } else {
    const double t0 = MPI_Wtime();
    while ((fd = shm_open(g.shm_name, O_RDWR, 0600)) < 0) {
      usleep(2000);
      if (MPI_Wtime() - t0 > 120.0) fail("shm segment never appeared");
    }
    struct stat st;
    while (fstat(fd, &st) == 0 && (size_t)st.st_size < sizeof(Shared)) usleep(2000);
  }
  g.sh = (Shared*)mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (g.sh == MAP_FAILED) fail("mmap");
  if (g.rank == 0) {
    memset((void*)g.sh, 0, sizeof(Shared));
    g.sh->ready.store(1, std::memory_order_release);
  } else {
    while (g.sh->ready.load(std::memory_order_acquire) != 1) usleep(1000);
  }
  if (g.size > 1) {
    const size_t bytes = g.slot_bytes * kSlots * (size_t)g.size;
    if (cudaMalloc((void**)&g.my_box, bytes) != cudaSuccess) fail("cudaMalloc mailbox");
    if (cudaIpcGetMemHandle(&g.sh->mailbox[g.rank], g.my_box) != cudaSuccess) fail("cudaIpcGetMemHandle");
    g.sh->mailbox_ready[g.rank].store(1, std::memory_order_release);
    for (int p = 0; p < g.size; ++p) {
      if (p == g.rank) continue;
      while (g.sh->mailbox_ready[p].load(std::memory_order_acquire) != 1) usleep(1000);
      if (cudaIpcOpenMemHandle((void**)&g.peer_box[p], g.sh->mailbox[p], cudaIpcMemLazyEnablePeerAccess) !=
          cudaSuccess)
        fail("cudaIpcOpenMemHandle");
    }
  }
  g.up = true;
  MPI_Barrier(MPI_COMM_WORLD);
  if (g.rank == 0) shm_unlink(g.shm_name);  // everybody has it mapped
  return MPI_SUCCESS;
}

int MPI_Finalize(void) {
  if (!g.up) return MPI_SUCCESS;
  MPI_Barrier(MPI_COMM_WORLD);
  for (int p = 0; p < g.size; ++p)
    if (g.peer_box[p]) cudaIpcCloseMemHandle(g.peer_box[p]);
  MPI_Barrier(MPI_COMM_WORLD);
  if (g.my_box) cudaFree(g.my_box);
  g.up = false;
  return MPI_SUCCESS;
}

int MPI_Comm_rank(MPI_Comm, int* rank) { *rank = g.rank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm, int* size) { *size = g.size; return MPI_SUCCESS; }

int MPI_Barrier(MPI_Comm) {
  if (g.size == 1) return MPI_SUCCESS;
  g.local_sense ^= 1;
  if (g.sh->barrier_count.fetch_add(1, std::memory_order_acq_rel) == g.size - 1) {
    g.sh->barrier_count.store(0, std::memory_order_relaxed);
    g.sh->barrier_sense.store(g.local_sense, std::memory_order_release);
  } else {
    const double t0 = MPI_Wtime();
    unsigned long spins = 0;
    while (g.sh->barrier_sense.load(std::memory_order_acquire) != g.local_sense) {
      if ((++spins & 1023) == 0) {
        sched_yield();
        if (MPI_Wtime() - t0 > 120.0) fail("barrier timed out");
      }
    }
  }
  return MPI_SUCCESS;
}

int MPI_Send(const void* buf, int count, MPI_Datatype dt, int dest, int, MPI_Comm) {
  const long long bytes = (long long)count * type_bytes(dt);
  if ((size_t)bytes > g.slot_bytes) fail("message larger than a mailbox slot (raise HCREF_SLOT_BYTES)");
  Channel& ch = g.sh->chan[g.rank][dest];
  const unsigned long long seq = ch.sent.load(std::memory_order_relaxed);
  if (seq >= (unsigned long long)kSlots) spin_until(ch.taken, seq - kSlots + 1);  // slot reusable
  if (bytes > 0 && cudaMemcpy(out_slot(dest, seq), buf, (size_t)bytes, cudaMemcpyDefault) != cudaSuccess)
    fail("send copy");
  ch.nbytes[seq % kSlots] = bytes;
  ch.sent.store(seq + 1, std::memory_order_release);
  return MPI_SUCCESS;
}

static int recv_now(void* buf, long long cap, int source, MPI_Status* status) {
  Channel& ch = g.sh->chan[source][g.rank];
  const unsigned long long seq = ch.taken.load(std::memory_order_relaxed);
  spin_until(ch.sent, seq + 1);
  const long long bytes = ch.nbytes[seq % kSlots];
  if (bytes > cap) fail("message truncated");
  if (bytes > 0 && cudaMemcpy(buf, in_slot(source, seq), (size_t)bytes, cudaMemcpyDefault) != cudaSuccess)
    fail("recv copy");
  ch.taken.store(seq + 1, std::memory_order_release);
  if (status) {
    status->MPI_SOURCE = source;
    status->MPI_TAG = 0;
    status->MPI_ERROR = MPI_SUCCESS;
    status->count_bytes = bytes;
  }
  return MPI_SUCCESS;
}

int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
  MPI_Send(buf, count, dt, dest, tag, comm);  // buffered: complete on return
  hcref_request* r = (hcref_request*)calloc(1, sizeof(hcref_request));
  r->kind = 1;
  *req = r;
  return MPI_SUCCESS;
}

int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int, MPI_Comm, MPI_Request* req) {
  hcref_request* r = (hcref_request*)calloc(1, sizeof(hcref_request));
  r->kind = 0;
  r->buf = buf;
  r->cap = (long long)count * type_bytes(dt);
  r->peer = source;
  *req = r;
  return MPI_SUCCESS;
}

int MPI_Wait(MPI_Request* req, MPI_Status* status) {
  if (!req || !*req) return MPI_SUCCESS;
  hcref_request* r = *req;
  int rc = MPI_SUCCESS;
  if (r->kind == 0) rc = recv_now(r->buf, r->cap, r->peer, status);
  free(r);
  *req = MPI_REQUEST_NULL;
  return rc;
}

int MPI_Waitall(int n, MPI_Request* reqs, MPI_Status* statuses) {
  for (int i = 0; i < n; ++i) MPI_Wait(&reqs[i], statuses ? &statuses[i] : nullptr);
  return MPI_SUCCESS;
}

int MPI_Sendrecv(const void* sbuf, int scount, MPI_Datatype sdt, int dest, int stag, void* rbuf, int rcount,
                 MPI_Datatype rdt, int source, int, MPI_Comm comm, MPI_Status* status) {
  MPI_Send(sbuf, scount, sdt, dest, stag, comm);
  return recv_now(rbuf, (long long)rcount * type_bytes(rdt), source, status);
}

int MPI_Get_count(const MPI_Status* status, MPI_Datatype dt, int* count) {
  *count = (int)(status->count_bytes / type_bytes(dt));
  return MPI_SUCCESS;
}

int MPI_Comm_split_type(MPI_Comm, int, int, MPI_Info, MPI_Comm* newcomm) { *newcomm = MPI_COMM_WORLD; return MPI_SUCCESS; }
int MPI_Comm_split(MPI_Comm, int, int, MPI_Comm* newcomm) { *newcomm = MPI_COMM_NULL; return MPI_ERR_OTHER; }
int MPI_Comm_free(MPI_Comm* comm) { *comm = MPI_COMM_NULL; return MPI_SUCCESS; }
int MPI_Error_string(int code, char* str, int* len) {
  *len = snprintf(str, MPI_MAX_ERROR_STRING, "mpi shim error %d", code);
  return MPI_SUCCESS;
}
int MPI_Abort(MPI_Comm, int code) { _exit(code ? code : 1); }

}  // extern "C"
