// Compressed ring allreduce over peer-mapped memory.
//
// Algorithm (that of allreduce_ring_comprs_hom_sum_F, HomComp/src/cuda_awareallreduce.cu:166-264):
// ring reduce-scatter in which every hop adds the local chunk to the incoming compressed chunk in
// the quantised delta domain, then distribution of the reduced compressed chunks, decoded once per
// rank.  What differs is who moves the bytes.  The reference hands every compressed chunk to
// MPI_Send / MPI_Irecv and learns its size through a blocking copy to the host.  Here each step is
// one kernel whose storing side writes the stream straight into the next rank's receive slot
// (peer stores over NVLink) and raises one arrival flag per tile; the next rank's kernel of the
// following step consumes tiles as they land.  The last reduce-scatter step stores the reduced
// chunk into the all-gather buffers of ALL ranks, and a single decode kernel turns the P chunks
// into fp32.  The host never learns a size and never waits.
//
// Symmetric region of each rank (same layout everywhere):
//   receive slots   1 .. P-1      stream written by the previous rank at its step s-1
//   all-gather bufs [2][P]        reduced chunk c of calls with parity 0 / 1
//   arrival flags   one uint32 per tile for every slot and buffer above, value = call number
// Flags carry the call number, so nothing is ever reset; all-gather buffers alternate between two
// sets because a fast rank may start pushing call n+1 while a slow one still decodes call n.
#include <new>
#include <vector>

#include "hc_launch.h"
#include "homcomp_b200.h"

namespace {

constexpr size_t kAlign = 256;
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
  int world = 0;
  size_t chunk_max = 0;   // elements per chunk at max_count
  size_t slot_bytes = 0;  // capacity of one stream slot
  size_t flag_bytes = 0;  // flags of one slot
  size_t n_slots = 0;
  size_t flags_off = 0;
  size_t total = 0;
  Layout(int P, size_t max_count) {
    world = P;
    chunk_max = hc_chunk_elems(max_count, P);
    slot_bytes = round_up(hc::max_stream_bytes(chunk_max) + 64, kAlign);
    flag_bytes = round_up((hc::rate_bytes(chunk_max) / hc::kTileBlocks + 1) * sizeof(uint32_t), kAlign);
    n_slots = (size_t)(P - 1) + 2 * (size_t)P;
    flags_off = n_slots * slot_bytes;
    total = flags_off + n_slots * flag_bytes;
  }
  size_t rs_slot(int s) const { return (size_t)(s - 1); }                       // s in 1..P-1
  size_t ag_slot(int parity, int c) const { return (size_t)(world - 1) + (size_t)parity * world + c; }
  size_t data_off(size_t slot) const { return slot * slot_bytes; }
  size_t flag_off(size_t slot) const { return flags_off + slot * flag_bytes; }
};

}  // namespace

struct hc_comm {
  int rank = 0, world = 1;
  size_t max_count = 0;
  Layout lay{1, 0};
  std::vector<uint8_t*> peer;  // symmetric region of every rank as seen from here
  uint8_t* mc = nullptr;
  void* ws_mem = nullptr;      // look-back workspace (local)
  size_t ws_bytes = 0;
  uint64_t* sizes = nullptr;   // device words: stream size produced at each step of the last call
  uint32_t ws_epoch = 0;
  uint32_t call = 0;
  uint64_t spin_limit_ns = 2000ull * 1000 * 1000;
};

namespace {

hc::Workspace next_ws(hc_comm* c, cudaStream_t stream) {
  c->ws_epoch = (c->ws_epoch + 1) & hc::dev::kEpochMask;
  if (c->ws_epoch == 0) {
    cudaMemsetAsync(static_cast<uint8_t*>(c->ws_mem) + 256, 0, c->ws_bytes - 256, stream);
    c->ws_epoch = 1;
  }
  return hc::workspace_view(c->ws_mem, c->max_count, c->ws_epoch, c->spin_limit_ns);
}

}  // namespace

extern "C" {

size_t hc_comm_symmetric_bytes(int world, size_t max_count) {
  if (world < 1) return 0;
  return Layout(world, max_count).total;
}

int hc_comm_create(hc_comm** out, int rank, int world, size_t max_count, void* const* peer_bases, void* mc_base) {
  if (!out || world < 1 || world > hc::kMaxDst || rank < 0 || rank >= world || !peer_bases) return hc::kErrArgument;
  hc_comm* c = new (std::nothrow) hc_comm();
  if (!c) return hc::kErrArgument;
  c->rank = rank;
  c->world = world;
  c->max_count = max_count;
  c->lay = Layout(world, max_count);
  for (int r = 0; r < world; ++r) {
    if (!peer_bases[r] || (reinterpret_cast<uintptr_t>(peer_bases[r]) & 15u)) {
      delete c;
      return hc::kErrArgument;
    }
    c->peer.push_back(static_cast<uint8_t*>(peer_bases[r]));
  }
  c->mc = static_cast<uint8_t*>(mc_base);
  c->ws_bytes = hc::workspace_bytes(max_count);
  if (cudaMalloc(&c->ws_mem, c->ws_bytes) != cudaSuccess || cudaMemset(c->ws_mem, 0, c->ws_bytes) != cudaSuccess ||
      cudaMalloc(&c->sizes, 16 * sizeof(uint64_t)) != cudaSuccess ||
      cudaMemset(c->sizes, 0, 16 * sizeof(uint64_t)) != cudaSuccess) {
    hc_comm_destroy(c);
    return hc::kErrCuda;
  }
  *out = c;
  return hc::kOk;
}

void hc_comm_destroy(hc_comm* c) {
  if (!c) return;
  if (c->ws_mem) cudaFree(c->ws_mem);
  if (c->sizes) cudaFree(c->sizes);
  delete c;
}

int hc_comm_set_timeout_ms(hc_comm* c, unsigned ms) {
  if (!c || ms == 0) return hc::kErrArgument;
  c->spin_limit_ns = (uint64_t)ms * 1000ull * 1000ull;
  return hc::kOk;
}

int hc_comm_status(hc_comm* c, int clear) {
  if (!c) return hc::kErrArgument;
  uint32_t ctrl[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  if (cudaMemcpy(ctrl, c->ws_mem, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return hc::kErrCuda;
  if (clear && (ctrl[0] | ctrl[1] | ctrl[2])) cudaMemset(c->ws_mem, 0, 16);
  return (int)ctrl[2];
}

int hc_comm_last_stream_bytes(hc_comm* c, uint64_t* bytes, int n) {
  if (!c || !bytes || n < 1) return hc::kErrArgument;
  if (n > 16) n = 16;
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  return cudaMemcpy(bytes, c->sizes, n * sizeof(uint64_t), cudaMemcpyDeviceToHost) == cudaSuccess ? hc::kOk
                                                                                                  : hc::kErrCuda;
}

int hc_allreduce(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
  if (!c || !d_sbuf || !d_rbuf || !(eb > 0.0f) || count > c->max_count) return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  const int P = c->world, r = c->rank;
  const Layout& L = c->lay;
  const size_t B = hc_chunk_elems(count, P);
  auto chunk_len = [&](int ch) -> size_t {
    size_t lo = (size_t)ch * B;
    if (lo >= count) return 0;
    size_t hi = lo + B;
    return (hi > count ? count : hi) - lo;
  };
  c->call += 1;
  if (c->call == 0) c->call = 1;  // 0 means "never written"
  const uint32_t call = c->call;
  const int parity = (int)(call & 1u);
  const int next = (r + 1) % P;
  uint8_t* self = c->peer[r];

  // ---- reduce-scatter: steps 0 .. P-1 (the last one feeds the all-gather buffers) --------------
  for (int s = 0; s < P; ++s) {
    const int ch = ((r - s) % P + P) % P;
    const size_t n = chunk_len(ch);
    if (n == 0) continue;
    hc::EncParams p;
    memset(&p, 0, sizeof(p));
    p.local = d_sbuf + (size_t)ch * B;
    p.n = n;
    p.recip = 0.5f / eb;
    p.ring_epoch = call;
    p.out_cap = L.slot_bytes;
    p.size_out = c->sizes + s;
    if (s > 0) {
      const size_t slot = L.rs_slot(s);
      p.in = self + L.data_off(slot);
      p.in_size = L.slot_bytes;
      p.in_ready = reinterpret_cast<const uint32_t*>(self + L.flag_off(slot));
    }
    if (s < P - 1) {
      const size_t slot = L.rs_slot(s + 1);
      p.n_dst = 1;
      p.out[0] = c->peer[next] + L.data_off(slot);
      p.out_ready[0] = reinterpret_cast<uint32_t*>(c->peer[next] + L.flag_off(slot));
    } else {
      // reduced chunk: to the all-gather buffer of every rank, own copy first
      const size_t slot = L.ag_slot(parity, ch);
      p.n_dst = (uint32_t)P;
      for (int k = 0; k < P; ++k) {
        const int dst = (r + k) % P;
        p.out[k] = c->peer[dst] + L.data_off(slot);
        p.out_ready[k] = reinterpret_cast<uint32_t*>(c->peer[dst] + L.flag_off(slot));
      }
    }
    p.ws = next_ws(c, stream);
    if (hc::launch_encode(s == 0 ? hc::kOpCompress : hc::kOpAddF32, hc::kModeOutlier, p, stream) != cudaSuccess)
      return hc::kErrCuda;
  }

  // ---- all-gather side: one kernel decodes the P reduced chunks as their tiles arrive ------------
  hc::DecParams d;
  memset(&d, 0, sizeof(d));
  d.eb = eb;
  d.ring_epoch = call;
  // own chunk first (it is produced locally), then in the order the others finish
  for (int k = 0; k < P; ++k) {
    const int ch = (r + 1 + k) % P;
    const size_t n = chunk_len(ch);
    if (n == 0) continue;
    const size_t slot = L.ag_slot(parity, ch);
    hc::DecSegment& sg = d.seg[d.n_seg++];
    sg.in = self + L.data_off(slot);
    sg.in_size = L.slot_bytes;
    sg.in_ready = reinterpret_cast<const uint32_t*>(self + L.flag_off(slot));
    sg.out = d_rbuf + (size_t)ch * B;
    sg.n = n;
  }
  d.ws = next_ws(c, stream);
  if (hc::launch_decode(hc::kModeOutlier, d, stream) != cudaSuccess) return hc::kErrCuda;
  return hc::kOk;
}

// ---- CUDA IPC helpers ---------------------------------------------------------------------------
int hc_ipc_alloc(void** d_ptr, size_t bytes, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!d_ptr || !handle) return hc::kErrArgument;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return hc::kErrCuda;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(p);
    return hc::kErrCuda;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return hc::kErrCuda;
  }
  memcpy(handle, &h, 64);
  *d_ptr = p;
  return hc::kOk;
}

int hc_ipc_open(const uint8_t handle[64], void** d_ptr) {
  if (!d_ptr || !handle) return hc::kErrArgument;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

int hc_ipc_close(void* d_ptr) { return cudaIpcCloseMemHandle(d_ptr) == cudaSuccess ? hc::kOk : hc::kErrCuda; }
int hc_ipc_free(void* d_ptr) { return cudaFree(d_ptr) == cudaSuccess ? hc::kOk : hc::kErrCuda; }

}  // extern "C"
