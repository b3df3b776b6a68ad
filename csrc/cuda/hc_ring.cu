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
//   arrival flags   one uint64 per tile for every slot and buffer above: call number and the
//                   byte offset of the tile's payload, so consumers never re-derive offsets
// Flags carry the call number, so nothing is ever reset; all-gather buffers alternate between two
// sets because a fast rank may start pushing call n+1 while a slow one still decodes call n.
#include <nvtx3/nvToolsExt.h>

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
  size_t slot_elems = 0;  // values whose stream one slot holds in the worst case
  size_t slot_bytes = 0;  // capacity of one stream slot
  size_t flag_bytes = 0;  // flags of one slot
  size_t n_slots = 0;
  size_t flags_off = 0;
  size_t raw_flags_off = 0;
  size_t total = 0;
  Layout(int P, size_t max_count) {
    world = P;
    chunk_max = hc_chunk_elems(max_count, P);
    // Two ranks: the one-step form moves as many bytes as the other two and has a phase less, so the
    // slots hold a whole message there and every call can take it.
    slot_elems = P == 2 ? (max_count > chunk_max ? max_count : chunk_max) : chunk_max;
    slot_bytes = round_up(hc::max_stream_bytes(slot_elems) + 64, kAlign);
    flag_bytes = round_up((hc::rate_bytes(slot_elems) / hc::kTileBlocks + 1) * sizeof(uint64_t), kAlign);
    n_slots = (size_t)(P - 1) + 2 * (size_t)P;
    flags_off = n_slots * slot_bytes;
    raw_flags_off = flags_off + n_slots * flag_bytes;
    total = raw_flags_off + 4096;
  }
  // uncompressed two-shot allreduce: staging area S (count floats) at the start of the region,
  // result area R right behind it; three flag rows of `world` uint32 each
  size_t raw_capacity_floats() const { return flags_off / (2 * sizeof(float)); }
  size_t raw_flag(int row, int rank) const { return raw_flags_off + ((size_t)row * 64 + rank) * sizeof(uint32_t); }
  size_t rs_slot(int s) const { return (size_t)(s - 1); }                       // s in 1..P-1
  size_t ag_slot(int parity, int c) const { return (size_t)(world - 1) + (size_t)parity * world + c; }
  size_t data_off(size_t slot) const { return slot * slot_bytes; }
  size_t flag_off(size_t slot) const { return flags_off + slot * flag_bytes; }
};

}  // namespace

constexpr int kMaxHostPieces = 32;

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
  uint32_t raw_call = 0;
  int algorithm = 1;              // 0 ring (P + 1 kernels), 1 direct (3 kernels), 2 one step (2 kernels) where it fits
  size_t small_count = 0;         // direct: messages of at most this many values take the one-step form
  int last_form = 1;              // the form the last hc_allreduce took (0 ring, 1 direct, 2 one step)
  bool trace = false;             // record one CUDA event per step of hc_allreduce
  bool overlap = true;            // direct algorithm: steps 2 and 3 start while their predecessor drains
  int share_scatter = 0, share_reduce = 0;  // direct algorithm: quarters of the GPU for steps 1 and 2 (0: all of it)
  int reduce_variant = 0;
  bool sparse = true;  // tiles at fixed offsets in the transport buffers: no look-back across CTAs in any step
  hc_host_transport host_tp = {nullptr, nullptr, nullptr};  // for the host-staged variant
  hc_codec* host_codec = nullptr;                           // created on its first use
  cudaEvent_t ev[hc::kMaxDst + 3] = {};
  int n_ev = 0;
  uint64_t spin_limit_ns = 2000ull * 1000 * 1000;
  // hierarchical allreduce: communicator of the ranks with this local index in the other groups, and
  // the buffer for this rank's slice of the group sum (created on first use)
  hc_comm* inter = nullptr;
  float* slice = nullptr;
  // hc_allreduce_host: device staging (created on first use), copy streams, one event pair per piece
  float* host_in = nullptr;
  float* host_out = nullptr;
  cudaStream_t s_h2d = nullptr, s_d2h = nullptr;
  cudaEvent_t ev_in[kMaxHostPieces] = {}, ev_out[kMaxHostPieces] = {}, ev_fork = nullptr, ev_join = nullptr;
};

namespace {

// NVTX range on the host thread: shows where each step of a collective is enqueued in a timeline
// tool; a no-op when no tool is attached
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

hc::Workspace next_ws(hc_comm* c, cudaStream_t stream) {
  c->ws_epoch = (c->ws_epoch + 1) & hc::dev::kEpochMask;
  if (c->ws_epoch == 0) {
    cudaMemsetAsync(static_cast<uint8_t*>(c->ws_mem) + hc::kWorkspaceHeader, 0, c->ws_bytes - hc::kWorkspaceHeader, stream);
    c->ws_epoch = 1;
  }
  return hc::workspace_view(c->ws_mem, c->max_count, c->ws_epoch, c->spin_limit_ns, hc::kMaxWorkspaceSets);
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
  // Where the one-step form stops paying (values per message; measured on B200 + NVSwitch at 2 and 4
  // ranks, 64 MiB / 4 Mi values being the largest sizes tried; above 4 ranks a guess on the safe side)
  c->small_count = world == 2 ? (size_t)12 << 20 : world <= 4 ? (size_t)3 << 19 : (size_t)1 << 19;
  for (int r = 0; r < world; ++r) {
    if (!peer_bases[r] || (reinterpret_cast<uintptr_t>(peer_bases[r]) & 15u)) {
      delete c;
      return hc::kErrArgument;
    }
    c->peer.push_back(static_cast<uint8_t*>(peer_bases[r]));
  }
  c->mc = static_cast<uint8_t*>(mc_base);
  c->ws_bytes = hc::workspace_bytes(max_count, hc::kMaxWorkspaceSets);
  if (cudaMalloc(&c->ws_mem, c->ws_bytes) != cudaSuccess || cudaMemset(c->ws_mem, 0, c->ws_bytes) != cudaSuccess ||
      cudaMalloc(&c->sizes, 16 * sizeof(uint64_t)) != cudaSuccess ||
      cudaMemset(c->sizes, 0, 16 * sizeof(uint64_t)) != cudaSuccess) {
    hc_comm_destroy(c);
    return hc::kErrCuda;
  }
  for (auto& e : c->ev)
    if (cudaEventCreate(&e) != cudaSuccess) {
      hc_comm_destroy(c);
      return hc::kErrCuda;
    }
  *out = c;
  return hc::kOk;
}

int hc_comm_set_trace(hc_comm* c, int on) {
  if (!c) return hc::kErrArgument;
  c->trace = on != 0;
  return hc::kOk;
}

// device time of every step of the last traced hc_allreduce: ms[0..world-1] the reduce-scatter
// steps, ms[world] the decode; returns the number of entries (synchronises the device)
int hc_comm_last_step_ms(hc_comm* c, float* ms, int n) {
  if (!c || !ms) return 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return 0;
  int k = 0;
  for (; k + 1 < c->n_ev && k < n; ++k)
    if (cudaEventElapsedTime(&ms[k], c->ev[k], c->ev[k + 1]) != cudaSuccess) break;
  return k;
}

void hc_comm_destroy(hc_comm* c) {
  if (!c) return;
  for (auto& e : c->ev)
    if (e) cudaEventDestroy(e);
  if (c->ws_mem) cudaFree(c->ws_mem);
  if (c->sizes) cudaFree(c->sizes);
  if (c->host_codec) hc_codec_destroy(c->host_codec);
  if (c->slice) cudaFree(c->slice);
  if (c->host_in) cudaFree(c->host_in);
  if (c->host_out) cudaFree(c->host_out);
  if (c->s_h2d) cudaStreamDestroy(c->s_h2d);
  if (c->s_d2h) cudaStreamDestroy(c->s_d2h);
  for (auto& e : c->ev_in)
    if (e) cudaEventDestroy(e);
  for (auto& e : c->ev_out)
    if (e) cudaEventDestroy(e);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  delete c;
}

int hc_comm_set_timeout_ms(hc_comm* c, unsigned ms) {
  if (!c || ms == 0) return hc::kErrArgument;
  c->spin_limit_ns = (uint64_t)ms * 1000ull * 1000ull;
  return hc::kOk;
}

int hc_comm_status(hc_comm* c, int clear) {
  if (!c) return hc::kErrArgument;
  // words 0-3: status of the codec kernels (2) and the first wait that ran out (3); words 32-35: the
  // counters and the status word (34) of the uncompressed / hierarchical kernels
  uint32_t ctrl[36];
  memset(ctrl, 0, sizeof(ctrl));
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  if (cudaMemcpy(ctrl, c->ws_mem, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return hc::kErrCuda;
  const uint32_t st = ctrl[2] > ctrl[34] ? ctrl[2] : ctrl[34];
  if (clear && (ctrl[0] | ctrl[1] | ctrl[2] | ctrl[3] | ctrl[33] | ctrl[34])) {
    cudaMemset(c->ws_mem, 0, 64);                                      // status and ticket counters
    cudaMemset(static_cast<uint32_t*>(c->ws_mem) + 32, 0, 4 * sizeof(uint32_t));  // raw kernels' counter and status
  }
  return (int)st;
}

// after a status 3: which wait ran out first (codes of hc_codec_status_site); read before clearing
int hc_comm_status_site(hc_comm* c) {
  if (!c) return -1;
  uint32_t ctrl[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(ctrl, c->ws_mem, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)ctrl[3];
}

int hc_comm_last_stream_bytes(hc_comm* c, uint64_t* bytes, int n) {
  if (!c || !bytes || n < 1) return hc::kErrArgument;
  if (n > 16) n = 16;
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  return cudaMemcpy(bytes, c->sizes, n * sizeof(uint64_t), cudaMemcpyDeviceToHost) == cudaSuccess ? hc::kOk
                                                                                                  : hc::kErrCuda;
}

static int allreduce_ring(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
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
  if ((c->call & 0xffffffu) == 0) c->call += 1;  // flags carry 24 bits of it; 0 means "never written"
  const uint32_t call = c->call;
  const int parity = (int)(call & 1u);
  const int next = (r + 1) % P;
  uint8_t* self = c->peer[r];

  c->n_ev = 0;
  auto mark = [&]() {
    if (c->trace) cudaEventRecord(c->ev[c->n_ev++], stream);
  };
  // Every hop consumes only what arrival flags announce and each launch has a workspace set of its own
  // (epoch % kMaxWorkspaceSets), so a hop may fill the SMs while the hop before it drains, as in the
  // direct form.  At most kMaxWorkspaceSets kernels may be in flight together, hence a normal launch
  // (which waits for everything before it) after every kMaxWorkspaceSets - 1 overlapped ones; the first
  // launch of a call is always a normal one, which the reuse of slots and flags across calls needs.
  const bool overlap = c->overlap && !c->trace;
  int chain = 0;
  bool launched = false;
  auto overlapped = [&]() -> bool {
    const bool yes = overlap && launched && chain < hc::kMaxWorkspaceSets - 1;
    chain = yes ? chain + 1 : 0;
    launched = true;
    return yes;
  };
  mark();
  // ---- reduce-scatter: steps 0 .. P-1 (the last one feeds the all-gather buffers) --------------
  for (int s = 0; s < P; ++s) {
    const int ch = ((r - s) % P + P) % P;
    const size_t n = chunk_len(ch);
    if (n == 0) continue;
    NvtxRange step_range(s == 0 ? "hc ring: compress" : (s < P - 1 ? "hc ring: hop" : "hc ring: last hop + all-gather"));
    hc::EncParams p;
    memset(&p, 0, sizeof(p));
    p.n_seg = 1;
    p.local[0] = d_sbuf + (size_t)ch * B;
    p.n[0] = n;
    p.recip = 0.5f / eb;
    p.ring_epoch = call;
    p.out_cap = L.slot_bytes;
    p.size_out = c->sizes + s;
    if (s > 0) {
      const size_t slot = L.rs_slot(s);
      p.n_in = 1;
      p.in[0] = self + L.data_off(slot);
      p.in_size[0] = L.slot_bytes;
      p.in_ready[0] = reinterpret_cast<const uint64_t*>(self + L.flag_off(slot));
    }
    if (s < P - 1) {
      const size_t slot = L.rs_slot(s + 1);
      p.n_dst = 1;
      p.out[0] = c->peer[next] + L.data_off(slot);
      p.out_ready[0] = reinterpret_cast<uint64_t*>(c->peer[next] + L.flag_off(slot));
    } else {
      // reduced chunk: to the all-gather buffer of every rank, own copy first
      const size_t slot = L.ag_slot(parity, ch);
      p.n_dst = (uint32_t)P;
      for (int k = 0; k < P; ++k) {
        const int dst = (r + k) % P;
        p.out[k] = c->peer[dst] + L.data_off(slot);
        p.out_ready[k] = reinterpret_cast<uint64_t*>(c->peer[dst] + L.flag_off(slot));
      }
      if (c->mc && P > 1) p.out_mc = c->mc + L.data_off(slot);  // one multimem store reaches all P copies
    }
    p.sparse = c->sparse ? 1u : 0u;
    p.ws = next_ws(c, stream);
    if (hc::launch_encode(s == 0 ? hc::kOpCompress : hc::kOpAddF32, hc::kModeOutlier, p, stream, overlapped()) !=
        cudaSuccess)
      return hc::kErrCuda;
    mark();
  }

  // ---- all-gather side: one kernel decodes the P reduced chunks as their tiles arrive ------------
  NvtxRange decode_range("hc ring: decode");
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
    sg.in_ready = reinterpret_cast<const uint64_t*>(self + L.flag_off(slot));
    sg.out = d_rbuf + (size_t)ch * B;
    sg.n = n;
  }
  d.ws = next_ws(c, stream);
  if (hc::launch_decode(hc::kModeOutlier, d, stream, overlapped()) != cudaSuccess) return hc::kErrCuda;
  mark();
  return hc::kOk;
}

}  // extern "C" (collective entry points continue below)

// Direct ("one-shot") form of the same reduction for a switched fabric, three kernels per call:
//   1. one multi-segment compress: chunk d of the local data is compressed straight into rank d's
//      receive slot for this source, for every d != rank (P-1 segments, peer stores, one arrival
//      flag per tile);
//   2. one homomorphic add over the own chunk: the P-1 incoming streams are decoded to deltas,
//      summed with the quantised local chunk in the integer domain and encoded once; the reduced
//      stream goes to the all-gather buffer of every rank;
//   3. the multi-segment decode.
// Integer addition is associative, so the reduced streams are byte-identical to the ring's (and to
// hc_cpu_ring_allreduce); only the number of launches and the traffic pattern differ: every rank
// talks to every other rank at once, which is what NVSwitch is built for.
static int allreduce_direct(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
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
  if ((c->call & 0xffffffu) == 0) c->call += 1;  // flags carry 24 bits of it; 0 means "never written"
  const uint32_t call = c->call;
  const int parity = (int)(call & 1u);
  uint8_t* self = c->peer[r];
  c->n_ev = 0;
  auto mark = [&]() {
    if (c->trace) cudaEventRecord(c->ev[c->n_ev++], stream);
  };
  // Steps 2 and 3 only consume what arrival flags announce and use a workspace set of their own, so
  // they may start while the step before them drains (never across calls: step 1 of the next call
  // waits for this call to end, which the reuse of slots and flags relies on).  An event between two
  // launches would undo the overlap, hence not while tracing.
  const bool overlap = c->overlap && !c->trace;
  bool launched = false;  // a kernel of this call is already on the stream
  mark();
  // ---- 1. scatter: chunk d -> rank d's slot for source r ------------------------------------------
  if (P > 1) {
    NvtxRange step_range("hc direct: scatter-compress");
    hc::EncParams p;
    memset(&p, 0, sizeof(p));
    p.recip = 0.5f / eb;
    p.ring_epoch = call;
    p.out_cap = L.slot_bytes;
    p.size_out = c->sizes;
    for (int k = 1; k < P; ++k) {
      const int d = (r + k) % P;
      const size_t n = chunk_len(d);
      if (n == 0) continue;
      const size_t slot = L.rs_slot((r - d + P) % P);  // slots are indexed by distance to the source
      const uint32_t g = p.n_seg++;
      p.local[g] = d_sbuf + (size_t)d * B;
      p.n[g] = n;
      p.out[g] = c->peer[d] + L.data_off(slot);
      p.out_ready[g] = reinterpret_cast<uint64_t*>(c->peer[d] + L.flag_off(slot));
    }
    if (p.n_seg) {
      p.n_dst = 1;
      p.sparse = c->sparse ? 1u : 0u;
      if (overlap && c->share_scatter) p.grid_limit = (uint32_t)(hc::device_sm_count() * c->share_scatter);
      p.ws = next_ws(c, stream);
      if (hc::launch_encode(hc::kOpCompress, hc::kModeOutlier, p, stream) != cudaSuccess) return hc::kErrCuda;
      launched = true;
    }
  }
  mark();
  // ---- 2. reduce the own chunk and push the result to everybody -----------------------------------
  if (const size_t n = chunk_len(r)) {
    NvtxRange step_range("hc direct: reduce + all-gather");
    hc::EncParams p;
    memset(&p, 0, sizeof(p));
    p.n_seg = 1;
    p.local[0] = d_sbuf + (size_t)r * B;
    p.n[0] = n;
    p.recip = 0.5f / eb;
    p.ring_epoch = call;
    p.out_cap = L.slot_bytes;
    p.size_out = c->sizes + (P - 1);  // after the P-1 scattered streams
    for (int k = 1; k < P; ++k) {
      const size_t slot = L.rs_slot(k);
      const uint32_t q = p.n_in++;
      p.in[q] = self + L.data_off(slot);
      p.in_size[q] = L.slot_bytes;
      p.in_ready[q] = reinterpret_cast<const uint64_t*>(self + L.flag_off(slot));
    }
    const size_t slot = L.ag_slot(parity, r);
    p.n_dst = (uint32_t)P;
    for (int k = 0; k < P; ++k) {
      const int dst = (r + k) % P;
      p.out[k] = c->peer[dst] + L.data_off(slot);
      p.out_ready[k] = reinterpret_cast<uint64_t*>(c->peer[dst] + L.flag_off(slot));
    }
    if (c->mc && P > 1) p.out_mc = c->mc + L.data_off(slot);  // one multimem store reaches all P copies
    if (overlap && launched && c->share_reduce) p.grid_limit = (uint32_t)(hc::device_sm_count() * c->share_reduce);
    p.variant = (uint32_t)c->reduce_variant;
    p.sparse = c->sparse ? 1u : 0u;
    p.ws = next_ws(c, stream);
    if (hc::launch_encode(P > 1 ? hc::kOpAddF32 : hc::kOpCompress, hc::kModeOutlier, p, stream, overlap && launched) !=
        cudaSuccess)
      return hc::kErrCuda;
    launched = true;
  }
  mark();
  // ---- 3. decode the P reduced chunks as their tiles arrive ----------------------------------------
  NvtxRange decode_range("hc direct: decode");
  hc::DecParams d;
  memset(&d, 0, sizeof(d));
  d.eb = eb;
  d.ring_epoch = call;
  for (int k = 0; k < P; ++k) {
    const int ch = (r + k) % P;  // own chunk first: it is produced locally
    const size_t n = chunk_len(ch);
    if (n == 0) continue;
    const size_t slot = L.ag_slot(parity, ch);
    hc::DecSegment& sg = d.seg[d.n_seg++];
    sg.in = self + L.data_off(slot);
    sg.in_size = L.slot_bytes;
    sg.in_ready = reinterpret_cast<const uint64_t*>(self + L.flag_off(slot));
    sg.out = d_rbuf + (size_t)ch * B;
    sg.n = n;
  }
  d.ws = next_ws(c, stream);
  if (hc::launch_decode(hc::kModeOutlier, d, stream, overlap && launched) != cudaSuccess) return hc::kErrCuda;
  mark();
  return hc::kOk;
}

// One-step form for messages that fit one all-gather slot (count <= max_count / world, rounded to the
// chunk geometry), two kernels per call:
//   1. compress the WHOLE local message once and push the stream to every rank's all-gather slot for
//      this source (peer stores or one multimem store per unit; one arrival flag per tile);
//   2. one decode that stages tile t of all P streams as their flags arrive, adds the quantised
//      values in registers and writes the fp32 sum.
// The sum of the ranks' quantised values is the same integer whatever the grouping, so the result
// has the bits of the other two forms; what changes is one network phase instead of two and no
// re-encoding, at the price of P-1 instead of 2 (P-1)/P messages on the wire: the form for small
// messages, where a call is made of fixed costs.  Slots and flags are those of the all-gather phase
// (set `call & 1`), and step 1 is a normal launch behind the previous call, so the argument for
// reusing them without a reset is the one of the direct form.
static int allreduce_onestep(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
  const int P = c->world, r = c->rank;
  const Layout& L = c->lay;
  c->call += 1;
  if ((c->call & 0xffffffu) == 0) c->call += 1;
  const uint32_t call = c->call;
  const int parity = (int)(call & 1u);
  uint8_t* self = c->peer[r];
  c->n_ev = 0;
  auto mark = [&]() {
    if (c->trace) cudaEventRecord(c->ev[c->n_ev++], stream);
  };
  const bool overlap = c->overlap && !c->trace;
  mark();
  {
    NvtxRange step_range("hc one-step: compress + broadcast");
    hc::EncParams p;
    memset(&p, 0, sizeof(p));
    p.n_seg = 1;
    p.local[0] = d_sbuf;
    p.n[0] = count;
    p.recip = 0.5f / eb;
    p.ring_epoch = call;
    p.out_cap = L.slot_bytes;
    p.size_out = c->sizes;
    const size_t slot = L.ag_slot(parity, r);
    p.n_dst = (uint32_t)P;
    for (int k = 0; k < P; ++k) {
      const int dst = (r + k) % P;
      p.out[k] = c->peer[dst] + L.data_off(slot);
      p.out_ready[k] = reinterpret_cast<uint64_t*>(c->peer[dst] + L.flag_off(slot));
    }
    if (c->mc && P > 1) p.out_mc = c->mc + L.data_off(slot);
    p.sparse = c->sparse ? 1u : 0u;
    p.ws = next_ws(c, stream);
    if (hc::launch_encode(hc::kOpCompress, hc::kModeOutlier, p, stream) != cudaSuccess) return hc::kErrCuda;
  }
  mark();
  NvtxRange decode_range("hc one-step: decode + sum");
  hc::DecParams d;
  memset(&d, 0, sizeof(d));
  d.eb = eb;
  d.ring_epoch = call;
  d.sum = 1;
  for (int k = 0; k < P; ++k) {
    const int src = (r + k) % P;  // own stream first: it is stored locally
    const size_t slot = L.ag_slot(parity, src);
    hc::DecSegment& sg = d.seg[d.n_seg++];
    sg.in = self + L.data_off(slot);
    sg.in_size = L.slot_bytes;
    sg.in_ready = reinterpret_cast<const uint64_t*>(self + L.flag_off(slot));
    sg.out = d_rbuf;
    sg.n = count;
  }
  d.ws = next_ws(c, stream);
  if (hc::launch_decode(hc::kModeOutlier, d, stream, overlap) != cudaSuccess) return hc::kErrCuda;
  mark();
  // the other words of the size report belong to steps this form does not have
  if (P > 1 && cudaMemsetAsync(c->sizes + 1, 0, (size_t)(P - 1) * sizeof(uint64_t), stream) != cudaSuccess) return hc::kErrCuda;
  return hc::kOk;
}

// Largest count the one-step form can take: what one stream slot holds.
static size_t onestep_capacity(const hc_comm* c) { return c->lay.slot_elems; }

extern "C" int hc_comm_last_form(hc_comm* c) { return c ? c->last_form : -1; }

extern "C" int hc_comm_set_small_count(hc_comm* c, size_t count) {
  if (!c) return hc::kErrArgument;
  c->small_count = count;
  return hc::kOk;
}

extern "C" int hc_comm_set_algorithm(hc_comm* c, int algorithm) {
  if (!c || algorithm < 0 || algorithm > 2) return hc::kErrArgument;
  c->algorithm = algorithm;
  return hc::kOk;
}

extern "C" int hc_comm_set_host_transport(hc_comm* c, const hc_host_transport* t) {
  if (!c || !t || !t->send || !t->recv) return hc::kErrArgument;
  c->host_tp = *t;
  return hc::kOk;
}

extern "C" int hc_comm_allreduce_host_staged(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb,
                                             hc_stream_t stream) {
  if (!c || !c->host_tp.send || count > c->max_count) return hc::kErrArgument;
  if (!c->host_codec) {
    const size_t per_rank = hc_chunk_elems(c->max_count, c->world);
    if (hc_codec_create(&c->host_codec, per_rank) != hc::kOk) return hc::kErrCuda;
    hc_codec_set_timeout_ms(c->host_codec, (unsigned)(c->spin_limit_ns / 1000000ull));
  }
  return hc_allreduce_host_staged(c->host_codec, &c->host_tp, c->rank, c->world, d_sbuf, d_rbuf, count, eb, stream);
}

extern "C" int hc_comm_set_shares(hc_comm* c, int scatter_ctas_per_sm, int reduce_ctas_per_sm, int reduce_variant) {
  if (!c || scatter_ctas_per_sm < 0 || reduce_ctas_per_sm < 0 || reduce_variant < 0 || reduce_variant > 2) return hc::kErrArgument;
  c->share_scatter = scatter_ctas_per_sm;
  c->share_reduce = reduce_ctas_per_sm;
  c->reduce_variant = reduce_variant;
  return hc::kOk;
}

extern "C" int hc_comm_set_sparse_tiles(hc_comm* c, int on) {
  if (!c) return hc::kErrArgument;
  c->sparse = on != 0;
  return hc::kOk;
}

// Call numbers tag every arrival flag, so all ranks must count the same calls.  After a call that
// some rank did not make (or gave up on before enqueueing), the ranks agree on the largest number
// any of them has reached (over their host channel) and set it everywhere: the next call then uses
// a number that no stale flag of the broken call carries.
extern "C" int hc_comm_call_numbers(hc_comm* c, uint32_t out[2]) {
  if (!c || !out) return hc::kErrArgument;
  out[0] = c->call;
  out[1] = c->raw_call;
  return hc::kOk;
}
extern "C" int hc_comm_resync(hc_comm* c, uint32_t call, uint32_t raw_call) {
  if (!c || call < c->call || raw_call < c->raw_call) return hc::kErrArgument;  // numbers only move forward
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;              // nothing of an old call in flight
  c->call = call;
  c->raw_call = raw_call;
  return hc::kOk;
}

extern "C" int hc_comm_set_overlap(hc_comm* c, int on) {
  if (!c) return hc::kErrArgument;
  c->overlap = on != 0;
  return hc::kOk;
}

extern "C" int hc_allreduce(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, float eb, hc_stream_t stream) {
  if (!c || !d_sbuf || !d_rbuf || !(eb > 0.0f) || count > c->max_count) return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  NvtxRange call_range("hc_allreduce");
  c->last_form = c->algorithm == 0 ? 0 : 1;
  if (c->algorithm == 0) return allreduce_ring(c, d_sbuf, d_rbuf, count, eb, stream);
  // one step for every message that fits (algorithm 2), or for those up to the small-message limit
  if (c->world > 1 && count <= onestep_capacity(c) && (c->algorithm == 2 || count <= c->small_count)) {
    c->last_form = 2;
    return allreduce_onestep(c, d_sbuf, d_rbuf, count, eb, stream);
  }
  return allreduce_direct(c, d_sbuf, d_rbuf, count, eb, stream);
}

// Host buffers in, host buffers out.  The reference's hostptr entry points copy the whole input up,
// run, and copy the whole output down, one after the other (GSZ_compress_hostptr,
// HomComp/src/GSZ_entry.cu:28-84).  Here the message is cut into pieces and three streams work as a
// pipeline: piece i+1 crosses PCIe upwards while piece i is reduced and piece i-1 goes back down,
// so the call costs about one direction of the PCIe transfer instead of two plus the collective.
// Every piece is an ordinary hc_allreduce of its own (same partition on all ranks).
extern "C" int hc_allreduce_host(hc_comm* c, const float* h_sbuf, float* h_rbuf, size_t count, float eb, int pieces,
                                 hc_stream_t stream) {
  if (!c || !h_sbuf || !h_rbuf || !(eb > 0.0f) || count > c->max_count) return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  if (pieces < 1) {  // default: pieces of 4 MiB, at most 16 (fill and drain of the pipeline cost one piece each)
    const size_t want = count / ((size_t)1 << 20);
    pieces = want < 1 ? 1 : (want > 16 ? 16 : (int)want);
  }
  if (pieces > kMaxHostPieces) pieces = kMaxHostPieces;
  if (!c->host_in) {  // first use: staging buffers, streams and events (set-up, not the call path)
    const size_t bytes = c->max_count * sizeof(float);
    if (cudaMalloc(&c->host_in, bytes) != cudaSuccess || cudaMalloc(&c->host_out, bytes) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->s_h2d, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->s_d2h, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess)
      return hc::kErrCuda;
    for (int i = 0; i < kMaxHostPieces; ++i)
      if (cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming) != cudaSuccess ||
          cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming) != cudaSuccess)
        return hc::kErrCuda;
  }
  // pieces of whole tiles for every rank's chunk, the last one takes the remainder
  const size_t unit = (size_t)hc::kTileElems * (size_t)c->world;
  size_t piece = (count + (size_t)pieces - 1) / (size_t)pieces;
  piece = (piece + unit - 1) / unit * unit;
  // both copy streams start behind everything already on `stream` (an earlier call's kernels still
  // read the staging input; its copies down still read the staging output, ordered by ev_join)
  if (cudaEventRecord(c->ev_fork, stream) != cudaSuccess || cudaStreamWaitEvent(c->s_h2d, c->ev_fork, 0) != cudaSuccess ||
      cudaStreamWaitEvent(c->s_d2h, c->ev_fork, 0) != cudaSuccess)
    return hc::kErrCuda;
  int i = 0;
  for (size_t off = 0; off < count; off += piece, ++i) {
    const size_t len = count - off < piece ? count - off : piece;
    if (cudaMemcpyAsync(c->host_in + off, h_sbuf + off, len * sizeof(float), cudaMemcpyHostToDevice, c->s_h2d) !=
            cudaSuccess ||
        cudaEventRecord(c->ev_in[i], c->s_h2d) != cudaSuccess || cudaStreamWaitEvent(stream, c->ev_in[i], 0) != cudaSuccess)
      return hc::kErrCuda;
    if (int rc = hc_allreduce(c, c->host_in + off, c->host_out + off, len, eb, stream)) return rc;
    if (cudaEventRecord(c->ev_out[i], stream) != cudaSuccess || cudaStreamWaitEvent(c->s_d2h, c->ev_out[i], 0) != cudaSuccess ||
        cudaMemcpyAsync(h_rbuf + off, c->host_out + off, len * sizeof(float), cudaMemcpyDeviceToHost, c->s_d2h) != cudaSuccess)
      return hc::kErrCuda;
  }
  // `stream` ends behind the last copy down: synchronising it means the result is on the host
  if (cudaEventRecord(c->ev_join, c->s_d2h) != cudaSuccess || cudaStreamWaitEvent(stream, c->ev_join, 0) != cudaSuccess)
    return hc::kErrCuda;
  return hc::kOk;
}

extern "C" {

// ---- uncompressed allreduce over the same peer mappings ------------------------------------------
// Two-shot direct algorithm for NVSwitch: every rank stages its input in its symmetric region,
// rank r sums chunk r over all ranks (peer loads, fixed rank order, so the result is bit-identical
// everywhere) and stores it into every rank's result area (peer stores).  With a multicast mapping
// the sum is formed inside the switch instead (multimem.ld_reduce) and replicated by it (multimem.st).  Takes the place of the
// reference's Open-MPI-style uncompressed ring (allreduce_ring_gpu,
// HomComp/src/cuda_awareallreduce.cu:895-1038) and of the raw intra-node phases of its hierarchical
// allreduce (:588-671).
namespace {

struct RawParams {
  const float* src;
  float* dst;
  uint64_t count;
  uint64_t chunk;  // floats per rank
  int rank, world;
  uint32_t call;
  uint8_t* peer[hc::kMaxDst];
  uint8_t* mc;                    // multicast alias of the regions (NVLS), or null
  uint64_t s_off, r_off;          // byte offsets of the staging / result areas in a region
  uint64_t flag_off[4];           // staged, reduced, done, pushed rows
  float* slice;                   // reduce-scatter: the sum of this rank's chunk goes here only
  const float* push_src;          // all-gather: this rank's chunk to be stored into every rank's result area
  uint32_t* ctrl;                 // [1] CTA exit counter, [2] status
  uint64_t limit_ns;
};

__device__ __forceinline__ bool raw_wait(const uint32_t* f, uint32_t want, const RawParams& p) {
  return hc::dev::wait_flag(f, want, p.limit_ns, p.ctrl + 2);
}

// the last CTA to finish raises this rank's flag of `row` on every peer
__device__ __forceinline__ void raw_publish(const RawParams& p, int row) {
  __syncthreads();
  __shared__ uint32_t last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(p.ctrl + 1, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (last) {
    if ((int)threadIdx.x < p.world) {
      __threadfence_system();
      hc::dev::st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer[threadIdx.x] + p.flag_off[row]) + p.rank, p.call);
    }
    if (threadIdx.x == 0) p.ctrl[1] = 0;
  }
}

__global__ void __launch_bounds__(256) hc_raw_stage_kernel(const RawParams p) {
  float* S = reinterpret_cast<float*>(p.peer[p.rank] + p.s_off);
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool al = ((reinterpret_cast<uintptr_t>(p.src) & 15u) == 0);
  const uint64_t n4 = al ? p.count / 4 : 0;
  for (uint64_t i = i0; i < n4; i += stride) reinterpret_cast<float4*>(S)[i] = reinterpret_cast<const float4*>(p.src)[i];
  for (uint64_t i = n4 * 4 + i0; i < p.count; i += stride) S[i] = p.src[i];
  raw_publish(p, 0);
}

__global__ void __launch_bounds__(256) hc_raw_reduce_kernel(const RawParams p) {
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.flag_off[0]);
  const uint32_t* done = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.flag_off[2]);
  __shared__ uint32_t ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    // everybody has staged this call's input and (unless the sum stays here) has finished reading
    // the previous call's result
    bool good = raw_wait(mine + threadIdx.x, p.call, p);
    if (good && p.call > 1 && p.slice == nullptr) good = raw_wait(done + threadIdx.x, p.call - 1, p);
    if (!good) {
      atomicMax(p.ctrl + 2, (uint32_t)hc::kErrPeer);
      ok = 0;
    }
  }
  __syncthreads();
  const uint64_t lo = (uint64_t)p.rank * p.chunk;
  const uint64_t hi = lo + p.chunk < p.count ? lo + p.chunk : p.count;
  if (ok && lo < hi && p.mc != nullptr) {
    // NVLS: the switch adds the P staged copies on the way in (one multimem load per 16 bytes) and
    // replicates the result on the way out (one multimem store); the order of the additions is the
    // switch's, the stored bits are the same on every rank
    const uint64_t n = hi - lo, n4 = n / 4;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint8_t* S = p.mc + p.s_off + lo * sizeof(float);
    uint8_t* R = p.mc + p.r_off + lo * sizeof(float);
    for (uint64_t i = i0; i < n4; i += stride) {
      const float4 acc = hc::dev::multimem_ld_reduce_add_v4(S + 16 * i);
      if (p.slice) reinterpret_cast<float4*>(p.slice)[i] = acc;
      else
        hc::dev::multimem_st_v4(R + 16 * i, __float_as_uint(acc.x), __float_as_uint(acc.y), __float_as_uint(acc.z),
                                __float_as_uint(acc.w));
    }
    for (uint64_t i = n4 * 4 + i0; i < n; i += stride) {
      const float acc = hc::dev::multimem_ld_reduce_add_f32(S + 4 * i);
      if (p.slice) p.slice[i] = acc;
      else hc::dev::multimem_st_f32(R + 4 * i, acc);
    }
  } else if (ok && lo < hi) {
    const uint64_t n = hi - lo, n4 = n / 4;  // chunk starts are multiples of 32 floats
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (uint64_t i = i0; i < n4; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < p.world; ++q) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.peer[q] + p.s_off) + lo / 4 + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (p.slice) reinterpret_cast<float4*>(p.slice)[i] = acc;
      else
        for (int q = 0; q < p.world; ++q) reinterpret_cast<float4*>(p.peer[q] + p.r_off)[lo / 4 + i] = acc;
    }
    for (uint64_t i = n4 * 4 + i0; i < n; i += stride) {
      float acc = 0.f;
      for (int q = 0; q < p.world; ++q) acc += __ldcg(reinterpret_cast<const float*>(p.peer[q] + p.s_off) + lo + i);
      if (p.slice) p.slice[i] = acc;
      else
        for (int q = 0; q < p.world; ++q) reinterpret_cast<float*>(p.peer[q] + p.r_off)[lo + i] = acc;
    }
  }
  raw_publish(p, 1);
}

// all-gather half of the hierarchical allreduce: this rank's chunk (push_src) into the result area of
// every rank of the group, peer stores or one multimem store per 16 bytes
__global__ void __launch_bounds__(256) hc_raw_push_kernel(const RawParams p) {
  const uint32_t* done = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.flag_off[2]);
  __shared__ uint32_t ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  // everybody has finished reading the previous call's result out of its result area
  if ((int)threadIdx.x < p.world && p.call > 1 && !raw_wait(done + threadIdx.x, p.call - 1, p)) {
    atomicMax(p.ctrl + 2, (uint32_t)hc::kErrPeer);
    ok = 0;
  }
  __syncthreads();
  const uint64_t lo = (uint64_t)p.rank * p.chunk;
  const uint64_t hi = lo + p.chunk < p.count ? lo + p.chunk : p.count;
  if (ok && lo < hi) {
    const uint64_t n = hi - lo, n4 = n / 4;  // chunk starts are multiples of 32 floats
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (uint64_t i = i0; i < n4; i += stride) {
      const float4 v = reinterpret_cast<const float4*>(p.push_src)[i];
      if (p.mc)
        hc::dev::multimem_st_v4(p.mc + p.r_off + (lo + 4 * i) * sizeof(float), __float_as_uint(v.x), __float_as_uint(v.y),
                                __float_as_uint(v.z), __float_as_uint(v.w));
      else
        for (int q = 0; q < p.world; ++q) reinterpret_cast<float4*>(p.peer[q] + p.r_off)[lo / 4 + i] = v;
    }
    for (uint64_t i = n4 * 4 + i0; i < n; i += stride) {
      const float v = p.push_src[i];
      if (p.mc) hc::dev::multimem_st_f32(p.mc + p.r_off + (lo + i) * sizeof(float), v);
      else
        for (int q = 0; q < p.world; ++q) reinterpret_cast<float*>(p.peer[q] + p.r_off)[lo + i] = v;
    }
  }
  raw_publish(p, 3);
}

__global__ void __launch_bounds__(256) hc_raw_gather_kernel(const RawParams p) {
  const uint32_t* red = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.flag_off[1]);
  const uint32_t* pushed = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.flag_off[3]);
  __shared__ uint32_t ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  // every rank is through with reading the staged inputs (row "reduced"); in the hierarchical form the
  // result area is filled by the push kernels instead (row "pushed")
  if ((int)threadIdx.x < p.world &&
      (!raw_wait(red + threadIdx.x, p.call, p) || (p.push_src && !raw_wait(pushed + threadIdx.x, p.call, p)))) {
    atomicMax(p.ctrl + 2, (uint32_t)hc::kErrPeer);
    ok = 0;
  }
  __syncthreads();
  if (ok) {
    const float* R = reinterpret_cast<const float*>(p.peer[p.rank] + p.r_off);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool al = ((reinterpret_cast<uintptr_t>(p.dst) & 15u) == 0);
    const uint64_t n4 = al ? p.count / 4 : 0;
    for (uint64_t i = i0; i < n4; i += stride) reinterpret_cast<float4*>(p.dst)[i] = __ldcg(reinterpret_cast<const float4*>(R) + i);
    for (uint64_t i = n4 * 4 + i0; i < p.count; i += stride) p.dst[i] = __ldcg(R + i);
  }
  raw_publish(p, 2);
}

}  // namespace

namespace {
int raw_params(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, RawParams* out) {
  const Layout& L = c->lay;
  if (count > L.raw_capacity_floats()) return hc::kErrArgument;
  c->raw_call += 1;
  if (c->raw_call == 0) c->raw_call = 1;
  RawParams& p = *out;
  memset(&p, 0, sizeof(p));
  p.src = d_sbuf;
  p.dst = d_rbuf;
  p.count = count;
  p.chunk = hc_chunk_elems(count, c->world);
  p.rank = c->rank;
  p.world = c->world;
  p.call = c->raw_call;
  for (int r = 0; r < c->world; ++r) p.peer[r] = c->peer[r];
  p.mc = c->world > 1 ? c->mc : nullptr;
  p.s_off = 0;
  p.r_off = (uint64_t)L.raw_capacity_floats() * sizeof(float);
  for (int k = 0; k < 4; ++k) p.flag_off[k] = L.raw_flag(k, 0);
  p.ctrl = static_cast<uint32_t*>(c->ws_mem) + 32;  // own counters, apart from the codec's
  p.limit_ns = c->spin_limit_ns;
  return hc::kOk;
}
}  // namespace

extern "C" int hc_allreduce_raw(hc_comm* c, const float* d_sbuf, float* d_rbuf, size_t count, hc_stream_t stream) {
  if (!c || !d_sbuf || !d_rbuf) return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  RawParams p;
  if (int rc = raw_params(c, d_sbuf, d_rbuf, count, &p)) return rc;
  const int grid = hc::device_sm_count() * 4;
  hc_raw_stage_kernel<<<grid, 256, 0, stream>>>(p);
  hc_raw_reduce_kernel<<<grid, 256, 0, stream>>>(p);
  hc_raw_gather_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

// Hierarchical allreduce (mixed_compressed_allreduce, HomComp/src/cuda_awareallreduce.cu:673-706 with
// its phases at :588-636 and :638-671): raw fp32 reduce-scatter inside the group of `local`, compressed
// allreduce of this rank's slice of the group sum between the groups (over `inter`, the ranks with the
// same local index), raw all-gather inside the group.  The reference moves the raw phases with
// MPI_Isend / MPI_Irecv and a 4-input adder hard-wired to four ranks per node; here they are the
// peer-memory kernels above for any group size, and the middle phase is hc_allreduce.
extern "C" int hc_allreduce_mixed(hc_comm* local, hc_comm* inter, const float* d_sbuf, float* d_rbuf, size_t count,
                                  float eb, hc_stream_t stream) {
  if (!local || !d_sbuf || !d_rbuf || !(eb > 0.0f)) return hc::kErrArgument;
  if (count == 0) return hc::kOk;
  RawParams p;
  if (int rc = raw_params(local, d_sbuf, d_rbuf, count, &p)) return rc;
  if (!local->slice) {  // first use (set-up): room for this rank's slice at max_count
    const size_t floats = hc_chunk_elems(local->max_count, local->world);
    if (cudaMalloc(&local->slice, (floats ? floats : 1) * sizeof(float)) != cudaSuccess) return hc::kErrCuda;
  }
  const uint64_t lo = (uint64_t)p.rank * p.chunk;
  const uint64_t n_slice = lo >= count ? 0 : (lo + p.chunk < count ? p.chunk : count - lo);
  if (inter && inter->world > 1 && n_slice > inter->max_count) return hc::kErrArgument;
  const int grid = hc::device_sm_count() * 4;
  // 1. reduce-scatter inside the group: the sum of chunk `rank` lands in local->slice
  p.slice = local->slice;
  hc_raw_stage_kernel<<<grid, 256, 0, stream>>>(p);
  hc_raw_reduce_kernel<<<grid, 256, 0, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return hc::kErrCuda;
  // 2. compressed allreduce of the slice between the groups, in place
  if (inter && inter->world > 1 && n_slice)
    if (int rc = hc_allreduce(inter, local->slice, local->slice, (size_t)n_slice, eb, stream)) return rc;
  // 3. all-gather inside the group
  p.slice = nullptr;
  p.push_src = local->slice;
  hc_raw_push_kernel<<<grid, 256, 0, stream>>>(p);
  hc_raw_gather_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

extern "C" int hc_comm_set_inter(hc_comm* local, hc_comm* inter) {
  if (!local) return hc::kErrArgument;
  local->inter = inter;
  return hc::kOk;
}
extern "C" hc_comm* hc_comm_get_inter(hc_comm* local) { return local ? local->inter : nullptr; }

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
