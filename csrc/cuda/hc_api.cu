// C entry points of the device codec: a handle that owns (or borrows) the look-back workspace and
// hands out launch epochs.  Counterpart of the per-call cudaMalloc / cudaMemset / 4-byte D2H /
// cudaFree wrappers of the reference (HomComp/src/GSZ_entry.cu:263-301, :504-550) with none of
// those on the call path.
#include <new>

#include "hc_launch.h"
#include "homcomp_b200.h"

void hc_host_staged_release(const hc_codec* codec);  // hc_host_staged.cu

struct hc_codec {
  void* ws_mem = nullptr;
  size_t ws_bytes = 0;
  size_t max_elems = 0;
  bool owns = false;
  uint32_t epoch = 0;
  uint64_t spin_limit_ns = 2000ull * 1000 * 1000;
  bool prepass = true;  // large stand-alone inputs: tile offsets from a pre-pass instead of an input look-back
};

namespace {

hc::Workspace next_workspace(hc_codec* c, cudaStream_t stream) {
  c->epoch = (c->epoch + 1) & hc::dev::kEpochMask;
  if (c->epoch == 0) {
    // epoch tags wrapped: forget every old status word (2^22 launches apart)
    cudaMemsetAsync(static_cast<uint8_t*>(c->ws_mem) + hc::kWorkspaceHeader, 0, c->ws_bytes - hc::kWorkspaceHeader, stream);
    c->epoch = 1;
  }
  return hc::workspace_view(c->ws_mem, c->max_elems, c->epoch, c->spin_limit_ns);
}

// Streams of at least this many tiles get their tile offsets from the pre-pass (launch_offsets):
// below it the consuming kernel has a tile or two per CTA and its own look-back costs nothing extra.
constexpr uint32_t kPrepassMinTiles = 1024;

// Enqueues the pre-pass over `n_in` streams of n values each and returns the flag rows it fills
// (in the look-back words of the input chains, which the consumer then does not use); false when the
// streams are small or the workspace has no room, in which case the consumer walks the chains itself.
bool stage_offsets(hc_codec* c, const hc::Workspace& ws, const uint8_t* const* in, const size_t* in_size, uint32_t n_in,
                   size_t n, const uint64_t** flags, cudaStream_t stream) {
  const uint32_t tiles = (uint32_t)(hc::rate_bytes(n) / hc::kTileBlocks);
  if (!c->prepass || tiles < kPrepassMinTiles || !hc::offsets_fit(ws, c->max_elems, n_in, tiles)) return false;
  hc::OffsetParams o;
  memset(&o, 0, sizeof(o));
  o.n_in = n_in;
  o.tiles_per_seg = tiles;
  o.nrate = hc::rate_bytes(n);
  o.tag = ws.epoch;  // below 2^22: can never match a look-back status word left in the same place
  o.ws = ws;
  for (uint32_t q = 0; q < n_in; ++q) {
    o.in[q] = in[q];
    o.in_size[q] = in_size[q];
    o.flags[q] = ws.st_a + (size_t)q * tiles;
    flags[q] = o.flags[q];
  }
  return hc::launch_offsets(o, stream) == cudaSuccess;
}

int check_call(hc_codec* c, size_t n, float eb, bool needs_eb) {
  if (!c) return hc::kErrArgument;
  if (n > c->max_elems) return hc::kErrArgument;
  if (needs_eb && !(eb > 0.0f)) return hc::kErrArgument;
  return hc::kOk;
}

int encode_call(hc_codec* c, int op, int mode, const void* local, const uint8_t* in, size_t in_size,
                const uint8_t* in2, size_t in2_size, size_t n, float eb, uint8_t* out, size_t cap, uint64_t* d_size,
                cudaStream_t stream) {
  if (mode < 0 || mode > 2 || !out) return hc::kErrArgument;
  if (n == 0) {
    if (d_size) cudaMemsetAsync(d_size, 0, sizeof(uint64_t), stream);
    return hc::kOk;
  }
  hc::EncParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = 1;
  p.local[0] = local;
  p.n[0] = n;
  p.recip = 0.5f / eb;
  p.n_in = in2 ? 2u : (in ? 1u : 0u);
  p.in[0] = in;
  p.in_size[0] = in_size;
  p.in[1] = in2;
  p.in_size[1] = in2_size;
  p.n_dst = 1;
  p.out[0] = out;
  p.out_cap = cap;
  p.size_out = d_size;
  p.ws = next_workspace(c, stream);
  bool flagged = false;
  if (p.n_in) {
    const uint8_t* ins[2] = {in, in2};
    const size_t sizes[2] = {in_size, in2_size};
    flagged = stage_offsets(c, p.ws, ins, sizes, p.n_in, n, p.in_ready, stream);
    if (flagged) p.ring_epoch = p.ws.epoch;
    else p.in_ready[0] = p.in_ready[1] = nullptr;
  }
  // behind its pre-pass the kernel starts at once and consumes tiles as their flags appear
  return hc::launch_encode(op, mode, p, stream, flagged) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

}  // namespace

extern "C" {

size_t hc_codec_workspace_bytes(size_t max_elems) { return hc::workspace_bytes(max_elems); }

int hc_codec_create_in(hc_codec** out, void* d_workspace, size_t bytes, size_t max_elems, hc_stream_t stream) {
  if (!out || !d_workspace || bytes < hc::workspace_bytes(max_elems)) return hc::kErrArgument;
  if (reinterpret_cast<uintptr_t>(d_workspace) & 15u) return hc::kErrArgument;
  hc_codec* c = new (std::nothrow) hc_codec();
  if (!c) return hc::kErrArgument;
  c->ws_mem = d_workspace;
  c->ws_bytes = hc::workspace_bytes(max_elems);
  c->max_elems = max_elems;
  if (cudaMemsetAsync(d_workspace, 0, c->ws_bytes, stream) != cudaSuccess) {
    delete c;
    return hc::kErrCuda;
  }
  *out = c;
  return hc::kOk;
}

int hc_codec_create(hc_codec** out, size_t max_elems) {
  if (!out) return hc::kErrArgument;
  void* mem = nullptr;
  size_t bytes = hc::workspace_bytes(max_elems);
  if (cudaMalloc(&mem, bytes) != cudaSuccess) return hc::kErrCuda;
  int rc = hc_codec_create_in(out, mem, bytes, max_elems, nullptr);
  if (rc != hc::kOk) {
    cudaFree(mem);
    return rc;
  }
  (*out)->owns = true;
  return hc::kOk;
}

void hc_codec_destroy(hc_codec* c) {
  if (!c) return;
  hc_host_staged_release(c);  // bounce buffers of the host-staged allreduce, if this handle ever ran it
  if (c->owns) cudaFree(c->ws_mem);
  delete c;
}

int hc_codec_set_timeout_ms(hc_codec* c, unsigned ms) {
  if (!c || ms == 0) return hc::kErrArgument;
  c->spin_limit_ns = (uint64_t)ms * 1000ull * 1000ull;
  return hc::kOk;
}

int hc_codec_status_site(hc_codec* c) {
  if (!c) return -1;
  uint32_t ctrl[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(ctrl, c->ws_mem, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)ctrl[3];
}

int hc_codec_set_prepass(hc_codec* c, int on) {
  if (!c) return hc::kErrArgument;
  c->prepass = on != 0;
  return hc::kOk;
}

int hc_codec_status(hc_codec* c, int clear) {
  if (!c) return hc::kErrArgument;
  uint32_t ctrl[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  if (cudaMemcpy(ctrl, c->ws_mem, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return hc::kErrCuda;
  if (clear && (ctrl[2] != 0 || ctrl[0] != 0 || ctrl[1] != 0)) cudaMemset(c->ws_mem, 0, 64);  // status and ticket counters
  return (int)ctrl[2];
}

int hc_compress(hc_codec* c, const float* d_x, size_t n, float eb, int mode, uint8_t* d_out, size_t cap,
                uint64_t* d_size, hc_stream_t stream) {
  if (int rc = check_call(c, n, eb, true)) return rc;
  return encode_call(c, hc::kOpCompress, mode, d_x, nullptr, 0, nullptr, 0, n, eb, d_out, cap, d_size, stream);
}

int hc_hom_add_f32(hc_codec* c, const uint8_t* d_in, size_t in_size, const float* d_local, size_t n, float eb,
                   int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream) {
  if (int rc = check_call(c, n, eb, true)) return rc;
  return encode_call(c, hc::kOpAddF32, mode, d_local, d_in, in_size, nullptr, 0, n, eb, d_out, cap, d_size, stream);
}

int hc_hom_add_i32(hc_codec* c, const uint8_t* d_in, size_t in_size, const int32_t* d_deltas, size_t n, int mode,
                   uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream) {
  if (int rc = check_call(c, n, 1.0f, false)) return rc;
  return encode_call(c, hc::kOpAddI32, mode, d_deltas, d_in, in_size, nullptr, 0, n, 1.0f, d_out, cap, d_size, stream);
}

int hc_hom_add_stream(hc_codec* c, const uint8_t* d_a, size_t a_size, const uint8_t* d_b, size_t b_size, size_t n,
                      int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream) {
  if (int rc = check_call(c, n, 1.0f, false)) return rc;
  return encode_call(c, hc::kOpAddStream, mode, nullptr, d_a, a_size, d_b, b_size, n, 1.0f, d_out, cap, d_size, stream);
}

static int decompress_call(hc_codec* c, const uint8_t* d_in, size_t in_size, size_t n, float eb, int mode, float* d_x,
                           const uint64_t* d_tile_flags, uint32_t want, hc_stream_t stream) {
  if (int rc = check_call(c, n, eb, true)) return rc;
  if (mode < 0 || mode > 2 || !d_in || !d_x) return hc::kErrArgument;
  if (n == 0) return hc::kOk;
  hc::DecParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = 1;
  p.seg[0].in = d_in;
  p.seg[0].in_size = in_size;
  p.seg[0].in_ready = d_tile_flags;
  p.seg[0].out = d_x;
  p.seg[0].n = n;
  p.ring_epoch = want;
  p.eb = eb;
  p.ws = next_workspace(c, stream);
  bool flagged = false;
  if (!d_tile_flags) {
    flagged = stage_offsets(c, p.ws, &d_in, &in_size, 1, n, &p.seg[0].in_ready, stream);
    if (flagged) p.ring_epoch = p.ws.epoch;
    else p.seg[0].in_ready = nullptr;
  }
  return hc::launch_decode(mode, p, stream, flagged) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

int hc_decompress(hc_codec* c, const uint8_t* d_in, size_t in_size, size_t n, float eb, int mode, float* d_x,
                  hc_stream_t stream) {
  return decompress_call(c, d_in, in_size, n, eb, mode, d_x, nullptr, 0, stream);
}

int hc_decompress_flagged(hc_codec* c, const uint8_t* d_in, size_t in_size, size_t n, float eb, int mode, float* d_x,
                          const uint64_t* d_tile_flags, uint32_t want, hc_stream_t stream) {
  if (!d_tile_flags || want == 0 || want > 0xffffffu) return hc::kErrArgument;
  return decompress_call(c, d_in, in_size, n, eb, mode, d_x, d_tile_flags, want, stream);
}

size_t hc_tile_elems(void) { return hc::kTileElems; }

// Decode n_in streams of the same n values and add them in the quantised domain: d_x receives
// (sum of the quantised values) * 2 eb, the result a chain of homomorphic adds followed by one
// decompress would give, with one kernel and no intermediate stream.
int hc_decompress_sum(hc_codec* c, int n_in, const uint8_t* const* d_in, const size_t* in_size, size_t n, float eb,
                      float* d_x, hc_stream_t stream) {
  if (int rc = check_call(c, n, eb, true)) return rc;
  if (n_in < 1 || n_in > hc::kMaxDst || !d_in || !in_size || !d_x) return hc::kErrArgument;
  if ((size_t)n_in * hc::rate_bytes(n) > hc::rate_bytes(c->max_elems) + 64) return hc::kErrArgument;
  if (n == 0) return hc::kOk;
  hc::DecParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = (uint32_t)n_in;
  p.sum = 1;
  for (int q = 0; q < n_in; ++q) {
    p.seg[q].in = d_in[q];
    p.seg[q].in_size = in_size[q];
    p.seg[q].out = d_x;
    p.seg[q].n = n;
  }
  p.eb = eb;
  p.ws = next_workspace(c, stream);
  const uint64_t* ready[hc::kMaxIn] = {};
  const bool flagged = stage_offsets(c, p.ws, d_in, in_size, p.n_seg, n, ready, stream);
  if (flagged) {
    p.ring_epoch = p.ws.epoch;
    for (int q = 0; q < n_in; ++q) p.seg[q].in_ready = ready[q];
  }
  return hc::launch_decode(hc::kModeOutlier, p, stream, flagged) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

// Several independent tensors compressed by one launch (segments); sizes land in d_sizes[g].
int hc_compress_batch(hc_codec* c, int n_seg, const float* const* d_x, const size_t* n, float eb, int mode,
                      uint8_t* const* d_out, size_t cap_each, uint64_t* d_sizes, hc_stream_t stream) {
  if (!c || n_seg < 1 || n_seg > hc::kMaxDst || !(eb > 0.0f) || !d_x || !n || !d_out) return hc::kErrArgument;
  hc::EncParams p;
  memset(&p, 0, sizeof(p));
  size_t total = 0;
  for (int g = 0; g < n_seg; ++g) {
    p.local[g] = d_x[g];
    p.n[g] = n[g];
    p.out[g] = d_out[g];
    // whole chunks per segment: that is what the look-back chains of the workspace are sized in
    total += hc::rate_bytes(n[g]) * hc::kBlock;
  }
  if (total > hc::rate_bytes(c->max_elems) * hc::kBlock) return hc::kErrArgument;
  p.n_seg = (uint32_t)n_seg;
  p.n_dst = 1;
  p.recip = 0.5f / eb;
  p.out_cap = cap_each;
  p.size_out = d_sizes;
  p.ws = next_workspace(c, stream);
  return hc::launch_encode(hc::kOpCompress, mode, p, stream) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

// n_in streams (+) fp32 -> stream: every stream is decoded to deltas and summed in the integer
// domain together with the quantised local values, then encoded once.
int hc_hom_add_multi(hc_codec* c, int n_in, const uint8_t* const* d_in, const size_t* in_size, const float* d_local,
                     size_t n, float eb, int mode, uint8_t* d_out, size_t cap, uint64_t* d_size, hc_stream_t stream) {
  if (int rc = check_call(c, n, eb, true)) return rc;
  if (n_in < 1 || n_in > hc::kMaxIn || !d_in || !in_size || !d_local || !d_out) return hc::kErrArgument;
  if ((size_t)n_in * hc::rate_bytes(n) > hc::rate_bytes(c->max_elems) + 64) return hc::kErrArgument;
  if (n == 0) return hc::kOk;
  hc::EncParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = 1;
  p.local[0] = d_local;
  p.n[0] = n;
  p.recip = 0.5f / eb;
  p.n_in = (uint32_t)n_in;
  for (int q = 0; q < n_in; ++q) {
    p.in[q] = d_in[q];
    p.in_size[q] = in_size[q];
  }
  p.n_dst = 1;
  p.out[0] = d_out;
  p.out_cap = cap;
  p.size_out = d_size;
  p.ws = next_workspace(c, stream);
  const bool flagged = stage_offsets(c, p.ws, d_in, in_size, p.n_in, n, p.in_ready, stream);
  if (flagged) p.ring_epoch = p.ws.epoch;
  else
    for (int q = 0; q < n_in; ++q) p.in_ready[q] = nullptr;
  return hc::launch_encode(hc::kOpAddF32, mode, p, stream, flagged) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

int hc_quant_pred(const float* d_x, size_t n, float eb, int mode, int32_t* d_deltas, hc_stream_t stream) {
  if (!(eb > 0.0f) || !d_x || !d_deltas) return hc::kErrArgument;
  return hc::launch_quant_pred(mode, d_x, d_deltas, n, eb, stream) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

int hc_sum(float* d_dst, const float* d_a, const float* d_b, const float* d_c, const float* d_d, size_t n,
           hc_stream_t stream) {
  if (!d_dst || !d_a || !d_b) return hc::kErrArgument;
  return hc::launch_sum(d_dst, d_a, d_b, d_c, d_d, n, stream) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

const char* hc_status_string(int status) {
  switch (status) {
    case hc::kOk: return "ok";
    case hc::kErrCapacity: return "output buffer too small for the stream";
    case hc::kErrTruncated: return "input stream shorter than its rate bytes imply";
    case hc::kErrTimeout: return "a bounded device-side wait ran out";
    case hc::kErrArgument: return "invalid argument";
    case hc::kErrCuda: return "CUDA runtime error";
    case hc::kErrPeer: return "a peer failed or never arrived";
    default: return "unknown status";
  }
}

}  // extern "C"
