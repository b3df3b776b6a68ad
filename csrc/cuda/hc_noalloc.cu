// hc_compress_noalloc: the compressor for callers that may not allocate (see homcomp_noalloc.h).
// The look-back workspace that hc_codec handles normally get from cudaMalloc or from the caller
// lives here in a file-scope device array.  No counterpart in the reference.
#include "homcomp_noalloc.h"

#include "hc_launch.h"

namespace {

// look-back state for calls of up to HC_NOALLOC_MAX_ELEMS values: ~110 KB per device
constexpr size_t kScratchBytes = 128 * 1024;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct PerDevice {
  void* scratch = nullptr;  // device address of g_noalloc_scratch on that device
  uint32_t epoch = 0;
};
PerDevice g_dev[64];

// In host code the array's name is only a handle for the runtime, not an address a kernel could
// use; the device address has to be asked for, once per device, with that device current.
int device_scratch(PerDevice** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return hc::kErrCuda;
  PerDevice& d = g_dev[dev];
  if (!d.scratch) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return hc::kErrCuda;
    d.scratch = p;
  }
  *out = &d;
  return hc::kOk;
}

}  // namespace

extern "C" {

size_t hc_noalloc_scratch_bytes(void) { return kScratchBytes; }

int hc_compress_noalloc(const float* d_x, size_t n, float eb, uint8_t* d_out, size_t cap, uint64_t* d_size,
                        hc_stream_t stream) {
  if (!d_x || !d_out || !(eb > 0.0f)) return hc::kErrArgument;
  if (n > HC_NOALLOC_MAX_ELEMS) return hc::kErrArgument;  // beyond what the built-in scratch can track
  if (hc::workspace_bytes(HC_NOALLOC_MAX_ELEMS) > kScratchBytes) return hc::kErrArgument;
  PerDevice* d = nullptr;
  if (int rc = device_scratch(&d)) return rc;
  if (n == 0) {
    if (d_size && cudaMemsetAsync(d_size, 0, sizeof(uint64_t), stream) != cudaSuccess) return hc::kErrCuda;
    return hc::kOk;
  }
  // ticket counter, exit counter and the sticky error word must start at zero; the status words
  // behind them are told apart by the call number (epoch) instead
  if (cudaMemsetAsync(d->scratch, 0, 16, stream) != cudaSuccess) return hc::kErrCuda;
  d->epoch = (d->epoch + 1) & hc::dev::kEpochMask;
  if (d->epoch == 0) {  // call numbers wrapped: drop every old status word
    if (cudaMemsetAsync(d->scratch, 0, kScratchBytes, stream) != cudaSuccess) return hc::kErrCuda;
    d->epoch = 1;
  }
  hc::EncParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = 1;
  p.local[0] = d_x;
  p.n[0] = n;
  p.recip = 0.5f / eb;
  p.n_dst = 1;
  p.out[0] = d_out;
  p.out_cap = cap;
  p.size_out = d_size;
  p.ws = hc::workspace_view(d->scratch, HC_NOALLOC_MAX_ELEMS, d->epoch, 2000ull * 1000 * 1000);
  return hc::launch_encode(hc::kOpCompress, hc::kModeOutlier, p, stream) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

}  // extern "C"
