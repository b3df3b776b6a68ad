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

// upper bound of every device-side wait of the entry point, in nanoseconds (process-wide)
unsigned long long g_timeout_ns = 2000ull * 1000 * 1000;

}  // namespace

extern "C" {

size_t hc_noalloc_scratch_bytes(void) { return kScratchBytes; }

int hc_noalloc_set_timeout_ms(unsigned ms) {
  if (ms == 0) return hc::kErrArgument;
  g_timeout_ns = (unsigned long long)ms * 1000ull * 1000ull;
  return hc::kOk;
}

int hc_noalloc_status(int clear) {
  PerDevice* d = nullptr;
  if (int rc = device_scratch(&d)) return rc;
  uint32_t ctrl[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return hc::kErrCuda;
  if (cudaMemcpy(ctrl, d->scratch, sizeof(ctrl), cudaMemcpyDeviceToHost) != cudaSuccess) return hc::kErrCuda;
  // status word, first-time-out site and the ticket counters a failed launch may have left behind
  if (clear && cudaMemset(d->scratch, 0, 64) != cudaSuccess) return hc::kErrCuda;
  return (int)ctrl[2];
}

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
  // Nothing is cleared here.  The ticket and exit counters (words 8 and 9 of the array) are put back
  // to zero by the last CTA of every launch, the look-back words behind the header are told apart by
  // the call number (epoch), and the status word (word 2) is sticky on purpose: it keeps the first
  // error until hc_noalloc_status(1) has shown it to the caller, and a time-out left there makes
  // later calls return without output until then.
  d->epoch = (d->epoch + 1) & hc::dev::kEpochMask;
  if (d->epoch == 0) {  // call numbers wrapped: drop every old look-back word (not the header)
    if (cudaMemsetAsync(static_cast<uint8_t*>(d->scratch) + hc::kWorkspaceHeader, 0, kScratchBytes - hc::kWorkspaceHeader,
                        stream) != cudaSuccess)
      return hc::kErrCuda;
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
  p.ws = hc::workspace_view(d->scratch, HC_NOALLOC_MAX_ELEMS, d->epoch, g_timeout_ns);
  return hc::launch_encode(hc::kOpCompress, hc::kModeOutlier, p, stream) == cudaSuccess ? hc::kOk : hc::kErrCuda;
}

}  // extern "C"
