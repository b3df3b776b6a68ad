// Compression entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Typical cases are a plug-in
// called from inside another framework's memory pool (the pool owns all device memory and a
// stray cudaMalloc would synchronise the device or fragment the pool), a real-time or
// safety-certified loop that forbids allocation after start-up, and a process whose whole device
// budget was handed out before this library was loaded.  Such callers can still pass their own
// input and output buffers, but they cannot provide or create the scratch memory that the
// compressor needs for its look-back state (hc_codec_create allocates it, hc_codec_create_in
// needs a caller buffer that these callers may not have to spare either).
//
// hc_compress_noalloc therefore keeps that scratch in a fixed array that is part of the library
// image: a file-scope `static __device__` array, resident on every GPU that loads the library
// until the process ends.  The price is a size limit and shared state:
//
//   * n may not exceed HC_NOALLOC_MAX_ELEMS values; larger calls fail with status 4 (argument)
//     and do nothing.
//   * The FIRST call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current) and registers the kernel's shared-memory size.  Make that first
//     call before any stream capture begins.
//   * Every call on a device uses the same array, which keeps what the last call left in it.  The
//     counters that must start from zero are put back by the kernel itself when its last block
//     leaves, and everything else is tagged with a call number, so stale contents are ignored.
//     Two calls that can overlap on the GPU (different streams without an ordering between them,
//     or two host threads) race on that state: order them.
//   * Errors found on the device (output buffer too small: 1, a wait that ran out: 3) land in a
//     sticky word of the array; the call itself has returned 0 long before.  hc_noalloc_status
//     reads it.  When the buffer was too small *d_size is not written.  A time-out stays in force
//     (later calls produce nothing) until hc_noalloc_status(1) has cleared it.
//   * The call makes no cudaMalloc / cudaFree and uses no allocating library routine; it enqueues
//     one kernel on `stream` and returns without synchronising.
//
// Output is byte-identical to hc_compress with mode 0 (outlier codec).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "homcomp_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HC_NOALLOC_MAX_ELEMS ((size_t)16 * 1024 * 1024) /* 64 MiB of float32 per call */

// d_x: n float32 values, d_out: at least hc_max_compressed_bytes(n) bytes for a guaranteed fit,
// d_size: device word that receives the exact stream length.  Returns 0 or a hc::Status code.
int hc_compress_noalloc(const float* d_x, size_t n, float eb, uint8_t* d_out, size_t cap, uint64_t* d_size,
                        hc_stream_t stream);
// Synchronises the current device and returns the sticky device status of hc_compress_noalloc on it
// (0 ok, 1 output capacity exceeded, 3 a bounded wait ran out); clear != 0 also resets it.
int hc_noalloc_status(int clear);
// Upper bound of the kernel's waits (default 2000 ms); applies to later calls of this process.
int hc_noalloc_set_timeout_ms(unsigned ms);
// Bytes of the built-in scratch array (for the curious; the caller never touches it).
size_t hc_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
