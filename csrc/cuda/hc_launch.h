// Host-side launchers of the codec kernels (internal C++ interface; the C API sits on top).
#pragma once
#include <cuda_runtime.h>
#include <string.h>

#include "hc_kernels.cuh"

namespace hc {

// Bytes of device workspace for calls of up to max_elems values.  The workspace must be zeroed
// once when it is created; launches never clear it again.
// `sets` > 1 gives consecutive launches (epoch % sets) their own look-back words and ticket counters,
// so that a launch may start while its predecessor on the stream is still draining.
constexpr int kMaxWorkspaceSets = 4;
// bytes in front of the look-back words: status, ticket counters, raw-allreduce counters (first 256
// bytes), per-segment payload byte counts of the four sets (second 256 bytes)
constexpr size_t kWorkspaceHeader = 512;
size_t workspace_bytes(size_t max_elems, int sets = 1);
Workspace workspace_view(void* mem, size_t max_elems, uint32_t epoch, uint64_t spin_limit_ns, int sets = 1);
int device_sm_count();

// `overlap`: programmatic dependent launch: the kernel may start as soon as every CTA of the previous
// kernel on the stream is running, and fills the SMs as that kernel's CTAs leave.  Only for launches
// whose inputs are ordered by arrival flags, with a workspace view of their own set.
cudaError_t launch_encode(int op, int mode, EncParams p, cudaStream_t stream, bool overlap = false);
cudaError_t launch_decode(int mode, DecParams p, cudaStream_t stream, bool overlap = false);
// Per-tile payload offsets of stand-alone input streams as arrival flags (see OffsetParams);
// offsets_fit says whether the workspace of a handle sized for max_elems has room for the flags of
// n_in streams of tiles_per_seg tiles and for the pre-pass's own chain.
bool offsets_fit(const Workspace& ws, size_t max_elems, uint32_t n_in, uint32_t tiles_per_seg);
cudaError_t launch_offsets(const OffsetParams& p, cudaStream_t stream);
cudaError_t launch_quant_pred(int mode, const float* x, int32_t* deltas, uint64_t n, float eb, cudaStream_t stream);
cudaError_t launch_sum(float* dst, const float* a, const float* b, const float* c, const float* d, uint64_t n,
                       cudaStream_t stream);

}  // namespace hc
