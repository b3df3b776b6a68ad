// Host-side launchers of the codec kernels (internal C++ interface; the C API sits on top).
#pragma once
#include <cuda_runtime.h>
#include <string.h>

#include "hc_kernels.cuh"

namespace hc {

// Bytes of device workspace for calls of up to max_elems values.  The workspace must be zeroed
// once when it is created; launches never clear it again.
size_t workspace_bytes(size_t max_elems);
Workspace workspace_view(void* mem, size_t max_elems, uint32_t epoch, uint64_t spin_limit_ns);
int grid_for_tiles(uint32_t n_tiles, int ctas_per_sm);

cudaError_t launch_encode(int op, int mode, EncParams p, cudaStream_t stream);
cudaError_t launch_decode(int mode, DecParams p, cudaStream_t stream);
cudaError_t launch_quant_pred(int mode, const float* x, int32_t* deltas, uint64_t n, float eb, cudaStream_t stream);
cudaError_t launch_sum(float* dst, const float* a, const float* b, const float* c, const float* d, uint64_t n,
                       cudaStream_t stream);

}  // namespace hc
