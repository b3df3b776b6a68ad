// Device-side building blocks for the sm_100a kernels: mbarrier + TMA wrappers, scoped loads and
// stores, the tile status word of the decoupled look-back, bounded waits.
//
// Every wait in this library is bounded: it gives up after `spin_limit_ns` worth of SM clocks (or a
// hard iteration cap), records a hc::Status in the workspace's error word and lets the kernel run
// to its normal end, so a missing peer or a corrupted stream can never hang the GPU.  The reference
// spins without bound on its look-back flags (HomComp/src/GSZ.cu:204-207).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hc_format.h"

namespace hc {
namespace dev {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait; false = gave up
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit_clk = (long long)limit_ns * 2;  // SM clock is at most ~2 GHz
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u && clock64() - t0 > limit_clk) return false;
  }
  return false;
}

// ---- TMA (tiled, 2-D, no cluster features) -------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// brings a tensor map into the descriptor cache ahead of its first use (the map lives in kernel
// parameter space, __grid_constant__)
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x),
               "r"(y), "r"(smem_u32(smem_src))
               : "memory");
}
__device__ __forceinline__ void tma_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- scoped memory operations -------------------------------------------------------------------
__device__ __forceinline__ uint64_t ld_relaxed_gpu_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Arrival flag of a tile in a collective step: [63:40] call number, [39:0] byte offset of the tile's
// payload in the stream (all ones = the producer gave up on the tile).  Carrying the offset lets the
// consumer stage the tile without walking the stream's look-back chain again.
constexpr uint64_t kFlagOffsetMask = (1ull << 40) - 1;
__device__ __forceinline__ uint64_t flag_pack(uint32_t call, uint64_t offset) {
  return ((uint64_t)(call & 0xffffffu) << 40) | (offset & kFlagOffsetMask);
}
__device__ __forceinline__ bool flag_matches(uint64_t w, uint32_t call) { return (uint32_t)(w >> 40) == (call & 0xffffffu); }
// One 16-byte store that NVSwitch replicates into every GPU bound to the multicast object behind
// `mc_addr` (an address inside a multicast mapping; such addresses take multimem instructions only).
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}
// Sum over every GPU bound to the multicast object, formed inside NVSwitch: one 16-byte load returns
// the element-wise fp32 sum of the same 16 bytes of all bound memories.
__device__ __forceinline__ float4 multimem_ld_reduce_add_v4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ float multimem_ld_reduce_add_f32(const void* mc_addr) {
  float v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(v) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f32(void* mc_addr, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc_addr), "f"(v) : "memory");
}
// programmatic dependent launch: lets the runtime schedule the next kernel of the stream (if it was
// launched with programmatic serialisation) once every CTA of this grid has got here or has left
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t ld_cg_u8(const uint8_t* p) { return (uint32_t)__ldcg(p); }

// ---- look-back status word ----------------------------------------------------------------------
// [63:62] state (0 empty, 1 tile aggregate, 2 inclusive prefix, 3 poisoned)
// [61:40] launch epoch (entries of older launches read as empty, so the array is never cleared)
// [39:0]  byte count
constexpr uint64_t kStAgg = 1, kStInc = 2, kStBad = 3;
constexpr uint32_t kEpochMask = (1u << 22) - 1;
__device__ __forceinline__ uint64_t st_pack(uint64_t state, uint32_t epoch, uint64_t value) {
  return (state << 62) | ((uint64_t)(epoch & kEpochMask) << 40) | (value & ((1ull << 40) - 1));
}
__device__ __forceinline__ uint32_t st_state(uint64_t w, uint32_t epoch) {
  return (((uint32_t)(w >> 40)) & kEpochMask) == (epoch & kEpochMask) ? (uint32_t)(w >> 62) : 0u;
}
__device__ __forceinline__ uint64_t st_value(uint64_t w) { return w & ((1ull << 40) - 1); }

// ---- warp / block scans ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

}  // namespace dev
}  // namespace hc
