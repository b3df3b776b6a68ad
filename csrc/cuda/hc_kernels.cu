// Kernel bodies and host launchers of the sm_100a codec (see hc_kernels.cuh for the design).
#include "hc_kernels.cuh"

#include <stdio.h>

#include "hc_launch.h"

namespace hc {
namespace dev {

struct __align__(16) CtaShared {
  uint64_t mbar[2];
  uint64_t base_in[2];  // exclusive payload prefix of the tile in input stream 0 / 1
  uint64_t base_out;
  int32_t tile[2];
  uint32_t tile_tma[2];  // 1 when a TMA load was issued for the tile in that stage
  uint32_t wsum_in[2][kThreads / 32];
  uint32_t wsum_out[kThreads / 32];
  uint32_t ok_in[2];
  uint32_t ok_out;
  uint32_t abort;
};

__device__ __forceinline__ void note_error(uint32_t* ctrl, uint32_t code) { atomicMax(ctrl + 2, code); }
// timeouts and peer failures end the launch early; capacity / truncation errors only skip data
__device__ __forceinline__ bool fatal_error(const uint32_t* ctrl) {
  return *((volatile const uint32_t*)(ctrl + 2)) >= (uint32_t)kErrTimeout;
}

// the last CTA to leave re-arms the ticket counter for the next launch
__device__ __forceinline__ void cta_epilogue(uint32_t* ctrl) {
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(ctrl + 1, 1u);
    if (done == gridDim.x - 1) {
      ctrl[0] = 0;
      ctrl[1] = 0;
      __threadfence();
    }
  }
}

// Stages one input stream's tile: rate byte per thread, block scan, look-back, bytes into `cbuf`.
// Returns the staged position of this thread's payload (or ~0u when the tile is unusable) and the
// thread's rate byte.
__device__ __forceinline__ uint32_t stage_input_tile(const uint8_t* in, uint64_t in_size, uint64_t n, uint32_t tile,
                                                     uint64_t* st, const Workspace& ws, CtaShared& sh, int which,
                                                     uint8_t* cbuf, uint32_t* rate_out) {
  const int tid = threadIdx.x;
  const uint64_t nrate = rate_bytes(n);
  uint32_t rate = 0;
  const uint64_t bidx = (uint64_t)tile * kTileBlocks + tid;
  if (bidx < in_size) rate = ld_cg_u8(in + bidx);
  const uint32_t len = payload_len(rate);
  uint32_t tot;
  const uint32_t rel = block_exclusive_scan(len, sh.wsum_in[which], &tot);
  if (tid < 32) {
    bool ok;
    uint64_t excl = lookback(st, tile, ws.epoch, tot, ws.spin_limit_ns, ws.ctrl + 2, &ok);
    if (tid == 0) {
      sh.base_in[which] = excl;
      sh.ok_in[which] = ok ? 1u : 0u;
    }
  }
  __syncthreads();
  const uint64_t base = nrate + sh.base_in[which];
  bool ok = sh.ok_in[which] != 0;
  if (ok && base + tot > in_size) {  // stream shorter than its rate bytes imply
    if (tid == 0) note_error(ws.ctrl, kErrTruncated);
    ok = false;
  }
  uint32_t phase = 0;
  if (ok && tot) phase = stage_stream_bytes(cbuf, in + base, tot);
  *rate_out = ok ? rate : 0u;
  __syncthreads();
  return phase + rel;
}

template <int OP, int MODE>
__global__ void __launch_bounds__(kThreads, 2)
hc_encode_kernel(const __grid_constant__ CUtensorMap tmap, const EncParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ CtaShared sh;
  constexpr bool kHasLocal = OP != kOpAddStream;
  constexpr bool kHasIn = OP != kOpCompress;
  uint8_t* stage[2] = {smem, smem + kStageBytes};
  uint8_t* cbuf = smem + 2 * kStageBytes;  // staged input stream; later the staged output
  uint8_t* cbuf2 = smem;                   // second input stream (no local tile in that op)

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const Workspace& ws = p.ws;
  const bool tma = kHasLocal && p.use_tma;
  const uint64_t nrate = rate_bytes(p.n);
  // rows the tensor map covers: int32 deltas come in whole blocks, fp32 data may end in a ragged row
  const uint64_t full_rows = OP == kOpAddI32 ? num_blocks(p.n) : p.n / kBlock;
  const uint64_t n_local = OP == kOpAddI32 ? num_blocks(p.n) * kBlock : p.n;

  if (tid == 0) {
    mbar_init(&sh.mbar[0], 1);
    mbar_init(&sh.mbar[1], 1);
    fence_mbar_init();
    sh.abort = fatal_error(ws.ctrl) ? 1u : 0u;
    int32_t t0 = (int32_t)atomicAdd(ws.ctrl, 1u);
    sh.tile[0] = t0;
    sh.tile_tma[0] = 0;
    // a tile that starts past the last full row has nothing to fetch (its rows read as zeros)
    if (tma && (uint32_t)t0 < p.n_tiles && (uint64_t)t0 * kTileBlocks < full_rows) {
      mbar_expect_tx(&sh.mbar[0], kTileBytes);
      tma_load_2d(stage[0], &tmap, 0, t0 * kTileBlocks, &sh.mbar[0]);
      sh.tile_tma[0] = 1;
    }
  }
  __syncthreads();

  uint32_t uses[2] = {0, 0};  // completed TMA loads per stage: the parity to wait for
  for (uint32_t it = 0;; ++it) {
    const int cur = it & 1;
    const uint32_t tile = (uint32_t)sh.tile[cur];
    if (tile >= p.n_tiles) break;
    const bool tile_tma = sh.tile_tma[cur] != 0;
    if (sh.abort) {
      // a failure somewhere: stop taking work; wait out our own copy in flight first
      if (tid == 0 && tile_tma) mbar_wait_bounded(&sh.mbar[cur], uses[cur] & 1, ws.spin_limit_ns);
      break;
    }
    if (tid == 0) {
      int32_t tn = (int32_t)atomicAdd(ws.ctrl, 1u);
      sh.tile[cur ^ 1] = tn;
      sh.tile_tma[cur ^ 1] = 0;
      if (tma && (uint32_t)tn < p.n_tiles && (uint64_t)tn * kTileBlocks < full_rows) {
        fence_proxy_async();
        mbar_expect_tx(&sh.mbar[cur ^ 1], kTileBytes);
        tma_load_2d(stage[cur ^ 1], &tmap, 0, tn * kTileBlocks, &sh.mbar[cur ^ 1]);
        sh.tile_tma[cur ^ 1] = 1;
      }
    }

    int32_t d[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) d[i] = 0;

    // ---- incoming stream(s) -> signed deltas ------------------------------------------------
    if (kHasIn) {
      if (p.in_ready) {
        if (tid == 0 && !wait_flag(p.in_ready + tile, p.ring_epoch, ws.spin_limit_ns, ws.ctrl + 2)) {
          note_error(ws.ctrl, kErrPeer);
          sh.abort = 1;
        }
        __syncthreads();
      }
      uint32_t rate_in;
      uint32_t pos = stage_input_tile(p.in, p.in_size, p.n, tile, ws.st_a, ws, sh, 0, cbuf, &rate_in);
      int W = plane_width(rate_in & 31u);
      W = __reduce_max_sync(0xffffffffu, W);
      if (__any_sync(0xffffffffu, rate_in != 0)) decode_block(cbuf, pos, rate_in, W, d);
      if (OP == kOpAddStream) {
        uint32_t rate2;
        uint32_t pos2 = stage_input_tile(p.in2, p.in2_size, p.n, tile, ws.st_b, ws, sh, 1, cbuf2, &rate2);
        int W2 = plane_width(rate2 & 31u);
        W2 = __reduce_max_sync(0xffffffffu, W2);
        if (__any_sync(0xffffffffu, rate2 != 0)) {
          int32_t d2[32];
          decode_block(cbuf2, pos2, rate2, W2, d2);
#pragma unroll
          for (int i = 0; i < 32; ++i) d[i] += d2[i];
        }
      }
    }

    // ---- local operand -------------------------------------------------------------------------
    if (kHasLocal) {
      uint32_t w[32];
      const uint64_t row = (uint64_t)tile * kTileBlocks + tid;
      if (tma) {
        if (tile_tma) {
          if (!mbar_wait_bounded(&sh.mbar[cur], uses[cur] & 1, ws.spin_limit_ns)) {
            note_error(ws.ctrl, kErrTimeout);
            sh.abort = 1;
          }
          ++uses[cur];
          load_row_swizzled(stage[cur], tid, w);  // rows past the map were zero-filled by the TMA unit
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = 0;
        }
        // the ragged last row of fp32 data is not part of the tensor map
        if (OP != kOpAddI32 && row * kBlock < p.n && (row + 1) * kBlock > p.n)
          load_row_global((const uint32_t*)p.local, p.n, row, w);
      } else {
        load_row_global((const uint32_t*)p.local, n_local, row, w);
      }
      int32_t q[32];
      if (OP == kOpAddI32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) d[i] += (int32_t)w[i];
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) q[i] = quantise(__uint_as_float(w[i]), p.recip);
        int32_t dl[32];
        lorenzo_forward<MODE>(q, dl);
#pragma unroll
        for (int i = 0; i < 32; ++i) d[i] += dl[i];
      }
    }

    // ---- encode ----------------------------------------------------------------------------------
    uint32_t A[32];
    BlockCode code = analyse_block<MODE>(d, A);
    uint32_t tot;
    const uint32_t rel = block_exclusive_scan(code.len, sh.wsum_out, &tot);  // barrier: inputs are in registers now
    if (tid < 32) {
      bool ok;
      uint64_t excl = lookback(ws.st_out, tile, ws.epoch, tot, ws.spin_limit_ns, ws.ctrl + 2, &ok);
      if (tid == 0) {
        sh.base_out = excl;
        sh.ok_out = ok ? 1u : 0u;
        if (ok && tile == p.n_tiles - 1 && p.size_out) *p.size_out = nrate + excl + tot;
      }
    }
    int W = plane_width(code.rate & 31u);
    W = __reduce_max_sync(0xffffffffu, W);
    transpose_forward(A, W);
    __syncthreads();

    const uint64_t obase = nrate + sh.base_out;
    bool ok = sh.ok_out != 0;
    if (ok && obase + tot > p.out_cap) {
      if (tid == 0) note_error(ws.ctrl, kErrCapacity);
      ok = false;
    }
    uint8_t* obuf = kHasIn ? cbuf : stage[cur];
    const uint32_t phase = (uint32_t)((reinterpret_cast<uintptr_t>(p.out[0]) + obase) & 15u);
    if (ok) write_payload(obuf, phase + rel, code, A, W);
    __syncthreads();
    if (ok) {
      // rate bytes (section A) and payload (section B) to every destination
      const uint64_t bidx = (uint64_t)tile * kTileBlocks + tid;
      const uint32_t nvec = (phase + tot + 15u) >> 4;
      const uint32_t lo_valid = phase, hi_valid = phase + tot;
#pragma unroll 1
      for (uint32_t dsti = 0; dsti < p.n_dst; ++dsti) {
        uint8_t* o = p.out[dsti];
        o[bidx] = (uint8_t)code.rate;
        uint8_t* al = o + obase - phase;
        for (uint32_t v = tid; v < nvec; v += kThreads) {
          const uint32_t lo = v << 4, hi = lo + 16;
          if (lo >= lo_valid && hi <= hi_valid) {
            *reinterpret_cast<uint4*>(al + lo) = reinterpret_cast<const uint4*>(obuf)[v];
          } else {
            for (uint32_t b = max(lo, lo_valid); b < min(hi, hi_valid); ++b) al[b] = obuf[b];
          }
        }
      }
    }
    if (p.out_ready[0] != nullptr) {  // ring step: tell the consumers that this tile has landed
      __syncthreads();
      if ((uint32_t)tid < p.n_dst && p.out_ready[tid] != nullptr) {
        __threadfence_system();
        st_release_sys_u32(p.out_ready[tid] + tile, ok ? p.ring_epoch : 0xffffffffu);
      }
    }
    if (tid == 0 && fatal_error(ws.ctrl)) sh.abort = 1;
    __syncthreads();
  }
  (void)lane;
  cta_epilogue(ws.ctrl);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 2)
hc_decode_kernel(const __grid_constant__ CUtensorMap tmap, const DecParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ CtaShared sh;
  uint8_t* obuf[2] = {smem, smem + kTileBytes};
  uint8_t* cbuf = smem + 2 * kTileBytes;

  const int tid = threadIdx.x;
  const Workspace& ws = p.ws;
  const bool tma = p.use_tma != 0;
  const float eb = p.eb;

  const uint64_t full_rows = p.n / kBlock;
  if (tid == 0) {
    sh.abort = fatal_error(ws.ctrl) ? 1u : 0u;
    sh.tile[0] = (int32_t)atomicAdd(ws.ctrl, 1u);
  }
  __syncthreads();

  for (uint32_t it = 0;; ++it) {
    const int cur = it & 1;
    const uint32_t tile = (uint32_t)sh.tile[cur];
    if (tile >= p.n_tiles) break;
    if (sh.abort) break;
    if (tid == 0) {
      sh.tile[cur ^ 1] = (int32_t)atomicAdd(ws.ctrl, 1u);
      if (tma) tma_wait_group_read<1>();  // the store that used obuf[cur] two tiles ago has drained
    }
    if (p.in_ready) {
      if (tid == 0 && !wait_flag(p.in_ready + tile, p.ring_epoch, ws.spin_limit_ns, ws.ctrl + 2)) {
        note_error(ws.ctrl, kErrPeer);
        sh.abort = 1;
      }
      __syncthreads();
    }
    uint32_t rate;
    uint32_t pos = stage_input_tile(p.in, p.in_size, p.n, tile, ws.st_a, ws, sh, 0, cbuf, &rate);
    int W = plane_width(rate & 31u);
    W = __reduce_max_sync(0xffffffffu, W);
    int32_t d[32];
    if (__any_sync(0xffffffffu, rate != 0)) {
      decode_block(cbuf, pos, rate, W, d);
      lorenzo_inverse<MODE>(d);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) d[i] = 0;
    }
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__fmul_rn(__fmul_rn((float)d[i], eb), 2.0f));

    const uint64_t row = (uint64_t)tile * kTileBlocks + tid;
    const bool ragged = row * kBlock < p.n && (row + 1) * kBlock > p.n;
    if (tma) {
      store_row_swizzled(obuf[cur], tid, w);
      fence_proxy_async();
      __syncthreads();
      if (tid == 0) {
        if ((uint64_t)tile * kTileBlocks < full_rows) tma_store_2d(&tmap, 0, (int)(tile * kTileBlocks), obuf[cur]);
        tma_commit_group();  // an empty group keeps the two-deep accounting uniform
      }
    }
    if (!tma || ragged) {
      const uint64_t o = row * kBlock;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (o + i < p.n) p.out[o + i] = __uint_as_float(w[i]);
    }
    if (tid == 0 && fatal_error(ws.ctrl)) sh.abort = 1;
    __syncthreads();
  }
  if (tid == 0 && tma) tma_wait_group<0>();
  cta_epilogue(ws.ctrl);
}

// fp32 -> int32 Lorenzo deltas of the quantised values, padded with zero deltas to whole blocks.
// Counterpart of kernel_quant_prediction (HomComp/src/homcomp.cu:1553-1602).
template <int MODE>
__global__ void __launch_bounds__(256) hc_quant_pred_kernel(const float* __restrict__ x, int32_t* __restrict__ out,
                                                            uint64_t n, uint64_t n_padded, float recip) {
  constexpr int S = MODE == kModeVec ? 4 : 1;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_padded; i += stride) {
    const float v = i < n ? x[i] : 0.0f;
    const int32_t q = quantise(v, recip);
    int32_t prev = 0;
    if ((i & 31) >= S) {
      const uint64_t j = i - S;
      prev = quantise(j < n ? x[j] : 0.0f, recip);
    }
    out[i] = q - prev;
  }
}

// dst = a + b (+ c + d): the fp32 adders of the uncompressed collectives
// (sum2arrays / sum4arrays, HomComp/src/cuda_awareallreduce.cu:885-893 and :577-586)
__global__ void __launch_bounds__(256) hc_sum_kernel(float* __restrict__ dst, const float* a, const float* b,
                                                     const float* c, const float* d, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t i0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool al = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                    reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d)) & 15u) == 0;
  const uint64_t n4 = al ? n / 4 : 0;
  for (uint64_t i = i0; i < n4; i += stride) {
    float4 va = reinterpret_cast<const float4*>(a)[i], vb = reinterpret_cast<const float4*>(b)[i];
    float4 r = make_float4(va.x + vb.x, va.y + vb.y, va.z + vb.z, va.w + vb.w);
    if (c) {
      float4 vc = reinterpret_cast<const float4*>(c)[i];
      r.x += vc.x; r.y += vc.y; r.z += vc.z; r.w += vc.w;
    }
    if (d) {
      float4 vd = reinterpret_cast<const float4*>(d)[i];
      r.x += vd.x; r.y += vd.y; r.z += vd.z; r.w += vd.w;
    }
    reinterpret_cast<float4*>(dst)[i] = r;
  }
  for (uint64_t i = n4 * 4 + i0; i < n; i += stride) {
    float r = a[i] + b[i];
    if (c) r += c[i];
    if (d) r += d[i];
    dst[i] = r;
  }
}

}  // namespace dev

// ---- host side ---------------------------------------------------------------------------------

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 2-D view {32, rows} of a 4-byte-element array, box {32, 256}, 128-byte swizzle
bool make_rows_map(CUtensorMap* map, const void* base, uint64_t rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || rows == 0 || (reinterpret_cast<uintptr_t>(base) & 15u)) return false;
  cuuint64_t dims[2] = {(cuuint64_t)kBlock, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kBlock * 4};
  cuuint32_t box[2] = {(cuuint32_t)kBlock, (cuuint32_t)kTileBlocks};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct DeviceInfo {
  int sms = 0;
  bool ready = false;
};
DeviceInfo& device_info() {
  static thread_local DeviceInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  DeviceInfo& d = info[dev & 63];
  if (!d.ready) {
    cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    d.ready = true;
  }
  return d;
}

constexpr int kEncSmemLocalOnly = 2 * kStageBytes + 1024;
constexpr int kEncSmemWithIn = 3 * kStageBytes + 1024;
constexpr int kDecSmem = 2 * kTileBytes + kStageBytes + 1024;

template <typename K>
cudaError_t set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int OP, int MODE>
cudaError_t launch_encode_t(const CUtensorMap& map, const EncParams& p, int grid, cudaStream_t stream) {
  constexpr int smem = OP == kOpCompress ? kEncSmemLocalOnly : kEncSmemWithIn;
  static thread_local bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = set_smem(dev::hc_encode_kernel<OP, MODE>, smem);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  dev::hc_encode_kernel<OP, MODE><<<grid, kThreads, smem, stream>>>(map, p);
  return cudaGetLastError();
}

template <int OP>
cudaError_t launch_encode_m(int mode, const CUtensorMap& map, const EncParams& p, int grid, cudaStream_t stream) {
  switch (mode) {
    case kModeOutlier: return launch_encode_t<OP, kModeOutlier>(map, p, grid, stream);
    case kModePlain: return launch_encode_t<OP, kModePlain>(map, p, grid, stream);
    case kModeVec: return launch_encode_t<OP, kModeVec>(map, p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

template <int MODE>
cudaError_t launch_decode_t(const CUtensorMap& map, const DecParams& p, int grid, cudaStream_t stream) {
  static thread_local bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = set_smem(dev::hc_decode_kernel<MODE>, kDecSmem);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  dev::hc_decode_kernel<MODE><<<grid, kThreads, kDecSmem, stream>>>(map, p);
  return cudaGetLastError();
}

}  // namespace

size_t workspace_bytes(size_t max_elems) {
  size_t tiles = rate_bytes(max_elems) / kTileBlocks + 1;
  return 256 + 3 * tiles * sizeof(uint64_t);
}

Workspace workspace_view(void* mem, size_t max_elems, uint32_t epoch, uint64_t spin_limit_ns) {
  size_t tiles = rate_bytes(max_elems) / kTileBlocks + 1;
  Workspace w;
  uint8_t* b = static_cast<uint8_t*>(mem);
  w.ctrl = reinterpret_cast<uint32_t*>(b);
  w.st_a = reinterpret_cast<uint64_t*>(b + 256);
  w.st_b = w.st_a + tiles;
  w.st_out = w.st_b + tiles;
  w.epoch = epoch;
  w.spin_limit_ns = spin_limit_ns;
  return w;
}

int grid_for_tiles(uint32_t n_tiles, int ctas_per_sm) {
  int cap = device_info().sms * ctas_per_sm;
  if (cap <= 0) cap = 148 * ctas_per_sm;
  return (int)(n_tiles < (uint32_t)cap ? n_tiles : (uint32_t)cap);
}

cudaError_t launch_encode(int op, int mode, EncParams p, cudaStream_t stream) {
  if (p.n == 0) return cudaSuccess;
  p.n_tiles = (uint32_t)(rate_bytes(p.n) / kTileBlocks);
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  p.use_tma = 0;
  if (op != kOpAddStream) {
    // int32 deltas are stored in whole blocks; fp32 data may end in a ragged row
    uint64_t rows = op == kOpAddI32 ? num_blocks(p.n) : p.n / kBlock;
    p.use_tma = make_rows_map(&map, p.local, rows) ? 1u : 0u;
  }
  int grid = grid_for_tiles(p.n_tiles, 2);
  switch (op) {
    case kOpCompress: return launch_encode_m<kOpCompress>(mode, map, p, grid, stream);
    case kOpAddF32: return launch_encode_m<kOpAddF32>(mode, map, p, grid, stream);
    case kOpAddI32: return launch_encode_m<kOpAddI32>(mode, map, p, grid, stream);
    case kOpAddStream: return launch_encode_m<kOpAddStream>(mode, map, p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_decode(int mode, DecParams p, cudaStream_t stream) {
  if (p.n == 0) return cudaSuccess;
  p.n_tiles = (uint32_t)(rate_bytes(p.n) / kTileBlocks);
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  p.use_tma = make_rows_map(&map, p.out, p.n / kBlock) ? 1u : 0u;
  int grid = grid_for_tiles(p.n_tiles, 2);
  switch (mode) {
    case kModeOutlier:
    case kModePlain: return launch_decode_t<kModeOutlier>(map, p, grid, stream);
    case kModeVec: return launch_decode_t<kModeVec>(map, p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_quant_pred(int mode, const float* x, int32_t* deltas, uint64_t n, float eb, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t n_padded = num_blocks(n) * kBlock;
  int grid = (int)((n_padded + 255) / 256 < 148ull * 16 ? (n_padded + 255) / 256 : 148ull * 16);
  float recip = 0.5f / eb;
  if (mode == kModeVec) dev::hc_quant_pred_kernel<kModeVec><<<grid, 256, 0, stream>>>(x, deltas, n, n_padded, recip);
  else dev::hc_quant_pred_kernel<kModeOutlier><<<grid, 256, 0, stream>>>(x, deltas, n, n_padded, recip);
  return cudaGetLastError();
}

cudaError_t launch_sum(float* dst, const float* a, const float* b, const float* c, const float* d, uint64_t n,
                       cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t want = (n / 4 + 255) / 256 + 1;
  int grid = (int)(want < 148ull * 8 ? want : 148ull * 8);
  dev::hc_sum_kernel<<<grid, 256, 0, stream>>>(dst, a, b, c, d, n);
  return cudaGetLastError();
}

}  // namespace hc
