// Kernel bodies and host launchers of the sm_100a codec (see hc_kernels.cuh for the design).
#include "hc_kernels.cuh"

#include <stdio.h>

#include "hc_launch.h"

namespace hc {
namespace dev {

constexpr int kEncThreads = kComputeThreads + 64;  // + loader warp + scanner warp
constexpr int kDecThreads = kComputeThreads + 32;  // + loader warp
constexpr uint32_t kNoTile = 0xffffffffu;

constexpr int kMaxStages = 2;
constexpr int kRing = 8;  // tiles a CTA may have between "total known" and "payload copied out"
struct __align__(16) EncShared {
  uint64_t tma_full[kMaxStages];    // fp32 tile landed in stage s (or "nothing to fetch"); also hands over the ticket
  uint64_t stage_free[kMaxStages];  // every compute thread holds its row of the tile in registers: refill the stage
  uint64_t scan_done[kRing];        // tile total known: the scanner may start its look-back
  uint64_t base_ready[kRing];       // look-back of the tile finished: out_base / out_ok valid
  uint64_t in_full[2];              // input stream bytes + meta staged in buffer b
  uint64_t in_free[2];              // compute threads have decoded from buffer b
  uint32_t tile[8];                 // ring of tile tickets, written by the loader
  uint32_t tile_tma[8];             // 1 when a TMA load was issued for that ring slot
  uint32_t in_phase[2];             // 16-byte phase of the staged bytes in buffer b
  uint32_t in_end[2];               // 1: buffer b carries the end marker instead of a stream (ops with inputs)
  uint32_t out_tile[kRing];         // ticket of this CTA's k-th tile (kNoTile: end of work), slot k % kRing
  uint32_t out_tot[kRing];          // its payload bytes
  uint32_t ring_start[kRing];       // where its payload starts in the ring
  uint32_t ring_end[kRing];         // first ring byte behind it
  uint32_t out_ok[kRing];           // 0: the tile is not to be stored (look-back failed, capacity exceeded)
  uint64_t out_base[kRing];         // byte offset of its payload in the output stream
  uint32_t wsum[2][kComputeThreads / 32];
  uint32_t copy_upto[2];            // turn k: tiles below copy_upto[k & 1] have their look-back result
  uint32_t stored_upto;             // tiles below it have been stored by every compute thread
  uint32_t abort;
  uint16_t in_rel[2][kTileBlocks];
  uint8_t in_rate[2][kTileBlocks];
};

__device__ __forceinline__ void note_error(uint32_t* ctrl, uint32_t code) { atomicMax(ctrl + 2, code); }
// timeouts and peer failures end the launch early; capacity / truncation errors only skip data
__device__ __forceinline__ bool fatal_error(const uint32_t* ctrl) {
  return *((volatile const uint32_t*)(ctrl + 2)) >= (uint32_t)kErrTimeout;
}

// Optional per-CTA timeline (compile with -DHC_TIMELINE): nanosecond stamps of the first tile's way
// through the roles (slots 0-15) and, for the first compute warp, SM-clock cycles accumulated per
// phase of the tile loop (slots 16-30) with the number of tiles in slot 31, for finding where a
// launch spends its time.  Not part of a normal build.
#ifdef HC_TIMELINE
constexpr int kTlSlots = 32;
__device__ unsigned long long g_timeline[4 * 1024 * kTlSlots];  // [launch epoch & 3][CTA][slot]
__device__ __forceinline__ unsigned long long timeline_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define HC_TL_DECL(epoch)                                                                                      \
  unsigned long long* const hc_tl =                                                                            \
      g_timeline + (((epoch)&3u) * 1024u + (blockIdx.x < 1024u ? blockIdx.x : 1023u)) * (unsigned)kTlSlots;     \
  long long hc_ph_t = 0
#define HC_TL_ZERO()                                \
  do {                                              \
    hc_tl[7] = hc_tl[14] = hc_tl[15] = 0;           \
    for (int i_ = 16; i_ < kTlSlots; ++i_) hc_tl[i_] = 0; \
  } while (0)
#define HC_STAMP(i) hc_tl[i] = timeline_now()
#define HC_STAMP_MAX(i) atomicMax(&hc_tl[i], timeline_now())
#define HC_TIC() const unsigned long long hc_tic = timeline_now()
#define HC_TOC(i) hc_tl[i] += timeline_now() - hc_tic
// phase accounting of one thread: HC_PH_START() once, then HC_PH(i) charges the cycles since the
// previous mark to phase i
#define HC_PH_START() hc_ph_t = clock64()
#define HC_PH(i)                                  \
  do {                                            \
    const long long now_ = clock64();             \
    hc_tl[16 + (i)] += (unsigned long long)(now_ - hc_ph_t); \
    hc_ph_t = now_;                               \
  } while (0)
#define HC_PH_COUNT() hc_tl[kTlSlots - 1] += 1
#else
#define HC_TL_DECL(epoch)
#define HC_TL_ZERO()
#define HC_STAMP(i)
#define HC_STAMP_MAX(i)
#define HC_TIC()
#define HC_TOC(i)
#define HC_PH_START()
#define HC_PH(i)
#define HC_PH_COUNT()
#endif

// the last CTA to leave re-arms the ticket counter for the next launch
// (returns true in thread 0 of that CTA)
__device__ __forceinline__ bool cta_epilogue(uint32_t* tick) {
  __syncthreads();
  bool last = false;
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(tick + 1, 1u);
    if (done == gridDim.x - 1) {
      tick[0] = 0;
      tick[1] = 0;
      __threadfence();
      last = true;
    }
  }
  return last;
}

// bounded mbarrier wait that records a timeout
// `site` says which wait it was; the first one to run out is kept in ctrl[3] (hc_codec_status_site),
// because every later time-out of the launch is only a consequence of it
enum WaitSite : uint32_t {
  kSiteLoaderStageFree = 1, kSiteLoaderInFree = 2, kSiteComputeInFull = 3, kSiteComputeTile = 4, kSiteComputeRing = 5,
  kSiteScannerTotal = 6, kSiteCopierBase = 7, kSiteCopierPacked = 8, kSiteDecodeInFree = 9, kSiteDecodeInFull = 10,
};
__device__ __forceinline__ bool wait_or_flag(uint64_t* bar, uint32_t parity, const Workspace& ws, volatile uint32_t* abort,
                                             uint32_t site) {
  if (mbar_wait_bounded(bar, parity, ws.spin_limit_ns)) return true;
  if (!*abort) atomicCAS(ws.ctrl + 3, 0u, site);
  note_error(ws.ctrl, kErrTimeout);
  *abort = 1;
  return false;
}

// Loader-warp work for one input stream, in two parts so that the rate bytes of the NEXT tile are
// already in flight while the look-back of the current one polls:
//   loader_fetch_rates   issues the loads of the tile's 128 rate bytes (4 per lane);
//   loader_stage_stream  per-block offsets -> tile aggregate published -> look-back -> (wait until
//                        the staging buffer is free) -> meta to shared memory -> one bulk copy of
//                        the tile's payload bytes into `cbuf` (16-byte phase preserved); arrives on
//                        `full`.
// The aggregate is published before the wait for the buffer, so a ticket never sits without its
// aggregate while this CTA's compute warps are busy.
constexpr int kRatesPerLane = kTileBlocks / 32;
__device__ __forceinline__ void loader_fetch_rates(const uint8_t* in, uint64_t in_size, uint32_t tile,
                                                   uint32_t (&rate)[kRatesPerLane]) {
  const int lane = threadIdx.x & 31;
  const uint64_t b0 = (uint64_t)tile * kTileBlocks + (uint64_t)lane * kRatesPerLane;
#pragma unroll
  for (int k = 0; k < kRatesPerLane; ++k) rate[k] = (b0 + k < in_size) ? ld_cg_u8(in + b0 + k) : 0u;
}

__device__ __forceinline__ void loader_stage_stream(const uint8_t* in, uint64_t in_size, uint64_t nrate, uint32_t tile,
                                                    const Chain& st, const Workspace& ws, uint8_t* cbuf, uint64_t* full,
                                                    uint16_t* s_rel, uint8_t* s_rate, uint32_t* s_phase, bool usable,
                                                    const uint32_t (&rate_in)[kRatesPerLane], uint64_t* free_bar,
                                                    uint32_t free_parity, bool wait_free, volatile uint32_t* abort,
                                                    bool base_known = false, uint64_t base_given = 0) {
  const int lane = threadIdx.x & 31;
  constexpr int kPer = kRatesPerLane;
  uint32_t rate[kPer], len[kPer], sum = 0;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    rate[k] = usable ? rate_in[k] : 0u;
    len[k] = payload_len(rate[k]);
    sum += len[k];
  }
  const uint32_t inc = warp_inclusive_scan(sum, lane);
  const uint32_t tot = __shfl_sync(0xffffffffu, inc, 31);
  // collective steps: the producer's arrival flag carries the tile's byte offset, no look-back
  bool ok = true;
  uint64_t base = base_given;
  if (!base_known) base = nrate + lookback(st, tile, ws.epoch, tot, ws.spin_limit_ns, ws.ctrl + 2, &ok);
  ok = ok && usable;
  if (ok && tot && base + tot > in_size) {  // stream shorter than its rate bytes imply
    if (lane == 0) note_error(ws.ctrl, kErrTruncated);
    ok = false;
  }
  // the staging buffer (bytes and meta) is free once the compute threads have decoded its previous tile
  if (wait_free && !wait_or_flag(free_bar, free_parity, ws, abort, kSiteLoaderInFree)) ok = false;
  uint32_t rel = inc - sum;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    s_rel[lane * kPer + k] = (uint16_t)rel;
    s_rate[lane * kPer + k] = ok ? (uint8_t)rate[k] : (uint8_t)0;
    rel += len[k];
  }
  const uint8_t* src = in + base;
  const uint32_t phase = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15u);
  if (lane == 0) *s_phase = phase;
  __syncwarp();
  if (lane == 0) {
    if (ok && tot) {
      const uint32_t bytes = (phase + tot + 15u) & ~15u;
      fence_proxy_async();
      mbar_expect_tx(full, bytes);
      bulk_load(cbuf, src - phase, bytes, full);
    } else {
      mbar_arrive(full);
    }
  }
}

// collective steps: one non-blocking look at the tile's arrival flag; 0 = not raised yet
__device__ __forceinline__ uint64_t flag_peek(const uint64_t* flag, uint32_t call) {
  uint64_t w = 0;
  if ((threadIdx.x & 31) == 0) {
    w = ld_acquire_sys_u64(flag);
    if (!flag_matches(w, call)) w = 0;
  }
  return __shfl_sync(0xffffffffu, w, 0);
}
// collective steps: bounded wait for the tile's arrival flag; 0 = the peer never delivered
__device__ __forceinline__ uint64_t flag_wait_warp(const uint64_t* flag, uint32_t call, const Workspace& ws) {
  uint64_t w = 0;
  if ((threadIdx.x & 31) == 0) {
    w = wait_tile_flag(flag, call, ws.spin_limit_ns, ws.ctrl + 2);
    if (w == 0) note_error(ws.ctrl, kErrPeer);
  }
  return __shfl_sync(0xffffffffu, w, 0);
}

// Shared-memory plan of the stream-producing kernel (offsets from a 1024-byte aligned base):
//   [1 KB guard | NS fp32 stages of 16 KB | payload ring + 64 guard bytes | cbuf 0 | cbuf 1]
// A stage receives the fp32 tile from the TMA unit and is free again as soon as every compute thread
// holds its row in registers.  The packed payload of a tile goes into the RING: a byte ring in which
// every tile takes just the bytes it needs (about 5 KB of the 16 KB at ratio 3.4), so that several
// packed tiles can wait there for their look-back while the compute warps go on with the next tiles.
// The scanner warp moves a tile from the ring to its final byte offset once the offset is known.
// A tile's look-back waits for the slowest of several hundred predecessor tiles; with the payload
// parked in the fp32 stage the compute warps of every CTA spent 35-50 % of their time waiting for it.
// In the IN-PLACE variant (one stage, ring = that stage, 54 KB: four CTAs per SM instead of three for
// the adds) a tile is packed over its own fp32 data and the stage is refilled after the copy-out:
// for launches with about one tile per CTA (the reduce step of a collective over many ranks).
constexpr int kRingBytesCompress = 19392;  // 4 CTAs per SM
constexpr int kRingBytesAdd = 17920;       // 3 CTAs per SM (shared memory is handed out in 1 KB steps)
constexpr int kRingBytesInPlace = kTileBytes + 32;
__host__ __device__ constexpr int enc_stages(int op) { return op == kOpCompress ? 2 : 1; }
__host__ __device__ constexpr int enc_ring_bytes(int op, bool inplace) {
  return inplace ? kRingBytesInPlace : (op == kOpCompress ? kRingBytesCompress : kRingBytesAdd);
}
// offset of the ring, and of the first staging buffer behind it
__host__ __device__ constexpr int enc_ring_off(int ns, bool inplace) { return inplace ? 1024 : 1024 + ns * kTileBytes + 16; }
__host__ __device__ constexpr int enc_cbuf_off(int op, int ns, bool inplace) {
  return inplace ? 1024 + kTileBytes + 1024 : enc_ring_off(ns, false) + enc_ring_bytes(op, false) + 48;
}
static_assert(kRingBytesCompress >= kTileBytes + 32 && kRingBytesAdd >= kTileBytes + 32, "a tile of 128-byte blocks must fit");

template <int OP, int MODE, int NS, bool INPLACE>
__global__ void __launch_bounds__(kEncThreads, (OP == kOpCompress || INPLACE) ? 4 : 3)
hc_encode_kernel(const __grid_constant__ TensorMaps tmaps, const EncParams p) {
  static_assert(NS <= kMaxStages && (!INPLACE || NS == 1), "stage count");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ EncShared sh;
  constexpr bool kHasLocal = OP != kOpAddStream;
  constexpr bool kHasIn = OP != kOpCompress;
  constexpr uint32_t kRingBytes = (uint32_t)enc_ring_bytes(OP, INPLACE);
  uint8_t* const stage0 = smem + 1024;
  uint8_t* const ring = smem + enc_ring_off(NS, INPLACE);
  uint8_t* cbuf[2] = {smem + enc_cbuf_off(OP, NS, INPLACE), smem + enc_cbuf_off(OP, NS, INPLACE) + kBufBytes};

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const Workspace& ws = p.ws;
  HC_TL_DECL(ws.epoch);
  const uint32_t Q = kHasIn ? p.n_in : 0u;  // input streams summed into every tile
  const uint32_t groups_per_seg = p.tiles_per_seg / 32 + 1;

  // what a role needs to know about the segment a tile belongs to
  struct Seg {
    uint32_t g, lt;      // segment, tile inside the segment
    uint64_t n, nrate;   // values and rate bytes of the segment
    uint64_t full_rows;  // rows the tensor map covers (int32 deltas come in whole blocks)
    uint64_t n_local;    // readable 4-byte values of the local operand
  };
  auto seg_of = [&](uint32_t tile) -> Seg {
    Seg v;
    // tickets go round the segments (ticket t: tile t / n_seg of segment t % n_seg), so that all the
    // streams of a launch grow at the same pace and their consumers can start on every one of them early
    v.lt = p.n_seg > 1 ? tile / p.n_seg : tile;
    v.g = p.n_seg > 1 ? tile - v.lt * p.n_seg : 0u;
    v.n = p.n[v.g];
    v.nrate = rate_bytes(v.n);
    v.full_rows = OP == kOpAddI32 ? num_blocks(v.n) : v.n / kBlock;
    v.n_local = OP == kOpAddI32 ? num_blocks(v.n) * kBlock : v.n;
    return v;
  };
  // destinations of a tile: every destination of the single segment, or the segment's own one
  auto dst_first = [&](const Seg& v) -> uint32_t { return p.n_seg > 1 ? v.g : 0u; };
  auto dst_count = [&](const Seg&) -> uint32_t { return p.n_seg > 1 ? 1u : p.n_dst; };

  if (tid == 32 && kHasLocal) {  // descriptor of the segment this CTA's first tile belongs to
    const uint32_t g0 = p.n_seg > 1 ? blockIdx.x % p.n_seg : 0u;
    if (p.use_tma[g0]) tma_prefetch_map(&tmaps.m[g0]);
  }
  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&sh.tma_full[i], 1);
      mbar_init(&sh.stage_free[i], kComputeThreads);
    }
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&sh.scan_done[i], 1);
      mbar_init(&sh.base_ready[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.in_full[i], 1);
      mbar_init(&sh.in_free[i], kComputeThreads);
    }
    fence_mbar_init();
    sh.abort = fatal_error(ws.ctrl) ? 1u : 0u;
    HC_TL_ZERO();
    launch_dependents();  // a following launch with programmatic serialisation may fill the SMs as CTAs leave
    sh.in_end[0] = sh.in_end[1] = 0u;
    sh.stored_upto = 0u;
  }
  __syncthreads();
  volatile uint32_t* abort = &sh.abort;
  if (tid == 0) HC_STAMP(0);

  if (warp == kComputeThreads / 32) {
    // ================================ loader warp ================================================
    // Tiles: CTA i starts with tile i (no round trip, and a CTA that starts late, behind a launch
    // that is still draining, finds its tile waiting instead of taken by an early starter); the
    // tiles past the grid come from a shared ticket counter.  Software pipeline over this CTA's
    // tiles: the ticket is taken two turns ahead and the rate bytes of the next input tile one
    // turn ahead, so neither round trip sits between two stagings.  Per tile: the input streams
    // first, then the fp32 tile's TMA load once its stage is free.
    // Input stream q of this CTA's k-th tile is staging job v = k * Q + q: buffer v & 1.
    auto take = [&]() -> uint32_t {
      uint32_t t = kNoTile;
      if (lane == 0 && !*abort) t = gridDim.x + atomicAdd(ws.tick, 1u);
      t = __shfl_sync(0xffffffffu, t, 0);
      return t < p.n_tiles ? t : kNoTile;
    };
    // non-blocking; fw receives the tile's arrival flag word when the stream has flags
    auto try_fetch = [&](uint32_t t, uint32_t q, uint32_t (&r)[kRatesPerLane], uint64_t& fw) -> bool {
      if (!kHasIn || t == kNoTile) return false;
      fw = 0;
      if (p.in_ready[q] && (fw = flag_peek(p.in_ready[q] + t, p.ring_epoch)) == 0) return false;
      loader_fetch_rates(p.in[q], p.in_size[q], t, r);
      return true;
    };
    uint32_t tile = (!*abort && blockIdx.x < p.n_tiles) ? blockIdx.x : kNoTile;
    if (lane == 0) HC_STAMP(1);
    uint32_t tile_n = tile != kNoTile ? take() : kNoTile;
    uint32_t rates[kRatesPerLane] = {}, rates_n[kRatesPerLane] = {};
    uint64_t fw = 0, fw_n = 0;  // arrival flag words that came with the prefetched rate bytes
    bool have = try_fetch(tile, 0, rates, fw), have_n = false;
    for (uint32_t k = 0;; ++k) {
      const int s = k % NS, slot = k & 7;
      const uint32_t tile_nn = (tile != kNoTile && tile_n != kNoTile) ? take() : kNoTile;
      // staging job q of this tile (input stream q -> buffer (k * Q + q) & 1)
      auto stage_job = [&](uint32_t q) {
        const uint64_t nrate = rate_bytes(p.n[0]);
        const uint32_t v = k * Q + q, b = v & 1u, u = v >> 1;
        // next staging job: the next stream of this tile, or the first stream of the next tile
        const bool last_q = q + 1 == Q;
        have_n = try_fetch(last_q ? tile_n : tile, last_q ? 0u : q + 1, rates_n, fw_n);
        bool usable = true;
        if (!have) {
          fw = 0;
          HC_TIC();
          if (p.in_ready[q] && (fw = flag_wait_warp(p.in_ready[q] + tile, p.ring_epoch, ws)) == 0) usable = false;
          if (lane == 0) HC_TOC(14);
          if (usable) loader_fetch_rates(p.in[q], p.in_size[q], tile, rates);
        }
        const bool flagged_in = p.in_ready[q] != nullptr;
        if (flagged_in && (fw & kFlagOffsetMask) == kFlagOffsetMask) usable = false;  // the producer gave up
        const Chain chain{ws.st_a + (size_t)q * p.tiles_per_seg, ws.grp_a + (size_t)q * groups_per_seg};
        loader_stage_stream(p.in[q], p.in_size[q], nrate, tile, chain, ws, cbuf[b], &sh.in_full[b], sh.in_rel[b],
                            sh.in_rate[b], &sh.in_phase[b], usable, rates, &sh.in_free[b], (u - 1) & 1, u >= 1, abort,
                            flagged_in, fw & kFlagOffsetMask);
        have = have_n;
        fw = fw_n;
#pragma unroll
        for (int i = 0; i < kRatesPerLane; ++i) rates[i] = rates_n[i];
      };
      // hand-over: the fp32 tile's TMA load into stage s (free once the compute threads hold the
      // rows of the tile that came in NS turns ago; in place: once that tile has been copied out)
      // and the ticket for the compute warps
      auto hand_over = [&]() -> uint32_t {
        uint32_t t_stage = tile;
        if (k >= NS && !wait_or_flag(&sh.stage_free[s], ((k / NS) - 1) & 1, ws, abort, kSiteLoaderStageFree)) t_stage = kNoTile;
        if (lane == 0) {
          sh.tile[slot] = t_stage;
          bool fetch = false;
          if (kHasLocal && t_stage != kNoTile) {
            const Seg v = seg_of(t_stage);
            fetch = p.use_tma[v.g] && (uint64_t)v.lt * kTileBlocks < v.full_rows;
            if (fetch) {
              fence_proxy_async();
              mbar_expect_tx(&sh.tma_full[s], kTileBytes);
              tma_load_2d(stage0 + s * kTileBytes, &tmaps.m[v.g], 0, (int)(v.lt * kTileBlocks), &sh.tma_full[s]);
            }
          }
          sh.tile_tma[slot] = fetch ? 1u : 0u;
          if (!fetch) mbar_arrive(&sh.tma_full[s]);
        }
        return t_stage;
      };
      if (kHasIn && tile == kNoTile) {
        // end of work: the compute warps look at the staging buffer first, so the marker goes there
        const uint32_t v = k * Q, b = v & 1u, u = v >> 1;
        if (u >= 1) wait_or_flag(&sh.in_free[b], (u - 1) & 1, ws, abort, kSiteLoaderInFree);
        if (lane == 0) {
          sh.tile[slot] = kNoTile;
          sh.in_end[b] = 1u;
          mbar_arrive(&sh.in_full[b]);
        }
      }
      // The first NS tiles find their stage free: their TMA load goes out before anything else.
      // Afterwards the first two input streams go in first (their buffers only depend on earlier
      // tiles).  Later streams reuse a buffer that the compute warps free while decoding THIS
      // tile's first streams.
      uint32_t t_stage = kNoTile;
      const bool early = k < (uint32_t)NS;
      // With a single stage the hand-over waits for the compute warps to have read the previous tile,
      // which they do after decoding ALL of its streams: every stream of this tile goes in first then.
      const uint32_t before = (NS == 1 && !early) ? Q : 2u;
      if (early) t_stage = hand_over();
      if (kHasIn && tile != kNoTile)
        for (uint32_t q = 0; q < Q && q < before; ++q) stage_job(q);
      if (!early) t_stage = hand_over();
      if (t_stage == kNoTile) break;
      if (kHasIn)
        for (uint32_t q = before; q < Q; ++q) stage_job(q);
      tile = tile_n;
      tile_n = tile_nn;
    }
    if (lane == 0) HC_STAMP(6);
  } else if (warp == kComputeThreads / 32 + 1) {
    // ================================ scanner warp ===============================================
    // runs the decoupled look-back of the output stream as soon as a tile's total is known, while the
    // compute warps are still transposing and packing, and hands them the tile's byte offset.  Every
    // other CTA's look-back waits for the words this warp publishes, so it does nothing that could
    // queue in front of a look-back, with one exception that has slack: in a collective step it
    // raises the consumers' arrival flags for the tiles the compute warps report as stored
    // (sh.stored_upto, written behind a barrier that follows the stores).  One system-scope fence
    // covers a batch of tiles: it waits for the peers' write acknowledgements, several microseconds
    // over NVLink.
    constexpr uint32_t kFlagBatch = 4;
    const bool raise = p.out_ready[0] != nullptr;  // this launch is a step of a collective
    uint32_t flagged = 0;                           // tiles [0, flagged) of this CTA have been announced
    uint32_t my_lt = 0, my_g = 0;                   // lane (j & 31) remembers this CTA's j-th tile
    uint64_t my_word = 0;
    auto raise_flags = [&](uint32_t upto) {  // tiles [flagged, upto) have left for their destinations
      if (!raise || upto <= flagged) return;
      HC_TIC();
      fence_acq_rel_sys();
      if (lane == 0) HC_TOC(15);
      if (((uint32_t)lane - flagged) % 32u < upto - flagged) {
        const uint32_t d0 = p.n_seg > 1 ? my_g : 0u, dn = p.n_seg > 1 ? 1u : p.n_dst;
        for (uint32_t dsti = 0; dsti < dn; ++dsti) {
          uint64_t* flags = p.out_ready[d0 + dsti];
          if (flags) st_relaxed_sys_u64(flags + my_lt, my_word);
        }
      }
      flagged = upto;
    };
    if (lane == 0) HC_PH_START();
    for (uint32_t k = 0;; ++k) {
      const int r = k % kRing;
      const uint32_t par = (k / kRing) & 1;
      if (!wait_or_flag(&sh.scan_done[r], par, ws, abort, kSiteScannerTotal)) break;
      if (lane == 0) HC_PH(10);
      const uint32_t tile = sh.out_tile[r];
      const uint32_t stored = *((volatile uint32_t*)&sh.stored_upto);  // written before scan_done was raised
      if (tile == kNoTile) {
        if (lane == 0) HC_STAMP(13);
        raise_flags(stored);  // the compute warps have stored every tile before they send the end marker
        if (lane == 0) HC_STAMP(9);
        break;
      }
      const Seg v = seg_of(tile);
      const uint32_t tot = sh.out_tot[r];
      bool ok = true;
      uint64_t excl;
      if (p.sparse) {
        // transport buffer of a collective: every tile at the offset it would have if all blocks
        // before it were incompressible.  No prefix over other CTAs' tiles, hence no waiting; the
        // consumer takes the offset from the tile's arrival flag.  Payload bytes are summed for the
        // statistics and turned into the length of the equivalent compact stream by the last CTA.
        excl = (uint64_t)v.lt * (uint64_t)(kTileBlocks * kMaxBlockPayload);
        if (lane == 0 && p.size_out) atomicAdd((unsigned long long*)(ws.size_acc + v.g), (unsigned long long)tot);
      } else {
        const Chain chain{ws.st_out + (size_t)v.g * p.tiles_per_seg, ws.grp_out + (size_t)v.g * groups_per_seg};
        excl = lookback(chain, v.lt, ws.epoch, tot, ws.spin_limit_ns, ws.ctrl + 2, &ok);
      }
      const uint64_t goff = v.nrate + excl;
      if (k == 0 && lane == 0) HC_STAMP(4);
      if (ok && tot && goff + tot > p.out_cap) {  // (a tile without payload stores nothing, wherever it would go)
        if (lane == 0) note_error(ws.ctrl, kErrCapacity);
        ok = false;
      }
      if (lane == 0) {
        sh.out_base[r] = goff;
        sh.out_ok[r] = ok ? 1u : 0u;
        mbar_arrive(&sh.base_ready[r]);
        // the last tile ends where the stream ends: no size for a stream that did not fit
        if (!p.sparse && ok && v.lt == p.tiles_per_seg - 1 && p.size_out && goff + tot <= p.out_cap) p.size_out[v.g] = goff + tot;
        if (fatal_error(ws.ctrl)) *abort = 1;
        HC_PH(11);
      }
      if ((uint32_t)lane == (k & 31u)) {
        my_lt = v.lt;
        my_g = v.g;
        my_word = flag_pack(p.ring_epoch, ok ? goff : kFlagOffsetMask);
      }
      if (stored - flagged >= kFlagBatch) raise_flags(stored);
    }
  } else {
    // ================================ compute warps ==============================================
    if (tid == 0) HC_PH_START();
    uint32_t head = 0;    // next free ring byte (same value in every compute thread)
    uint32_t copied = 0;  // this CTA's tiles [0, copied) have been moved out of the ring (same in every thread)
    // all compute threads: tile number j of this CTA -> global memory (its look-back must have finished)
    auto copy_tile = [&](uint32_t j) {
      const int rj = j % kRing;
      const Seg v = seg_of(sh.out_tile[rj]);
      if (sh.out_ok[rj])
        copy_out(ring + sh.ring_start[rj], p.out + dst_first(v), dst_count(v), sh.out_base[rj], sh.out_tot[rj],
                 (uint32_t)tid, (uint32_t)kComputeThreads, p.n_seg == 1 ? p.out_mc : nullptr);
    };
    // blocking: tiles [copied, upto) out, whatever their look-backs take
    auto drain_to = [&](uint32_t upto) {
      for (uint32_t j = copied; j < upto; ++j) {
        wait_or_flag(&sh.base_ready[j % kRing], (j / kRing) & 1, ws, abort, kSiteComputeRing);
        copy_tile(j);
      }
      copied = upto > copied ? upto : copied;
    };
    for (uint32_t k = 0;; ++k) {
      const int s = k % NS, slot = k & 7, r = k % kRing;
      uint8_t* const stage_s = stage0 + s * kTileBytes;
      int32_t d[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) d[i] = 0;

      // ---- incoming stream(s) -> signed deltas, summed -------------------------------------------
      bool end = false;
      if (kHasIn) {
        for (uint32_t q = 0; q < Q; ++q) {
          const uint32_t vv = k * Q + q, b = vv & 1u;
          const bool staged = wait_or_flag(&sh.in_full[b], (vv >> 1) & 1, ws, abort, kSiteComputeInFull);
          if (tid == 0) HC_PH(0);
          if (q == 0 && (!staged || sh.in_end[b])) {
            end = true;  // no tile this turn (or the loader gave up)
            break;
          }
          const uint32_t rate_in = staged ? sh.in_rate[b][tid] : 0u;
          const uint32_t pos = sh.in_phase[b] + sh.in_rel[b][tid];
          int W = plane_width(rate_in & 31u);
          W = __reduce_max_sync(0xffffffffu, W);
          if (__any_sync(0xffffffffu, rate_in != 0)) {
            int32_t d2[32];
            decode_block(cbuf[b], pos, rate_in, W, d2);
#pragma unroll
            for (int i = 0; i < 32; ++i) d[i] += d2[i];
          }
          mbar_arrive(&sh.in_free[b]);
          if (tid == 0) HC_PH(1);
          if (k == 0 && tid == 0 && q < 8) HC_STAMP(8 + q);
        }
      }
      if (INPLACE && k >= 1 && !end) {
        // the tile packed over the fp32 stage has to leave before the next fp32 tile can come in
        compute_barrier();  // every thread has packed tile k-1
        drain_to(k);
        mbar_arrive(&sh.stage_free[0]);
      }
      const bool alive = !end && wait_or_flag(&sh.tma_full[s], (k / NS) & 1, ws, abort, kSiteComputeTile);
      if (tid == 0) HC_PH(2);
      if (k == 0 && tid == 0) HC_STAMP(2);
      const uint32_t tile = alive ? sh.tile[slot] : kNoTile;
      if (tile == kNoTile) {
        // end of work: everything still in the ring leaves, then the scanner hears of the end through
        // the same barrier as of a tile
        compute_barrier();  // every thread has packed the last tile
        if (tid == 0) HC_STAMP(5);
        drain_to(k);
        if (tid == 0) HC_STAMP(12);
        if (INPLACE && k >= 1) mbar_arrive(&sh.stage_free[0]);  // the loader's last hand-over waits for it
        compute_barrier();  // every thread's stores are issued before the scanner announces them
        if (tid == 0) {
          sh.stored_upto = k;
          sh.out_tile[r] = kNoTile;
          mbar_arrive(&sh.scan_done[r]);
        }
        break;
      }
      const Seg v = seg_of(tile);

      // ---- local operand -------------------------------------------------------------------------
      if (kHasLocal) {
        uint32_t w[32];
        const uint64_t row = (uint64_t)v.lt * kTileBlocks + tid;
        if (p.use_tma[v.g]) {
          if (sh.tile_tma[slot]) {
            load_row_swizzled(stage_s, tid, w);  // rows past the map were zero-filled by the TMA unit
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) w[i] = 0;
          }
          // the ragged last row of fp32 data is not part of the tensor map
          if (OP != kOpAddI32 && row * kBlock < v.n && (row + 1) * kBlock > v.n)
            load_row_global((const uint32_t*)p.local[v.g], v.n, row, w);
        } else {
          load_row_global((const uint32_t*)p.local[v.g], v.n_local, row, w);
        }
        if (!INPLACE) mbar_arrive(&sh.stage_free[s]);  // this thread's row is in registers
        if (OP == kOpAddI32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) d[i] += (int32_t)w[i];
        } else {
          int32_t q[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) q[i] = quantise(__uint_as_float(w[i]), p.recip);
          int32_t dl[32];
          lorenzo_forward<MODE>(q, dl);
#pragma unroll
          for (int i = 0; i < 32; ++i) d[i] += dl[i];
        }
      } else if (!INPLACE) {
        mbar_arrive(&sh.stage_free[s]);
      }

      // ---- encode ----------------------------------------------------------------------------------
      if (tid == 0) HC_PH(3);
      uint32_t A[32];
      BlockCode code = analyse_block<MODE>(d, A);
      uint32_t tot;
      if (tid == 0) {
        HC_PH(4);
        // which of the packed tiles have their look-back result by now (no waiting); everybody reads
        // the answer behind the barrier of the scan, so all threads copy the same tiles this turn
        uint32_t n = copied;
        while (n < k && mbar_try_wait(&sh.base_ready[n % kRing], (n / kRing) & 1)) ++n;
        sh.copy_upto[k & 1] = n;
      }
      // the barrier inside the scan also orders: the packing of tile k-1 before its copy-out below, the
      // stores of earlier turns before `stored_upto` is seen by the scanner, and (in place) the last
      // read of the fp32 tile before the first write of the packed payload over it
      const uint32_t rel = compute_exclusive_scan(code.len, sh.wsum[k & 1], &tot);
      if (tid == 0) HC_PH(8);
      uint32_t upto = sh.copy_upto[k & 1];
      // ring bytes of this tile: [start, end), 16-byte aligned, never across the end of the ring;
      // every compute thread does the same arithmetic.  `dep` is the newest earlier tile that must
      // have left first: one whose bytes overlap, or the one kRing - 1 tiles back (slots of the
      // per-tile words and barriers).
      uint32_t start = head, end_b = head + ((tot + 15u) & ~15u) + 16u;
      if (INPLACE || end_b > kRingBytes) {
        start = 0;
        end_b = ((tot + 15u) & ~15u) + 16u;
      }
      head = end_b;
      int dep = (int)k - (kRing - 1);
      if (!INPLACE) {
#pragma unroll
        for (int back = 1; back < kRing - 1; ++back) {
          const int j = (int)k - back;
          if (j > dep && j >= 0 && sh.ring_start[j % kRing] < end_b && start < sh.ring_end[j % kRing]) dep = j;
        }
      }
      if (tid == 0) {
        // publish the tile aggregate right away: successors can look back through this tile
        if (v.lt != 0 && !p.sparse)
          st_relaxed_gpu_u64(ws.st_out + (size_t)v.g * p.tiles_per_seg + v.lt, st_pack(kStAgg, ws.epoch, tot));
        // every thread is past this turn's barrier, so its stores of the tiles copied in earlier turns
        // are issued: the scanner may announce them (it reads this after the arrival below)
        sh.stored_upto = copied;
        // slot r was last used kRing tiles ago, by a tile that left the ring at least a turn ago
        sh.out_tile[r] = tile;
        sh.out_tot[r] = tot;
        sh.ring_start[r] = start;
        sh.ring_end[r] = end_b;
        mbar_arrive(&sh.scan_done[r]);
        if (k == 0) HC_STAMP(3);
      }
      // rate bytes (section A) go straight to every destination; a segment shorter than the longest
      // one of the launch has tickets past its own section A, which must not touch its payload
      if ((uint64_t)v.lt * kTileBlocks < v.nrate) {
        const uint64_t bidx = (uint64_t)v.lt * kTileBlocks + tid;
        const uint32_t d0 = dst_first(v), dn = dst_count(v);
#pragma unroll 1
        for (uint32_t dsti = 0; dsti < dn; ++dsti) p.out[d0 + dsti][bidx] = (uint8_t)code.rate;
      }
      int W = plane_width(code.rate & 31u);
      W = __reduce_max_sync(0xffffffffu, W);
      transpose_forward(A, W);
      if (tid == 0) HC_PH(9);
      if (!INPLACE) {
        // packed tiles whose offset is known leave now; the ones this tile needs the room of leave
        // whatever their look-back takes
        const bool overlap_now = dep >= (int)copied;  // a tile this one is packed over leaves in this turn
        if (dep >= (int)upto) upto = (uint32_t)dep + 1u;
        drain_to(upto);
        if (tid == 0) HC_PH(6);
        if (overlap_now) compute_barrier();  // nobody still reads the bytes that this tile is packed over
      }
      write_payload(ring + start, rel, code, A, W);
      if (tid == 0) {
        HC_PH(7);
        HC_PH_COUNT();
      }
    }
  }
  if (lane == 0) HC_STAMP_MAX(7);
  if (cta_epilogue(ws.tick) && p.sparse && p.size_out) {
    // every CTA has added its tiles' payload bytes (device-scope atomics, fenced before the exit count)
    for (uint32_t g = 0; g < p.n_seg; ++g) {
      p.size_out[g] = rate_bytes(p.n[g]) + ws.size_acc[g];
      ws.size_acc[g] = 0;
    }
  }
}

struct __align__(16) DecShared {
  uint64_t in_full[2];
  uint64_t in_free[2];
  uint32_t tile[4];
  uint32_t in_phase[2];
  uint32_t abort;
  uint16_t in_rel[2][kTileBlocks];
  uint8_t in_rate[2][kTileBlocks];
};

// SUM: the n_seg streams hold contributions to ONE array (every rank's whole message in the one-step
// form of the allreduce): a CTA stages tile lt of every stream in turn, adds the decoded quantised
// values in registers and writes seg[0].out once per tile.  Tickets then count tiles, not (tile, stream).
template <int MODE, bool SUM>
__global__ void __launch_bounds__(kDecThreads, SUM ? 3 : 4)
hc_decode_kernel(const __grid_constant__ TensorMaps tmaps, const DecParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ DecShared sh;
  // one output tile (its TMA store has a whole tile time to read it out) + two staging buffers:
  // 51 KB per CTA, four CTAs per SM
  uint8_t* const obuf = smem;
  uint8_t* cbuf[2] = {smem + kTileBytes, smem + kTileBytes + kBufBytes};

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const Workspace& ws = p.ws;
  HC_TL_DECL(ws.epoch);
  const float eb = p.eb;
  const uint32_t groups_per_seg = p.tiles_per_seg / 32 + 1;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.in_full[i], 1);
      mbar_init(&sh.in_free[i], kComputeThreads);
    }
    fence_mbar_init();
    sh.abort = fatal_error(ws.ctrl) ? 1u : 0u;
    HC_TL_ZERO();
    launch_dependents();  // a following launch with programmatic serialisation may fill the SMs as CTAs leave
  }
  __syncthreads();
  volatile uint32_t* abort = &sh.abort;
  if (tid == 0) HC_STAMP(0);

  if (warp == kComputeThreads / 32) {
    // ================================ loader warp ================================================
    // CTA i starts with tile i, later tiles come from the shared ticket counter.  Software pipeline
    // over this CTA's tiles: the ticket is taken two turns ahead and the rate bytes one turn ahead,
    // so neither round trip sits between two look-backs.
    uint32_t handed = kNoTile, handed_sg = 0;  // SUM: the (tile, stream) pair handed out last
    auto take = [&]() -> uint32_t {  // lane 0 takes a ticket, every lane gets it
      if (SUM && handed != kNoTile && handed_sg + 1 < p.n_seg) {
        ++handed_sg;
        return ++handed;  // the next stream of the same tile
      }
      uint32_t t = kNoTile;
      if (lane == 0 && !*abort) t = gridDim.x + atomicAdd(ws.tick, 1u);
      t = __shfl_sync(0xffffffffu, t, 0);
      if (!SUM) return t < p.n_tiles ? t : kNoTile;
      handed = t < p.tiles_per_seg ? t * p.n_seg : kNoTile;
      handed_sg = 0;
      return handed;
    };
    // non-blocking; fw receives the tile's arrival flag word when the segment has flags
    auto try_fetch = [&](uint32_t t, uint32_t (&r)[kRatesPerLane], uint64_t& fw) -> bool {
      if (t == kNoTile) return false;
      const uint32_t lt = t / p.n_seg, sg = t - lt * p.n_seg;  // tickets go round the segments
      const DecSegment& seg = p.seg[sg];
      fw = 0;
      // a segment shorter than the longest one of the launch has tickets past its own tiles: nothing to
      // wait for and nothing to read there (its producer never raises those flags)
      if ((uint64_t)lt * kTileBlocks >= rate_bytes(seg.n)) {
#pragma unroll
        for (int i = 0; i < kRatesPerLane; ++i) r[i] = 0u;
        return true;
      }
      if (seg.in_ready && (fw = flag_peek(seg.in_ready + lt, p.ring_epoch)) == 0) return false;
      loader_fetch_rates(seg.in, seg.in_size, lt, r);
      return true;
    };
    uint32_t tile = (!*abort && blockIdx.x < (SUM ? p.tiles_per_seg : p.n_tiles)) ? blockIdx.x : kNoTile;
    if (SUM && tile != kNoTile) tile = handed = tile * p.n_seg;
    if (lane == 0) HC_STAMP(1);
    uint32_t tile_n = tile != kNoTile ? take() : kNoTile;
    uint32_t rates[kRatesPerLane] = {}, rates_n[kRatesPerLane] = {};
    uint64_t fw = 0, fw_n = 0;
    bool have = try_fetch(tile, rates, fw), have_n = false;
    for (uint32_t k = 0;; ++k) {
      const int s = k & 1;
      if (tile == kNoTile) {
        // end marker; the buffer's previous phase must have been consumed before it is re-armed
        if (k >= 2) wait_or_flag(&sh.in_free[s], ((k >> 1) - 1) & 1, ws, abort, kSiteDecodeInFree);
        if (lane == 0) sh.tile[k & 3] = kNoTile;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.in_full[s]);
        break;
      }
      const uint32_t tile_nn = tile_n != kNoTile ? take() : kNoTile;
      have_n = try_fetch(tile_n, rates_n, fw_n);
      const uint32_t lt = tile / p.n_seg, sg = tile - lt * p.n_seg;
      const DecSegment& seg = p.seg[sg];
      bool usable = true;
      if (!have) {  // (tickets past the segment's own tiles always come back from try_fetch with `have`)
        fw = 0;
        if (seg.in_ready && (fw = flag_wait_warp(seg.in_ready + lt, p.ring_epoch, ws)) == 0) usable = false;
        if (usable) loader_fetch_rates(seg.in, seg.in_size, lt, rates);
      }
      const bool flagged_in = seg.in_ready != nullptr;
      if (flagged_in && (fw & kFlagOffsetMask) == kFlagOffsetMask) usable = false;  // the producer gave up
      const Chain chain{ws.st_a + (size_t)sg * p.tiles_per_seg, ws.grp_a + (size_t)sg * groups_per_seg};
      if (lane == 0) sh.tile[k & 3] = tile;  // ring of 4 > 2 buffers: nobody still reads this slot
      loader_stage_stream(seg.in, seg.in_size, rate_bytes(seg.n), lt, chain, ws, cbuf[s], &sh.in_full[s], sh.in_rel[s],
                          sh.in_rate[s], &sh.in_phase[s], usable, rates, &sh.in_free[s], ((k >> 1) - 1) & 1, k >= 2,
                          abort, flagged_in, fw & kFlagOffsetMask);
      if (lane == 0 && fatal_error(ws.ctrl)) *abort = 1;
      tile = tile_n;
      tile_n = tile_nn;
      have = have_n;
      fw = fw_n;
#pragma unroll
      for (int i = 0; i < kRatesPerLane; ++i) rates[i] = rates_n[i];
    }
    if (lane == 0) HC_STAMP(6);
  } else {
    // ================================ compute warps ==============================================
    if (tid == 0) HC_PH_START();
    int32_t acc[SUM ? 32 : 1];
    for (uint32_t k = 0;; ++k) {
      const int s = k & 1;
      bool alive = wait_or_flag(&sh.in_full[s], (k >> 1) & 1, ws, abort, kSiteDecodeInFull);
      if (tid == 0) HC_PH(0);
      if (k == 0 && tid == 0) HC_STAMP(2);
      const uint32_t tile = alive ? sh.tile[k & 3] : kNoTile;
      if (tile == kNoTile) break;
      const uint32_t lt = tile / p.n_seg, sg = tile - lt * p.n_seg;
      const DecSegment& seg = p.seg[SUM ? 0u : sg];  // where the tile goes
      const bool tma = seg.use_tma != 0;
      const uint64_t full_rows = seg.n / kBlock;
      const uint32_t rate = sh.in_rate[s][tid];
      const uint32_t pos = sh.in_phase[s] + sh.in_rel[s][tid];
      int W = plane_width(rate & 31u);
      W = __reduce_max_sync(0xffffffffu, W);
      int32_t d[32];
      if (__any_sync(0xffffffffu, rate != 0)) {
        decode_block_quant<MODE>(cbuf[s], pos, rate, W, d);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) d[i] = 0;
      }
      mbar_arrive(&sh.in_free[s]);
      if (SUM) {
        if (sg == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = d[i];
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] += d[i];
        }
        if (sg + 1 < p.n_seg) continue;  // more streams of this tile to come
#pragma unroll
        for (int i = 0; i < 32; ++i) d[i] = acc[i];
      }
      if (tid == 0) HC_PH(1);
      if (k == 0 && tid == 0) HC_STAMP(3);
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__fmul_rn(__fmul_rn((float)d[i], eb), 2.0f));

      const uint64_t row = (uint64_t)lt * kTileBlocks + tid;
      const bool ragged = row * kBlock < seg.n && (row + 1) * kBlock > seg.n;
      // the TMA store of the previous tile must have finished reading obuf
      if (tid == 0) HC_PH(2);
      if (tid == 0) tma_wait_group_read<0>();
      compute_barrier();
      if (tid == 0) HC_PH(3);
      if (tma) {
        store_row_swizzled(obuf, tid, w);
        fence_proxy_async();
      }
      compute_barrier();
      if (tid == 0) {
        HC_PH(4);
        HC_PH_COUNT();
        if (tma && (uint64_t)lt * kTileBlocks < full_rows)
          tma_store_2d(&tmaps.m[SUM ? 0u : sg], 0, (int)(lt * kTileBlocks), obuf);
        tma_commit_group();
        if (k == 0) HC_STAMP(5);
      }
      if (!tma || ragged) {
        const uint64_t o = row * kBlock;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (o + i < seg.n) seg.out[o + i] = __uint_as_float(w[i]);
      }
    }
    if (tid == 0) tma_wait_group<0>();
  }
  if (lane == 0) HC_STAMP_MAX(7);
  cta_epilogue(ws.tick);
}

// Pre-pass for the stand-alone stream consumers (decompress and the homomorphic adds on streams that
// no collective step has flagged): reads the rate bytes of up to kMaxIn streams and writes, for every
// tile, the byte offset of its payload in the arrival-flag format (dev::flag_pack(tag, offset)), so
// that the consuming kernel stages each tile straight from its flag word instead of walking a
// look-back chain over the input tile by tile.  One CTA covers kOffTiles tiles of one stream: each
// warp sums the payload lengths of 32 tiles (lane j ends up with tile j's total), the CTA scans its
// totals, warp 0 chains the CTA totals with the two-level look-back, then every thread publishes one
// flag word.  A 256 MB input has 2 MiB of rate bytes and 64 CTAs here: a few microseconds.
constexpr int kOffThreads = 256;
constexpr int kOffTiles = kOffThreads;  // tiles per CTA, one flag word per thread
__global__ void __launch_bounds__(kOffThreads) hc_offsets_kernel(const OffsetParams p) {
  __shared__ uint32_t s_wsum[kOffThreads / 32];
  __shared__ uint64_t s_base;
  __shared__ uint32_t s_ok;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t q = blockIdx.y, cta = blockIdx.x;
  const uint8_t* in = p.in[q];
  const uint64_t in_size = p.in_size[q];
  if (tid == 0) launch_dependents();  // the consumer may fill the SMs right away; it waits on the flags
  const uint32_t t0 = cta * kOffTiles + warp * 32;
  uint32_t mine = 0;
#pragma unroll 8
  for (int j = 0; j < 32; ++j) {
    const uint32_t t = t0 + j;
    uint32_t sum = 0;
    if (t < p.tiles_per_seg) {
      const uint64_t b0 = (uint64_t)t * kTileBlocks + (uint64_t)lane * 4;
      uint32_t r4 = 0;
      if (b0 + 4 <= in_size && (reinterpret_cast<uintptr_t>(in) & 3u) == 0) {
        r4 = __ldcg(reinterpret_cast<const uint32_t*>(in + b0));
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (b0 + k < in_size) r4 |= ld_cg_u8(in + b0 + k) << (8 * k);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) sum += payload_len((r4 >> (8 * k)) & 0xffu);
    }
    sum = __reduce_add_sync(0xffffffffu, sum);
    if (lane == j) mine = sum;
  }
  const uint32_t inc = warp_inclusive_scan(mine, lane);
  if (lane == 31) s_wsum[warp] = inc;
  __syncthreads();
  uint32_t pre = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kOffThreads / 32; ++w) {
    const uint32_t v = s_wsum[w];
    if (w < warp) pre += v;
    tot += v;
  }
  if (warp == 0) {
    const uint32_t n_cta = (p.tiles_per_seg + kOffTiles - 1) / kOffTiles;
    const uint32_t stride = n_cta + n_cta / 32 + 4;  // CTA words, then the words of their groups of 32
    const Chain chain{p.ws.grp_a + (size_t)q * stride, p.ws.grp_a + (size_t)q * stride + n_cta + 1};
    bool ok = true;
    const uint64_t excl = lookback(chain, cta, p.ws.epoch, tot, p.ws.spin_limit_ns, p.ws.ctrl + 2, &ok);
    if (lane == 0) {
      s_base = p.nrate + excl;
      s_ok = ok ? 1u : 0u;
    }
  }
  __syncthreads();
  const uint32_t t = cta * kOffTiles + tid;
  if (t < p.tiles_per_seg) {
    const uint64_t off = s_ok ? s_base + pre + (inc - mine) : kFlagOffsetMask;
    st_relaxed_sys_u64(p.flags[q] + t, flag_pack(p.tag, off));
  }
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

constexpr int enc_smem_bytes(int op, int ns, bool inplace) {
  return dev::enc_cbuf_off(op, ns, inplace) + (op == kOpCompress ? 0 : 2 * kBufBytes) + 1024;
}
constexpr int kDecSmem = kTileBytes + 2 * kBufBytes + 1024;

template <typename K>
cudaError_t set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// launch with programmatic stream serialisation (see launch_encode in hc_launch.h)
template <typename... Params, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(Params...), int grid, int block, int smem, cudaStream_t stream,
                              const Args&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  memset(&attr, 0, sizeof(attr));
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// CTAs of `kernel` that one GPU holds at the same time, asked of the runtime once per device.  The
// kernels are written for a grid that is resident as a whole (CTA i owns tile i, and every look-back
// waits for tiles held by other CTAs of the grid), so the grid is cut to this number, never assumed.
template <typename K>
int resident_ctas(K kernel, int threads, int smem, int* cache) {
  int dev = 0;
  cudaGetDevice(&dev);
  int& c = cache[dev & 63];
  if (c == 0) {
    if (set_smem(kernel, smem) != cudaSuccess) return 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, (size_t)smem) != cudaSuccess) return 0;
    c = per_sm * device_info().sms;
  }
  return c;
}

template <int OP, int MODE, bool INPLACE = false>
int encode_capacity() {
  constexpr int NS = INPLACE ? 1 : dev::enc_stages(OP);
  static thread_local int cache[64] = {};
  return resident_ctas(dev::hc_encode_kernel<OP, MODE, NS, INPLACE>, dev::kEncThreads, enc_smem_bytes(OP, NS, INPLACE), cache);
}

template <int OP, int MODE, bool INPLACE = false>
cudaError_t launch_encode_t(const TensorMaps& map, const EncParams& p, cudaStream_t stream, bool overlap) {
  constexpr int NS = INPLACE ? 1 : dev::enc_stages(OP);
  constexpr int smem = enc_smem_bytes(OP, NS, INPLACE);
  const int cap = encode_capacity<OP, MODE, INPLACE>();
  if (cap <= 0) return cudaErrorLaunchOutOfResources;
  int grid = (int)(p.n_tiles < (uint32_t)cap ? p.n_tiles : (uint32_t)cap);
  if (p.grid_limit && (int)p.grid_limit < grid) grid = (int)p.grid_limit;
  if (overlap)
    return launch_overlapped(dev::hc_encode_kernel<OP, MODE, NS, INPLACE>, grid, dev::kEncThreads, smem, stream, map, p);
  dev::hc_encode_kernel<OP, MODE, NS, INPLACE><<<grid, dev::kEncThreads, smem, stream>>>(map, p);
  return cudaGetLastError();
}

template <int OP>
cudaError_t launch_encode_m(int mode, const TensorMaps& map, const EncParams& p, cudaStream_t stream, bool overlap) {
  switch (mode) {
    case kModeOutlier: return launch_encode_t<OP, kModeOutlier>(map, p, stream, overlap);
    case kModePlain: return launch_encode_t<OP, kModePlain>(map, p, stream, overlap);
    case kModeVec: return launch_encode_t<OP, kModeVec>(map, p, stream, overlap);
    default: return cudaErrorInvalidValue;
  }
}

template <int MODE, bool SUM = false>
cudaError_t launch_decode_t(const TensorMaps& maps, const DecParams& p, cudaStream_t stream, bool overlap) {
  static thread_local int cache[64] = {};
  const int cap = resident_ctas(dev::hc_decode_kernel<MODE, SUM>, dev::kDecThreads, kDecSmem, cache);
  if (cap <= 0) return cudaErrorLaunchOutOfResources;
  const uint32_t tickets = SUM ? p.tiles_per_seg : p.n_tiles;
  int grid = (int)(tickets < (uint32_t)cap ? tickets : (uint32_t)cap);
  if (p.grid_limit && (int)p.grid_limit < grid) grid = (int)p.grid_limit;
  if (overlap)
    return launch_overlapped(dev::hc_decode_kernel<MODE, SUM>, grid, dev::kDecThreads, kDecSmem, stream, maps, p);
  dev::hc_decode_kernel<MODE, SUM><<<grid, dev::kDecThreads, kDecSmem, stream>>>(maps, p);
  return cudaGetLastError();
}

}  // namespace

// sized for max_elems values split over up to kMaxDst segments (each rounded up to whole chunks)
static size_t workspace_tiles(size_t max_elems) {
  return rate_bytes(max_elems) / kTileBlocks + (size_t)kMaxDst * (kBlocksPerChunk / kTileBlocks) + 1;
}
size_t workspace_bytes(size_t max_elems, int sets) {
  size_t tiles = workspace_tiles(max_elems);
  size_t groups = tiles / 32 + 1 + kMaxDst;
  if (sets < 1) sets = 1;
  if (sets > kMaxWorkspaceSets) sets = kMaxWorkspaceSets;
  return kWorkspaceHeader + (size_t)sets * 3 * (tiles + groups) * sizeof(uint64_t);
}

Workspace workspace_view(void* mem, size_t max_elems, uint32_t epoch, uint64_t spin_limit_ns, int sets) {
  size_t tiles = workspace_tiles(max_elems);
  Workspace w;
  uint8_t* b = static_cast<uint8_t*>(mem);
  w.ctrl = reinterpret_cast<uint32_t*>(b);
  size_t groups = tiles / 32 + 1 + kMaxDst;
  if (sets < 1) sets = 1;
  if (sets > kMaxWorkspaceSets) sets = kMaxWorkspaceSets;
  const size_t set = epoch % (uint32_t)sets;
  w.tick = w.ctrl + 8 + 2 * set;  // words 8..15 of the header
  w.size_acc = reinterpret_cast<uint64_t*>(b + 256) + set * kMaxDst;  // second half of the header
  w.st_a = reinterpret_cast<uint64_t*>(b + kWorkspaceHeader) + set * 3 * (tiles + groups);
  w.st_b = w.st_a + tiles;
  w.st_out = w.st_b + tiles;
  w.grp_a = w.st_out + tiles;
  w.grp_b = w.grp_a + groups;
  w.grp_out = w.grp_b + groups;
  w.epoch = epoch;
  w.spin_limit_ns = spin_limit_ns;
  return w;
}

int device_sm_count() { return device_info().sms > 0 ? device_info().sms : 148; }

cudaError_t launch_encode(int op, int mode, EncParams p, cudaStream_t stream, bool overlap) {
  if (p.n_seg == 0 || p.n_seg > (uint32_t)kMaxDst || p.n_in > (uint32_t)kMaxIn) return cudaErrorInvalidValue;
  if (p.n_seg > 1 && (op != kOpCompress || p.n_in != 0)) return cudaErrorInvalidValue;
  if (op == kOpCompress) p.n_in = 0;
  uint64_t n_max = 0;
  for (uint32_t g = 0; g < p.n_seg; ++g) n_max = p.n[g] > n_max ? p.n[g] : n_max;
  if (n_max == 0) return cudaSuccess;
  p.tiles_per_seg = (uint32_t)(rate_bytes(n_max) / kTileBlocks);
  p.n_tiles = p.tiles_per_seg * p.n_seg;
  TensorMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (uint32_t g = 0; g < p.n_seg; ++g) {
    p.use_tma[g] = 0;
    if (op != kOpAddStream && p.n[g]) {
      // int32 deltas are stored in whole blocks; fp32 data may end in a ragged row
      uint64_t rows = op == kOpAddI32 ? num_blocks(p.n[g]) : p.n[g] / kBlock;
      p.use_tma[g] = make_rows_map(&maps.m[g], p.local[g], rows) ? 1u : 0u;
    }
  }
  if (op == kOpAddF32 && mode == kModeOutlier) {
    // the in-place variant holds a fourth CTA per SM: taken when that saves a whole round of tiles
    // (tiles per CTA, rounded up) and leaves at most two
    const uint32_t cap3 = (uint32_t)encode_capacity<kOpAddF32, kModeOutlier, false>();
    const uint32_t cap4 = (uint32_t)encode_capacity<kOpAddF32, kModeOutlier, true>();
    if (cap3 && cap4) {
      const uint32_t rounds3 = (p.n_tiles + cap3 - 1) / cap3, rounds4 = (p.n_tiles + cap4 - 1) / cap4;
      if (p.variant == 2 || (p.variant == 0 && rounds4 < rounds3 && rounds4 <= 2))
        return launch_encode_t<kOpAddF32, kModeOutlier, true>(maps, p, stream, overlap);
    }
  }
  switch (op) {
    case kOpCompress: return launch_encode_m<kOpCompress>(mode, maps, p, stream, overlap);
    case kOpAddF32: return launch_encode_m<kOpAddF32>(mode, maps, p, stream, overlap);
    case kOpAddI32: return launch_encode_m<kOpAddI32>(mode, maps, p, stream, overlap);
    case kOpAddStream: return launch_encode_m<kOpAddStream>(mode, maps, p, stream, overlap);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_decode(int mode, DecParams p, cudaStream_t stream, bool overlap) {
  if (p.n_seg == 0 || p.n_seg > (uint32_t)kMaxDst) return cudaErrorInvalidValue;
  uint64_t n_max = 0;
  for (uint32_t i = 0; i < p.n_seg; ++i) n_max = p.seg[i].n > n_max ? p.seg[i].n : n_max;
  if (n_max == 0) return cudaSuccess;
  p.tiles_per_seg = (uint32_t)(rate_bytes(n_max) / kTileBlocks);
  p.n_tiles = p.tiles_per_seg * p.n_seg;
  TensorMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (p.sum) {
    // one output: every stream must describe the same array
    for (uint32_t i = 1; i < p.n_seg; ++i)
      if (p.seg[i].n != p.seg[0].n) return cudaErrorInvalidValue;
    if (mode == kModeVec) return cudaErrorInvalidValue;
    p.seg[0].use_tma = make_rows_map(&maps.m[0], p.seg[0].out, p.seg[0].n / kBlock) ? 1u : 0u;
    return launch_decode_t<kModeOutlier, true>(maps, p, stream, overlap);
  }
  for (uint32_t i = 0; i < p.n_seg; ++i)
    p.seg[i].use_tma = make_rows_map(&maps.m[i], p.seg[i].out, p.seg[i].n / kBlock) ? 1u : 0u;
  switch (mode) {
    case kModeOutlier:
    case kModePlain: return launch_decode_t<kModeOutlier>(maps, p, stream, overlap);
    case kModeVec: return launch_decode_t<kModeVec>(maps, p, stream, overlap);
    default: return cudaErrorInvalidValue;
  }
}

bool offsets_fit(const Workspace& ws, size_t max_elems, uint32_t n_in, uint32_t tiles_per_seg) {
  (void)ws;
  const size_t tiles = workspace_tiles(max_elems);
  const size_t groups = tiles / 32 + 1 + kMaxDst;
  const size_t n_cta = (tiles_per_seg + dev::kOffTiles - 1) / dev::kOffTiles;
  return (size_t)n_in * (n_cta + n_cta / 32 + 4) <= 2 * groups && (size_t)n_in * tiles_per_seg <= 2 * tiles;
}

cudaError_t launch_offsets(const OffsetParams& p, cudaStream_t stream) {
  if (p.n_in == 0 || p.n_in > (uint32_t)kMaxIn || p.tiles_per_seg == 0) return cudaErrorInvalidValue;
  const dim3 grid((p.tiles_per_seg + dev::kOffTiles - 1) / dev::kOffTiles, p.n_in);
  dev::hc_offsets_kernel<<<grid, dev::kOffThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_quant_pred(int mode, const float* x, int32_t* deltas, uint64_t n, float eb, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t n_padded = num_blocks(n) * kBlock;
  const uint64_t cap = (uint64_t)(device_info().sms > 0 ? device_info().sms : 148) * 16;
  int grid = (int)((n_padded + 255) / 256 < cap ? (n_padded + 255) / 256 : cap);
  float recip = 0.5f / eb;
  if (mode == kModeVec) dev::hc_quant_pred_kernel<kModeVec><<<grid, 256, 0, stream>>>(x, deltas, n, n_padded, recip);
  else dev::hc_quant_pred_kernel<kModeOutlier><<<grid, 256, 0, stream>>>(x, deltas, n, n_padded, recip);
  return cudaGetLastError();
}

cudaError_t launch_sum(float* dst, const float* a, const float* b, const float* c, const float* d, uint64_t n,
                       cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t want = (n / 4 + 255) / 256 + 1;
  const uint64_t cap = (uint64_t)(device_info().sms > 0 ? device_info().sms : 148) * 8;
  int grid = (int)(want < cap ? want : cap);
  dev::hc_sum_kernel<<<grid, 256, 0, stream>>>(dst, a, b, c, d, n);
  return cudaGetLastError();
}

}  // namespace hc

// CTAs of one launch that the current device holds at once: op 0 compress, 1 fused add, 2 fused add
// in place (the variant for launches of about one tile per CTA), 3 decode
extern "C" int hc_resident_ctas(int op) {
  switch (op) {
    case 0: return hc::encode_capacity<hc::kOpCompress, hc::kModeOutlier, false>();
    case 1: return hc::encode_capacity<hc::kOpAddF32, hc::kModeOutlier, false>();
    case 2: return hc::encode_capacity<hc::kOpAddF32, hc::kModeOutlier, true>();
    case 3: {
      static thread_local int cache[64] = {};
      return hc::resident_ctas(hc::dev::hc_decode_kernel<hc::kModeOutlier, false>, hc::dev::kDecThreads, hc::kDecSmem, cache);
    }
    default: return 0;
  }
}

#ifdef HC_TIMELINE
// copies the stamps of the last four launches (4 x 1024 CTAs x 32 slots) to the host (synchronises) and clears them
extern "C" int hc_debug_timeline(unsigned long long* host) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(host, hc::dev::g_timeline, sizeof(hc::dev::g_timeline)) != cudaSuccess) return -1;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, hc::dev::g_timeline) == cudaSuccess) cudaMemset(sym, 0, sizeof(hc::dev::g_timeline));
  return 0;
}
#endif
