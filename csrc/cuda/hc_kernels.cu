// Kernel bodies and host launchers of the sm_100a codec (see hc_kernels.cuh for the design).
#include "hc_kernels.cuh"

#include <stdio.h>

#include "hc_launch.h"

namespace hc {
namespace dev {

constexpr int kEncThreads = kComputeThreads + 64;  // + loader warp + scanner warp
constexpr int kDecThreads = kComputeThreads + 32;  // + loader warp
constexpr uint32_t kNoTile = 0xffffffffu;

constexpr int kMaxStages = 4;
struct __align__(16) EncShared {
  uint64_t tma_full[kMaxStages];    // fp32 tile landed in stage s (or "nothing to fetch"); also hands over the ticket
  uint64_t stage_free[kMaxStages];  // compute threads have moved the packed tile out of stage s
  uint64_t scan_done[kMaxStages];   // tile total known: the scanner may start its look-back
  uint64_t base_ready[kMaxStages];  // look-back of the tile in stage s finished: out_base / out_ok valid
  uint64_t in_full[2];              // input stream bytes + meta staged in buffer b
  uint64_t in_free[2];              // compute threads have decoded from buffer b
  uint32_t tile[8];                 // ring of tile tickets, written by the loader
  uint32_t tile_tma[8];             // 1 when a TMA load was issued for that ring slot
  uint32_t in_phase[2];             // 16-byte phase of the staged bytes in buffer b
  uint32_t in_end[2];               // 1: buffer b carries the end marker instead of a stream (ops with inputs)
  uint32_t out_tot[kMaxStages];     // payload bytes of the tile in stage s
  uint32_t out_ok[kMaxStages];
  uint64_t out_base[kMaxStages];    // global byte offset of the tile's payload
  uint32_t wsum[2][kComputeThreads / 32];
  uint32_t abort;
  uint16_t in_rel[2][kTileBlocks];
  uint8_t in_rate[2][kTileBlocks];
};

__device__ __forceinline__ void note_error(uint32_t* ctrl, uint32_t code) { atomicMax(ctrl + 2, code); }
// timeouts and peer failures end the launch early; capacity / truncation errors only skip data
__device__ __forceinline__ bool fatal_error(const uint32_t* ctrl) {
  return *((volatile const uint32_t*)(ctrl + 2)) >= (uint32_t)kErrTimeout;
}

// Optional per-CTA timeline (compile with -DHC_TIMELINE): sixteen nanosecond stamps of the first tile's
// way through the roles, for finding where a launch spends its fixed time.  Not part of a normal build.
#ifdef HC_TIMELINE
__device__ unsigned long long g_timeline[4 * 1024 * 16];  // [launch epoch & 3][CTA][slot]
__device__ __forceinline__ unsigned long long timeline_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define HC_TL_DECL(epoch) \
  unsigned long long* const hc_tl = g_timeline + (((epoch)&3u) * 1024u + (blockIdx.x < 1024u ? blockIdx.x : 1023u)) * 16u
#define HC_TL_ZERO() hc_tl[7] = hc_tl[14] = hc_tl[15] = 0
#define HC_STAMP(i) hc_tl[i] = timeline_now()
#define HC_STAMP_MAX(i) atomicMax(&hc_tl[i], timeline_now())
#define HC_TIC() const unsigned long long hc_tic = timeline_now()
#define HC_TOC(i) hc_tl[i] += timeline_now() - hc_tic
#else
#define HC_TL_DECL(epoch)
#define HC_TL_ZERO()
#define HC_STAMP(i)
#define HC_STAMP_MAX(i)
#define HC_TIC()
#define HC_TOC(i)
#endif

// the last CTA to leave re-arms the ticket counter for the next launch
__device__ __forceinline__ void cta_epilogue(uint32_t* tick) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(tick + 1, 1u);
    if (done == gridDim.x - 1) {
      tick[0] = 0;
      tick[1] = 0;
      __threadfence();
    }
  }
}

// bounded mbarrier wait that records a timeout
__device__ __forceinline__ bool wait_or_flag(uint64_t* bar, uint32_t parity, const Workspace& ws, volatile uint32_t* abort) {
  if (mbar_wait_bounded(bar, parity, ws.spin_limit_ns)) return true;
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
  if (ok && base + tot > in_size) {  // stream shorter than its rate bytes imply
    if (lane == 0) note_error(ws.ctrl, kErrTruncated);
    ok = false;
  }
  // the staging buffer (bytes and meta) is free once the compute threads have decoded its previous tile
  if (wait_free && !wait_or_flag(free_bar, free_parity, ws, abort)) ok = false;
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
//   [1 KB guard | stage 0 (16 KB) | 1 KB guard | ... | stage NS-1 | 1 KB guard | cbuf 0 | cbuf 1]
// A stage first receives the fp32 tile from the TMA unit; once every compute thread holds its row
// in registers the same bytes become the packing buffer of the tile's payload, which leaves
// moves out before the loader refills the stage.  NS = 3 when nothing else needs shared memory
// (compress: 4 CTAs per SM), 2 when an input stream is staged too (3 CTAs per SM), and 1 in the
// variant for launches with about one tile per CTA, where a fourth CTA per SM is worth more than
// overlap between a CTA's own tiles (the reduce step of a collective over many ranks).
constexpr int kStagePitch = kTileBytes + 1024;
__host__ __device__ constexpr int enc_stages(int op) { return op == kOpCompress ? 3 : 2; }
__host__ __device__ constexpr int enc_smem_base(int ns) { return 1024 + ns * kStagePitch; }

template <int OP, int MODE, int NS>
__global__ void __launch_bounds__(kEncThreads, (OP == kOpCompress || NS == 1) ? 4 : 3)
hc_encode_kernel(const __grid_constant__ TensorMaps tmaps, const EncParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ EncShared sh;
  constexpr bool kHasLocal = OP != kOpAddStream;
  constexpr bool kHasIn = OP != kOpCompress;
  uint8_t* const stage0 = smem + 1024;
  uint8_t* cbuf[2] = {smem + enc_smem_base(NS), smem + enc_smem_base(NS) + kBufBytes};

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
    v.g = p.n_seg > 1 ? tile / p.tiles_per_seg : 0u;
    v.lt = tile - v.g * p.tiles_per_seg;
    v.n = p.n[v.g];
    v.nrate = rate_bytes(v.n);
    v.full_rows = OP == kOpAddI32 ? num_blocks(v.n) : v.n / kBlock;
    v.n_local = OP == kOpAddI32 ? num_blocks(v.n) * kBlock : v.n;
    return v;
  };
  // destinations of a tile: every destination of the single segment, or the segment's own one
  auto dst_first = [&](const Seg& v) -> uint32_t { return p.n_seg > 1 ? v.g : 0u; };
  auto dst_count = [&](const Seg&) -> uint32_t { return p.n_seg > 1 ? 1u : p.n_dst; };

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&sh.tma_full[i], 1);
      mbar_init(&sh.stage_free[i], kComputeThreads);
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
  }
  __syncthreads();
  volatile uint32_t* abort = &sh.abort;
  if (tid == 0) HC_STAMP(0);

  // The packed payload of a tile leaves one turn late, so that its look-back has a whole tile time
  // to finish: compress moves tile k-1 out at the end of turn k (three stages); the ops with input
  // streams move it out in the middle of turn k, between decoding the inputs of tile k (which needs
  // neither the tile's fp32 stage nor its number) and reading its local operand (two stages: the
  // stage freed here is refilled for tile k+1 while tile k is quantised and packed).
  auto move_out = [&](uint32_t j) {  // compute threads: tile number j of this CTA -> global memory
    const int sj = j % NS;
    wait_or_flag(&sh.base_ready[sj], (j / NS) & 1, ws, abort);
    const Seg v = seg_of(sh.tile[j & 7]);
    if (sh.out_ok[sj])
      copy_out(stage0 + sj * kStagePitch, p.out + dst_first(v), dst_count(v), sh.out_base[sj], sh.out_tot[sj], tid,
               kComputeThreads, p.n_seg == 1 ? p.out_mc : nullptr);
    mbar_arrive(&sh.stage_free[sj]);  // the loader may refill the stage
  };
  if (warp == kComputeThreads / 32) {
    // ================================ loader warp ================================================
    // Tiles: CTA i starts with tile i (no round trip, and a CTA that starts late, behind a launch
    // that is still draining, finds its tile waiting instead of taken by an early starter); the
    // tiles past the grid come from a shared ticket counter.  Software pipeline over this CTA's
    // tiles: the ticket is taken two turns ahead and the rate bytes of the next input tile one
    // turn ahead, so neither round trip sits between two look-backs.  Per tile: the input streams first (their aggregates are published before any
    // wait on this CTA's compute warps), then the fp32 tile's TMA load once its stage is free.
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
      // hand-over: the fp32 tile's TMA load into stage s (free once the tile packed there NS turns ago
      // has been moved out) and the ticket for the compute and scanner warps
      auto hand_over = [&]() -> uint32_t {
        uint32_t t_stage = tile;
        if (k >= NS && !wait_or_flag(&sh.stage_free[s], ((k / NS) - 1) & 1, ws, abort)) t_stage = kNoTile;
        if (lane == 0) {
          sh.tile[slot] = t_stage;
          bool fetch = false;
          if (kHasLocal && t_stage != kNoTile) {
            const Seg v = seg_of(t_stage);
            fetch = p.use_tma[v.g] && (uint64_t)v.lt * kTileBlocks < v.full_rows;
            if (fetch) {
              fence_proxy_async();
              mbar_expect_tx(&sh.tma_full[s], kTileBytes);
              tma_load_2d(stage0 + s * kStagePitch, &tmaps.m[v.g], 0, (int)(v.lt * kTileBlocks), &sh.tma_full[s]);
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
        if (u >= 1) wait_or_flag(&sh.in_free[b], (u - 1) & 1, ws, abort);
        if (lane == 0) {
          sh.tile[slot] = kNoTile;
          sh.in_end[b] = 1u;
          mbar_arrive(&sh.in_full[b]);
        }
      }
      // The first NS tiles find their stage free: their TMA load goes out before anything else.
      // Afterwards the first two input streams go in first (their buffers only depend on earlier
      // tiles and free up before the stage does).  Later streams reuse a buffer that the compute
      // warps free while decoding THIS tile's first streams.
      uint32_t t_stage = kNoTile;
      const bool early = k < (uint32_t)NS;
      // With a single stage the hand-over waits for the previous tile to leave, which the compute
      // warps only do after decoding ALL of this tile's streams: every stream goes in first then.
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
    // runs the decoupled look-back of the output stream as soon as a tile's total is known, while
    // the compute warps are still transposing and packing; hands them the tile's global offset.
    // In a collective step it also raises the consumers' arrival flags: by the time the compute
    // warps announce tile k's total, all of them have passed a barrier that follows the stores of
    // tile k-1 (ops with input streams) or k-2 (compress), so those tiles can be announced.  One
    // system-scope fence covers a batch of tiles: it waits for the peers' write acknowledgements,
    // several microseconds over NVLink, and this warp has a tile time of slack that the loader
    // and the compute warps do not.
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
    for (uint32_t k = 0;; ++k) {
      const int s = k % NS;
      const uint32_t par = (k / NS) & 1;
      if (!wait_or_flag(&sh.scan_done[s], par, ws, abort)) break;
      const uint32_t tile = sh.tile[k & 7];
      if (tile == kNoTile) {
        raise_flags(k);  // the compute warps have stored every tile before they send the end marker
        break;
      }
      const Seg v = seg_of(tile);
      const uint32_t tot = sh.out_tot[s];
      bool ok = true;
      const Chain chain{ws.st_out + (size_t)v.g * p.tiles_per_seg, ws.grp_out + (size_t)v.g * groups_per_seg};
      const uint64_t excl = lookback(chain, v.lt, ws.epoch, tot, ws.spin_limit_ns, ws.ctrl + 2, &ok);
      const uint64_t goff = v.nrate + excl;
      if (k == 0 && lane == 0) HC_STAMP(4);
      if (ok && goff + tot > p.out_cap) {
        if (lane == 0) note_error(ws.ctrl, kErrCapacity);
        ok = false;
      }
      if (lane == 0) {
        sh.out_base[s] = goff;
        sh.out_ok[s] = ok ? 1u : 0u;
        mbar_arrive(&sh.base_ready[s]);
        if (ok && v.lt == p.tiles_per_seg - 1 && p.size_out) p.size_out[v.g] = goff + tot;
        if (fatal_error(ws.ctrl)) *abort = 1;
      }
      if ((uint32_t)lane == (k & 31u)) {
        my_lt = v.lt;
        my_g = v.g;
        my_word = flag_pack(p.ring_epoch, ok ? goff : kFlagOffsetMask);
      }
      const uint32_t out = kHasIn ? k : (k >= 1 ? k - 1 : 0u);  // tiles [0, out) are stored
      if (out - flagged >= kFlagBatch) raise_flags(out);
    }
  } else {
    // ================================ compute warps ==============================================
    for (uint32_t k = 0;; ++k) {
      const int s = k % NS, slot = k & 7;
      uint8_t* const stage_s = stage0 + s * kStagePitch;
      int32_t d[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) d[i] = 0;

      // ---- incoming stream(s) -> signed deltas, summed -------------------------------------------
      bool end = false;
      if (kHasIn) {
        for (uint32_t q = 0; q < Q; ++q) {
          const uint32_t vv = k * Q + q, b = vv & 1u;
          const bool staged = wait_or_flag(&sh.in_full[b], (vv >> 1) & 1, ws, abort);
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
          if (k == 0 && tid == 0 && q < 8) HC_STAMP(8 + q);
        }
        if (k >= 1) {
          compute_barrier();  // every thread has packed tile k-1
          move_out(k - 1);
          if (k == 1 && tid == 0) HC_STAMP(5);
        }
      }
      const bool alive = !end && wait_or_flag(&sh.tma_full[s], (k / NS) & 1, ws, abort);
      if (k == 0 && tid == 0) HC_STAMP(2);
      const uint32_t tile = alive ? sh.tile[slot] : kNoTile;
      if (tile == kNoTile) {
        if (!kHasIn && k >= 1) {
          compute_barrier();  // no scan barrier this turn: wait until every thread has packed
          move_out(k - 1);
          if (k == 1 && tid == 0) HC_STAMP(5);
        }
        compute_barrier();  // every thread's stores of the last tile are issued before the scanner hears of the end
        if (tid == 0) mbar_arrive(&sh.scan_done[s]);  // wakes the scanner, which sees the end marker too
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
      }

      // ---- encode ----------------------------------------------------------------------------------
      uint32_t A[32];
      BlockCode code = analyse_block<MODE>(d, A);
      uint32_t tot;
      // the barrier inside the scan also separates the last read of the fp32 tile from the first
      // write of the packed payload into the same stage
      const uint32_t rel = compute_exclusive_scan(code.len, sh.wsum[k & 1], &tot);
      if (tid == 0) {
        // publish the tile aggregate right away: successors can look back through this tile
        if (v.lt != 0)
          st_relaxed_gpu_u64(ws.st_out + (size_t)v.g * p.tiles_per_seg + v.lt, st_pack(kStAgg, ws.epoch, tot));
        sh.out_tot[s] = tot;
        mbar_arrive(&sh.scan_done[s]);
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
      write_payload(stage_s, rel, code, A, W);
      if (!kHasIn && k >= 1) {
        move_out(k - 1);  // packed before this turn's scan barrier
        if (k == 1 && tid == 0) HC_STAMP(5);
      }
    }
  }
  if (lane == 0) HC_STAMP_MAX(7);
  cta_epilogue(ws.tick);
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

template <int MODE>
__global__ void __launch_bounds__(kDecThreads, 4)
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
    auto take = [&]() -> uint32_t {  // lane 0 takes a ticket, every lane gets it
      uint32_t t = kNoTile;
      if (lane == 0 && !*abort) t = gridDim.x + atomicAdd(ws.tick, 1u);
      t = __shfl_sync(0xffffffffu, t, 0);
      return t < p.n_tiles ? t : kNoTile;
    };
    // non-blocking; fw receives the tile's arrival flag word when the segment has flags
    auto try_fetch = [&](uint32_t t, uint32_t (&r)[kRatesPerLane], uint64_t& fw) -> bool {
      if (t == kNoTile) return false;
      const uint32_t sg = t / p.tiles_per_seg, lt = t - sg * p.tiles_per_seg;
      const DecSegment& seg = p.seg[sg];
      fw = 0;
      if (seg.in_ready && (fw = flag_peek(seg.in_ready + lt, p.ring_epoch)) == 0) return false;
      loader_fetch_rates(seg.in, seg.in_size, lt, r);
      return true;
    };
    uint32_t tile = (!*abort && blockIdx.x < p.n_tiles) ? blockIdx.x : kNoTile;
    if (lane == 0) HC_STAMP(1);
    uint32_t tile_n = tile != kNoTile ? take() : kNoTile;
    uint32_t rates[kRatesPerLane] = {}, rates_n[kRatesPerLane] = {};
    uint64_t fw = 0, fw_n = 0;
    bool have = try_fetch(tile, rates, fw), have_n = false;
    for (uint32_t k = 0;; ++k) {
      const int s = k & 1;
      if (tile == kNoTile) {
        // end marker; the buffer's previous phase must have been consumed before it is re-armed
        if (k >= 2) wait_or_flag(&sh.in_free[s], ((k >> 1) - 1) & 1, ws, abort);
        if (lane == 0) sh.tile[k & 3] = kNoTile;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.in_full[s]);
        break;
      }
      const uint32_t tile_nn = tile_n != kNoTile ? take() : kNoTile;
      have_n = try_fetch(tile_n, rates_n, fw_n);
      const uint32_t sg = tile / p.tiles_per_seg, lt = tile - sg * p.tiles_per_seg;
      const DecSegment& seg = p.seg[sg];
      bool usable = true;
      if (!have) {
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
    for (uint32_t k = 0;; ++k) {
      const int s = k & 1;
      bool alive = wait_or_flag(&sh.in_full[s], (k >> 1) & 1, ws, abort);
      if (k == 0 && tid == 0) HC_STAMP(2);
      const uint32_t tile = alive ? sh.tile[k & 3] : kNoTile;
      if (tile == kNoTile) break;
      const uint32_t sg = tile / p.tiles_per_seg, lt = tile - sg * p.tiles_per_seg;
      const DecSegment& seg = p.seg[sg];
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
      if (k == 0 && tid == 0) HC_STAMP(3);
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__fmul_rn(__fmul_rn((float)d[i], eb), 2.0f));

      const uint64_t row = (uint64_t)lt * kTileBlocks + tid;
      const bool ragged = row * kBlock < seg.n && (row + 1) * kBlock > seg.n;
      // the TMA store of the previous tile must have finished reading obuf
      if (tid == 0) tma_wait_group_read<0>();
      compute_barrier();
      if (tma) {
        store_row_swizzled(obuf, tid, w);
        fence_proxy_async();
      }
      compute_barrier();
      if (tid == 0) {
        if (tma && (uint64_t)lt * kTileBlocks < full_rows)
          tma_store_2d(&tmaps.m[sg], 0, (int)(lt * kTileBlocks), obuf);
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

constexpr int enc_smem_bytes(int op, int ns) { return dev::enc_smem_base(ns) + (op == kOpCompress ? 0 : 2 * kBufBytes) + 1024; }
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

template <int OP, int MODE, int NS = dev::enc_stages(OP)>
cudaError_t launch_encode_t(const TensorMaps& map, const EncParams& p, int grid, cudaStream_t stream, bool overlap) {
  constexpr int smem = enc_smem_bytes(OP, NS);
  static thread_local bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = set_smem(dev::hc_encode_kernel<OP, MODE, NS>, smem);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  if (overlap) return launch_overlapped(dev::hc_encode_kernel<OP, MODE, NS>, grid, dev::kEncThreads, smem, stream, map, p);
  dev::hc_encode_kernel<OP, MODE, NS><<<grid, dev::kEncThreads, smem, stream>>>(map, p);
  return cudaGetLastError();
}

template <int OP>
cudaError_t launch_encode_m(int mode, const TensorMaps& map, const EncParams& p, int grid, cudaStream_t stream,
                            bool overlap) {
  switch (mode) {
    case kModeOutlier: return launch_encode_t<OP, kModeOutlier>(map, p, grid, stream, overlap);
    case kModePlain: return launch_encode_t<OP, kModePlain>(map, p, grid, stream, overlap);
    case kModeVec: return launch_encode_t<OP, kModeVec>(map, p, grid, stream, overlap);
    default: return cudaErrorInvalidValue;
  }
}

template <int MODE>
cudaError_t launch_decode_t(const TensorMaps& maps, const DecParams& p, int grid, cudaStream_t stream, bool overlap) {
  static thread_local bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = set_smem(dev::hc_decode_kernel<MODE>, kDecSmem);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  if (overlap) return launch_overlapped(dev::hc_decode_kernel<MODE>, grid, dev::kDecThreads, kDecSmem, stream, maps, p);
  dev::hc_decode_kernel<MODE><<<grid, dev::kDecThreads, kDecSmem, stream>>>(maps, p);
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
  return 256 + (size_t)sets * 3 * (tiles + groups) * sizeof(uint64_t);
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
  w.st_a = reinterpret_cast<uint64_t*>(b + 256) + set * 3 * (tiles + groups);
  w.st_b = w.st_a + tiles;
  w.st_out = w.st_b + tiles;
  w.grp_a = w.st_out + tiles;
  w.grp_b = w.grp_a + groups;
  w.grp_out = w.grp_b + groups;
  w.epoch = epoch;
  w.spin_limit_ns = spin_limit_ns;
  return w;
}

int grid_for_tiles(uint32_t n_tiles, int ctas_per_sm) {
  int cap = device_info().sms * ctas_per_sm;
  if (cap <= 0) cap = 148 * ctas_per_sm;
  return (int)(n_tiles < (uint32_t)cap ? n_tiles : (uint32_t)cap);
}

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
  int grid = grid_for_tiles(p.n_tiles, op == kOpCompress ? 4 : 3);
  if (op == kOpAddF32 && mode == kModeOutlier) {
    // a fourth CTA per SM when that saves a whole round of tiles (tiles per CTA, rounded up)
    const int grid4 = grid_for_tiles(p.n_tiles, 4);
    const uint32_t rounds3 = (p.n_tiles + grid - 1) / grid, rounds4 = (p.n_tiles + grid4 - 1) / grid4;
    if (rounds4 < rounds3 && rounds4 <= 2)
      return launch_encode_t<kOpAddF32, kModeOutlier, 1>(maps, p, grid4, stream, overlap);
  }
  switch (op) {
    case kOpCompress: return launch_encode_m<kOpCompress>(mode, maps, p, grid, stream, overlap);
    case kOpAddF32: return launch_encode_m<kOpAddF32>(mode, maps, p, grid, stream, overlap);
    case kOpAddI32: return launch_encode_m<kOpAddI32>(mode, maps, p, grid, stream, overlap);
    case kOpAddStream: return launch_encode_m<kOpAddStream>(mode, maps, p, grid, stream, overlap);
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
  for (uint32_t i = 0; i < p.n_seg; ++i)
    p.seg[i].use_tma = make_rows_map(&maps.m[i], p.seg[i].out, p.seg[i].n / kBlock) ? 1u : 0u;
  int grid = grid_for_tiles(p.n_tiles, 4);
  switch (mode) {
    case kModeOutlier:
    case kModePlain: return launch_decode_t<kModeOutlier>(maps, p, grid, stream, overlap);
    case kModeVec: return launch_decode_t<kModeVec>(maps, p, grid, stream, overlap);
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

#ifdef HC_TIMELINE
// copies the stamps of the last four launches (4 x 1024 CTAs x 16 slots) to the host (synchronises) and clears them
extern "C" int hc_debug_timeline(unsigned long long* host) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(host, hc::dev::g_timeline, sizeof(hc::dev::g_timeline)) != cudaSuccess) return -1;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, hc::dev::g_timeline) == cudaSuccess) cudaMemset(sym, 0, sizeof(hc::dev::g_timeline));
  return 0;
}
#endif
