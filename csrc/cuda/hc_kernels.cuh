// The sm_100a codec kernels: one persistent, warp-specialised kernel family for everything that
// produces a stream (compress, and the three homomorphic adds) and one for everything that
// consumes a stream into fp32 (decompress).
//
// Geometry.  A tile is 128 consecutive 32-element blocks (4096 values, 16 KB of fp32).  A CTA has
// four COMPUTE warps in which thread t owns block t of the tile, i.e. one thread per block with
// the whole block in registers, plus a LOADER warp and a SCANNER warp:
//   loader   starts with tile blockIdx.x and takes further tiles from a ticket counter two turns
//            ahead, issues the 2-D TMA tiled load of the fp32 tile ({32, 128} box, 128-byte
//            swizzle; 3 stages for compress, 2 for the adds, 1 in the add variant that runs four
//            CTAs per SM); for the homomorphic adds it also reads the rate bytes of every input
//            stream's tile one turn ahead, scans them, learns the payload offset (from the tile's
//            arrival flag in a collective step, from a look-back over the INPUT stream otherwise)
//            and brings the payload bytes into shared memory with one bulk copy (up to 8 streams
//            per tile through two staging buffers);
//   compute  decodes the staged payloads to deltas and sums them, moves the PREVIOUS tile's packed
//            payload to its byte offset in global or peer memory (16-byte stores, or one multimem
//            store for all ranks), then quantises the local values, adds, chooses the block mode,
//            transposes the magnitudes to bit planes in registers (hc_bitplane.h) and packs the
//            tile's payload into the stage the fp32 tile came in;
//   scanner  runs the two-level decoupled look-back of the OUTPUT stream as soon as the tile total
//            is known and hands the compute warps the tile's global offset; when the launch is a
//            step of a collective it raises the consumers' arrival flags (call number and payload
//            offset in one 64-bit word), one system-scope fence per four stored tiles.
// The roles hand tiles to each other through mbarriers, so the compute warps never wait on a
// global-memory round trip of their own.  Look-back status words are 64-bit and epoch-tagged:
// the workspace is never cleared between launches, and the exact stream size lands in device
// memory (no host round trip).  The grid never exceeds what the GPU holds at once, so every tile's
// predecessors are in the hands of CTAs that run, have finished, or are next in line for an SM slot
// (other kernels on the GPU can delay them, not starve them); every wait is bounded all the same.
//
// The reference runs one warp per CTA, one thread per 32 blocks with a 4 KB local-memory array per
// thread, and needs a 4-byte device-to-host copy after every launch
// (HomComp/src/GSZ.cu:33-756, HomComp/src/GSZ_entry.cu:263-301).
#pragma once
#include "hc_bitplane.h"
#include "hc_device.cuh"

namespace hc {

constexpr int kTileBlocks = 128;
constexpr int kTileElems = kTileBlocks * kBlock;  // 4096
constexpr int kTileBytes = kTileElems * 4;        // 16384
constexpr int kBufBytes = 17 * 1024;              // a tile of stream bytes + alignment slack
constexpr int kComputeThreads = kTileBlocks;
constexpr int kMaxDst = 8;

enum Op : int {
  kOpCompress = 0,   // fp32 -> stream
  kOpAddF32 = 1,     // stream (+) fp32 -> stream
  kOpAddI32 = 2,     // stream (+) int32 deltas -> stream
  kOpAddStream = 3,  // stream (+) stream -> stream
};

struct Workspace {
  uint32_t* ctrl;    // [2] sticky error (hc::Status); the other words of the 256-byte header hold the tick sets
  uint64_t* st_a;    // look-back chain of the first input stream (tile words, then group words)
  uint64_t* st_b;    // look-back chain of the second input stream
  uint64_t* st_out;  // look-back chain of the output stream
  uint64_t* grp_a;
  uint64_t* grp_b;
  uint64_t* grp_out;
  uint32_t* tick;  // [0] tile ticket counter, [1] CTAs that have left; re-armed by the last CTA of a launch
  uint64_t* size_acc;  // [kMaxDst] payload bytes per segment of a launch with sparse tiles; zeroed by its last CTA
  uint32_t epoch;
  uint64_t spin_limit_ns;
};

// A launch of the stream-producing kernel.
//   * up to kMaxDst input streams are summed into every tile (n_in; 0 for compress);
//   * the output goes either to n_dst destinations that all receive the same stream (n_seg == 1:
//     a ring step, or the reduced chunk pushed to every rank), or, for compress only, to n_seg
//     independent streams ("segments": segment g compresses local[g] of n[g] values into out[g]);
//     tickets go round the segments, each of which has its own look-back chain.
constexpr int kMaxIn = kMaxDst;
struct EncParams {
  const void* local[kMaxDst];  // fp32 values or int32 deltas, per segment
  uint64_t n[kMaxDst];         // values per segment
  uint32_t use_tma[kMaxDst];
  uint32_t n_seg;
  uint32_t tiles_per_seg;
  uint32_t n_tiles;  // n_seg * tiles_per_seg
  uint32_t n_in;
  float recip;       // 0.5f / eb
  const uint8_t* in[kMaxIn];
  uint64_t in_size[kMaxIn];
  const uint64_t* in_ready[kMaxIn];  // one arrival flag per tile (dev::flag_pack), or null
  uint32_t ring_epoch;
  uint32_t n_dst;                // destinations of the single segment (ignored when n_seg > 1)
  uint8_t* out[kMaxDst];         // n_seg == 1: destinations; n_seg > 1: out[g] of segment g
  uint64_t* out_ready[kMaxDst];  // arrival flags on the consumers, laid out like `out`, or null
  uint8_t* out_mc;               // n_seg == 1 only: multicast alias of all n_dst destinations (NVLS), or null
  uint64_t out_cap;
  uint64_t* size_out;  // device words receiving the exact stream length of each segment (or null)
  uint32_t sparse;      // 1: tile t's payload goes to byte rate_bytes + t * 16384 of the output instead of right
                        //    behind tile t-1's (transport buffers of a collective, read through arrival flags only)
  uint32_t grid_limit;  // at most this many CTAs (0: as many as the GPU holds), to leave room for a concurrent launch
  uint32_t variant;     // fused add: 0 launcher's choice, 1 payload ring (3 CTAs per SM), 2 in place (4 per SM)
  Workspace ws;
};

// One decode launch can take several independent streams ("segments"): the all-gather phase of a
// collective decodes the P reduced chunks with one kernel.  Every segment owns tiles_per_seg
// consecutive tile tickets and its own look-back chain.
struct DecSegment {
  const uint8_t* in;
  uint64_t in_size;
  const uint64_t* in_ready;  // one arrival flag per tile (dev::flag_pack), or null
  float* out;
  uint64_t n;
  uint32_t use_tma;
  uint32_t pad;
};
struct DecParams {
  DecSegment seg[kMaxDst];
  uint32_t n_seg;
  uint32_t tiles_per_seg;
  uint32_t n_tiles;  // n_seg * tiles_per_seg
  uint32_t ring_epoch;
  float eb;
  uint32_t grid_limit;  // at most this many CTAs (0: as many as the GPU holds)
  uint32_t sum;         // 1: the n_seg streams are contributions to one array of seg[0].n values; their
                        //    quantised values are added tile by tile and seg[0].out receives the sum
  Workspace ws;
};
struct TensorMaps {
  CUtensorMap m[kMaxDst];
};
// Pre-pass that turns the rate bytes of n_in streams (tiles_per_seg tiles each, nrate rate bytes
// each) into per-tile arrival flags: flags[q][t] = flag_pack(tag, byte offset of tile t's payload).
struct OffsetParams {
  const uint8_t* in[kMaxIn];
  uint64_t in_size[kMaxIn];
  uint64_t* flags[kMaxIn];
  uint32_t n_in;
  uint32_t tiles_per_seg;
  uint64_t nrate;
  uint32_t tag;
  Workspace ws;  // grp_a / grp_b hold the chain of CTA totals
};

namespace dev {

// ---- per-thread block arithmetic ------------------------------------------------------------

__device__ __forceinline__ int32_t quantise(float x, float recip) {
  float t = __fmul_rn(x, recip);  // two roundings: the stream is defined without FMA contraction
  float u = __fadd_rn(t, 0.5f);
  return __float2int_rz(u) - ((t >= -0.5f) ? 0 : 1);
}

// 32 values of row `row` from a tile stored with the 128-byte TMA swizzle
__device__ __forceinline__ void load_row_swizzled(const uint8_t* stage, int row, uint32_t (&w)[32]) {
  const uint8_t* r = stage + row * 128;
  const int x = row & 7;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v = *reinterpret_cast<const uint4*>(r + ((c ^ x) << 4));
    w[4 * c + 0] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
  }
}
__device__ __forceinline__ void store_row_swizzled(uint8_t* stage, int row, const uint32_t (&w)[32]) {
  uint8_t* r = stage + row * 128;
  const int x = row & 7;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(r + ((c ^ x) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

// plain-load path (unaligned base, tiny inputs) and the ragged last row
__device__ __forceinline__ void load_row_global(const uint32_t* base, uint64_t n, uint64_t row, uint32_t (&w)[32]) {
  uint64_t o = row * kBlock;
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = (o + i < n) ? __ldg(base + o + i) : 0u;
}

template <int MODE>
__device__ __forceinline__ void lorenzo_forward(const int32_t (&q)[32], int32_t (&d)[32]) {
  constexpr int S = MODE == kModeVec ? 4 : 1;
#pragma unroll
  for (int i = 31; i >= 0; --i) d[i] = i >= S ? q[i] - q[i - S] : q[i];
}
template <int MODE>
__device__ __forceinline__ void lorenzo_inverse(int32_t (&d)[32]) {
  constexpr int S = MODE == kModeVec ? 4 : 1;
#pragma unroll
  for (int i = S; i < 32; ++i) d[i] += d[i - S];
}

struct BlockCode {
  uint32_t rate;      // rate byte
  uint32_t len;       // payload bytes
  uint32_t a0;        // |d0| when outlier mode
  uint32_t sign_mem;  // sign map as the little-endian word that goes to memory
};

// signed deltas -> rows A[j] = |d[j ^ 7]| plus the block's code
template <int MODE>
__device__ __forceinline__ BlockCode analyse_block(const int32_t (&d)[32], uint32_t (&A)[32]) {
  uint32_t sign = 0, or_tail = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    A[i ^ 7] = (uint32_t)abs(d[i]);
    sign = __funnelshift_l((uint32_t)d[i], sign, 1);
  }
#pragma unroll
  for (int i = 1; i < 31; i += 2) or_tail |= A[i ^ 7] | A[(i + 1) ^ 7];  // one 3-input LOP3 per pair
  or_tail |= A[31 ^ 7];
  uint32_t or_all = or_tail | A[7];
  if (or_all & 0x80000000u) {  // INT_MIN deltas: magnitude keeps 31 bits (outside the contract)
    or_tail = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      A[i ^ 7] &= 0x7fffffffu;
      if (i) or_tail |= A[i ^ 7];
    }
    or_all = or_tail | A[7];
  }
  BlockCode c;
  c.a0 = A[7];
  c.rate = choose_rate(or_all, or_tail, c.a0, MODE != kModePlain);
  c.len = payload_len(c.rate);
  c.sign_mem = __byte_perm(sign, 0, 0x0123);
  if (c.rate & 0x80u) A[7] = 0;
  return c;
}

__device__ __forceinline__ void transpose_forward(uint32_t (&A)[32], int W) {
  switch (W) {
    case 4: planes_from_rows<4>(A); break;
    case 8: planes_from_rows<8>(A); break;
    case 16: planes_from_rows<16>(A); break;
    case 32: planes_from_rows<32>(A); break;
    default: break;
  }
}

// Writes the block's payload at byte `pos` of the staging buffer.  T[0..W-1] hold the planes
// (planes at and above F are zero because every magnitude is below 2^F).
template <int W>
__device__ __forceinline__ void write_payload_w(uint8_t* obuf, uint32_t pos, const BlockCode& c, const uint32_t (&T)[32]) {
  const uint32_t F = c.rate & 31u;
  const bool outl = (c.rate & 0x80u) != 0;
  if (!outl && F == 0) return;
  uint32_t p2 = pos;
  if (outl) {
    const uint32_t nout = ((c.rate >> 5) & 3u) + 1u;
#pragma unroll
    for (uint32_t k = 0; k < 4; ++k)
      if (k < nout) obuf[pos + k] = (uint8_t)(c.a0 >> (8 * k));
    p2 += nout;
  }
  const uint32_t s = p2 & 3u;
  if (s == 0) {  // word-aligned block: plain predicated word stores
    uint32_t* wp = reinterpret_cast<uint32_t*>(obuf + p2);
    wp[0] = c.sign_mem;
#pragma unroll
    for (int j = 1; j <= W; ++j)
      if ((uint32_t)j <= F) wp[j] = T[j - 1];
  } else {  // shifted block: every aligned word takes bytes of two neighbours
    const uint32_t sh = 8u * s;
    uint8_t* wb = obuf + (p2 & ~3u);
    uint32_t prev = c.sign_mem;
    const uint32_t head = prev << sh;
#pragma unroll
    for (uint32_t b = 1; b < 4; ++b)
      if (b >= s) wb[b] = (uint8_t)(head >> (8 * b));
#pragma unroll
    for (int j = 1; j <= W; ++j) {
      const uint32_t x = T[j - 1];
      const bool live = (uint32_t)j <= F;
      if (live) *reinterpret_cast<uint32_t*>(wb + 4 * j) = __funnelshift_l(prev, x, sh);
      prev = live ? x : prev;
    }
    const uint32_t tail = prev >> (32u - sh);  // the last word's upper bytes spill into the next aligned word
    uint8_t* tb = wb + 4 * (F + 1);
#pragma unroll
    for (uint32_t b = 0; b < 3; ++b)
      if (b < s) tb[b] = (uint8_t)(tail >> (8 * b));
  }
}
__device__ __forceinline__ void write_payload(uint8_t* obuf, uint32_t pos, const BlockCode& c, const uint32_t (&T)[32],
                                              int W) {
  switch (W) {
    case 0: {  // only "outlier with F = 0" blocks carry bytes here
      write_payload_w<0>(obuf, pos, c, T);
      break;
    }
    case 4: write_payload_w<4>(obuf, pos, c, T); break;
    case 8: write_payload_w<8>(obuf, pos, c, T); break;
    case 16: write_payload_w<16>(obuf, pos, c, T); break;
    default: write_payload_w<32>(obuf, pos, c, T); break;
  }
}

// Reads the block's payload at byte `pos` of a staged stream; returns the sign map (memory form),
// planes in T[0..W-1] (zero at and above F) and |d0| of an outlier block in a0.  Word-aligned
// blocks take predicated 32-bit loads; shifted ones rebuild every word from two neighbours.
template <int W>
__device__ __forceinline__ void read_payload_w(const uint8_t* cbuf, uint32_t pos, uint32_t rate, uint32_t& sign_mem,
                                               uint32_t& a0, uint32_t (&T)[32]) {
  const uint32_t F = rate & 31u;
  const bool outl = (rate & 0x80u) != 0;
  a0 = 0;
  sign_mem = 0;
#pragma unroll
  for (int j = 0; j < (W ? W : 1); ++j) T[j] = 0;
  if (!outl && F == 0) return;
  uint32_t p2 = pos;
  if (outl) {
    const uint32_t nout = ((rate >> 5) & 3u) + 1u;
#pragma unroll
    for (uint32_t k = 0; k < 4; ++k)
      if (k < nout) a0 |= (uint32_t)cbuf[pos + k] << (8 * k);
    p2 += nout;
  }
  const uint32_t s = p2 & 3u;
  const uint32_t* wp = reinterpret_cast<const uint32_t*>(cbuf + (p2 & ~3u));
  if (s == 0) {
    sign_mem = wp[0];
#pragma unroll
    for (int j = 1; j <= W; ++j)
      if ((uint32_t)j <= F) T[j - 1] = wp[j];
  } else {
    const uint32_t sh = 8u * s;
    uint32_t prev = wp[0];
#pragma unroll
    for (int j = 0; j <= W; ++j) {
      const bool live = (uint32_t)j <= F;
      const uint32_t nxt = live ? wp[j + 1] : 0u;
      const uint32_t x = __funnelshift_r(prev, nxt, sh);
      if (j == 0) sign_mem = x;
      else if (live) T[j - 1] = x;
      prev = nxt;
    }
  }
}

// staged payload -> rows R[j] = |d[j ^ 7]| and the sign map in value form (element i at bit 31 - i)
__device__ __forceinline__ uint32_t decode_magnitudes(const uint8_t* cbuf, uint32_t pos, uint32_t rate, int W,
                                                      uint32_t (&T)[32]) {
  uint32_t sign_mem, a0;
  switch (W) {
    case 0:
      read_payload_w<0>(cbuf, pos, rate, sign_mem, a0, T);
#pragma unroll
      for (int i = 0; i < 32; ++i) T[i] = 0;
      break;
    case 4: read_payload_w<4>(cbuf, pos, rate, sign_mem, a0, T); rows_from_planes<4>(T); break;
    case 8: read_payload_w<8>(cbuf, pos, rate, sign_mem, a0, T); rows_from_planes<8>(T); break;
    case 16: read_payload_w<16>(cbuf, pos, rate, sign_mem, a0, T); rows_from_planes<16>(T); break;
    default: read_payload_w<32>(cbuf, pos, rate, sign_mem, a0, T); rows_from_planes<32>(T); break;
  }
  if (rate & 0x80u) T[7] = a0 & 0x7fffffffu;
  return __byte_perm(sign_mem, 0, 0x0123);
}

// staged payload -> signed deltas d[0..31]
__device__ __forceinline__ void decode_block(const uint8_t* cbuf, uint32_t pos, uint32_t rate, int W, int32_t (&d)[32]) {
  uint32_t T[32];
  const uint32_t sign = decode_magnitudes(cbuf, pos, rate, W, T);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int32_t m = (int32_t)(sign << i) >> 31;
    d[i] = ((int32_t)T[i ^ 7] ^ m) - m;
  }
}

// staged payload -> quantised values q[0..31]: sign application and inverse Lorenzo in one pass
// (q_i = q_{i-S} + (|d_i| ^ m_i) - m_i is a single three-input add per element)
template <int MODE>
__device__ __forceinline__ void decode_block_quant(const uint8_t* cbuf, uint32_t pos, uint32_t rate, int W,
                                                   int32_t (&q)[32]) {
  constexpr int S = MODE == kModeVec ? 4 : 1;
  uint32_t T[32];
  const uint32_t sign = decode_magnitudes(cbuf, pos, rate, W, T);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int32_t m = (int32_t)(sign << i) >> 31;
    const int32_t t = (int32_t)T[i ^ 7] ^ m;
    q[i] = i >= S ? q[i - S] + t - m : t - m;
  }
}

// ---- cooperative helpers --------------------------------------------------------------------

__device__ __forceinline__ void compute_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory"); }

// exclusive scan of one value per compute thread; *total = sum.  One named barrier; `s_wsum` must
// not be reused by the next scan before another barrier (callers alternate two arrays).
__device__ __forceinline__ uint32_t compute_exclusive_scan(uint32_t v, uint32_t* s_wsum, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = warp_inclusive_scan(v, lane);
  if (lane == 31) s_wsum[warp] = inc;
  compute_barrier();
  uint32_t pre = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kComputeThreads / 32; ++w) {
    uint32_t t = s_wsum[w];
    if (w < warp) pre += t;
    tot += t;
  }
  *total = tot;
  return inc - v + pre;
}

__device__ __forceinline__ uint64_t warp_sum_u64(uint64_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Two-level decoupled look-back, run by one full warp.
//
// Level 1: status word per tile.  Level 2: status word per GROUP of 32 tiles, published by the
// group's last tile (aggregate of the group as soon as its 32 tile aggregates are known, inclusive
// prefix once that tile has resolved its own).  A tile first sums the aggregates of the earlier
// tiles of its own group (one 32-wide poll), then walks back over whole groups, 32 groups = 1024
// tiles per poll.  With hundreds of tiles in flight a one-level walk needs (tiles in flight / 64)
// dependent polls per wave; this needs two or three.
//
// Publishes this tile's aggregate first and returns the exclusive prefix.  *ok = false when a
// predecessor was poisoned or the bounded wait ran out (then this tile is poisoned too).
struct Chain {
  uint64_t* tile_st;   // one word per tile
  uint64_t* group_st;  // one word per 32 tiles
};

// One 32-wide look at `st[idx], st[idx-1], ...` (lane l looks at idx - l; indices below `lo` count
// as "inclusive 0").  Consumes the longest ready run starting at idx.  Returns the number of
// entries consumed; *sum gets their total, *hit whether the run ended on an inclusive entry,
// *bad whether a poisoned entry was met.
__device__ __forceinline__ uint32_t look_once(const uint64_t* st, int64_t idx, int64_t lo, uint32_t epoch, uint64_t* sum,
                                              bool* hit, bool* bad) {
  const int lane = threadIdx.x & 31;
  const int64_t j = idx - lane;
  uint64_t w = st_pack(kStInc, epoch, 0);
  if (j >= lo) w = ld_relaxed_gpu_u64(st + j);
  const uint32_t s = st_state(w, epoch);
  const uint32_t notready = __ballot_sync(0xffffffffu, s == 0);
  const uint32_t incs = __ballot_sync(0xffffffffu, s == kStInc);
  const uint32_t bads = __ballot_sync(0xffffffffu, s == kStBad);
  // the run ends at the first inclusive entry (taken) or before the first missing / poisoned one
  const uint32_t stop_excl = notready | bads;
  const int first_stop = stop_excl ? __ffs(stop_excl) - 1 : 32;
  const int first_inc = incs ? __ffs(incs) - 1 : 32;
  int take;
  if (first_inc < first_stop) {
    take = first_inc + 1;
    *hit = true;
  } else {
    take = first_stop;
    *hit = false;
  }
  *bad = bads != 0 && (__ffs(bads) - 1) == take;
  *sum = warp_sum_u64(lane < take ? st_value(w) : 0ull);
  return (uint32_t)take;
}

__device__ __forceinline__ uint64_t lookback(const Chain& ch, uint32_t tile, uint32_t epoch, uint64_t agg,
                                             uint64_t limit_ns, volatile uint32_t* err_word, bool* ok) {
  const int lane = threadIdx.x & 31;
  const uint32_t grp = tile >> 5, pos = tile & 31u;
  *ok = true;
  if (tile == 0) {
    if (lane == 0) st_relaxed_gpu_u64(ch.tile_st, st_pack(kStInc, epoch, agg));
    return 0;
  }
  if (lane == 0) st_relaxed_gpu_u64(ch.tile_st + tile, st_pack(kStAgg, epoch, agg));
  const long long t0 = clock64();
  const long long limit_clk = (long long)limit_ns * 2;  // SM clock is at most ~2 GHz
  uint64_t excl = 0;
  bool good = true, done = false;
  uint32_t idle = 0;
  auto stalled = [&]() -> bool {  // called after a poll that made no progress
    ++idle;
    if ((idle & 15u) != 15u) return false;
    return clock64() - t0 > limit_clk || idle > (1u << 24) || *err_word >= (uint32_t)kErrTimeout;
  };
  // ---- level 1: the earlier tiles of this group ------------------------------------------------
  {
    int64_t idx = (int64_t)tile - 1;
    const int64_t lo = (int64_t)grp * 32;
    while (idx >= lo) {
      uint64_t sum;
      bool hit, bad;
      const uint32_t n = look_once(ch.tile_st, idx, lo, epoch, &sum, &hit, &bad);
      excl += sum;
      idx -= n;
      if (bad) { good = false; break; }
      if (hit) {
        if (idx + 1 >= lo) done = true;  // a real inclusive entry, not the virtual one below `lo`
        break;
      }
      if (n == 0 && stalled()) { good = false; break; }
    }
  }
  // the group's last tile knows the group aggregate now: let later groups skip over this one
  if (good && !done && pos == 31 && lane == 0)
    st_relaxed_gpu_u64(ch.group_st + grp, st_pack(kStAgg, epoch, excl + agg));
  // ---- level 2: whole groups -------------------------------------------------------------------
  if (good && !done && grp > 0) {
    int64_t idx = (int64_t)grp - 1;
    while (true) {
      uint64_t sum;
      bool hit, bad;
      const uint32_t n = look_once(ch.group_st, idx, 0, epoch, &sum, &hit, &bad);
      excl += sum;
      idx -= n;
      if (bad) { good = false; break; }
      if (hit) break;  // a group's inclusive prefix, or the virtual zero before group 0
      if (n == 0 && stalled()) { good = false; break; }
    }
  }
  if (lane == 0) {
    const uint64_t word = st_pack(good ? kStInc : kStBad, epoch, excl + agg);
    st_relaxed_gpu_u64(ch.tile_st + tile, word);
    if (pos == 31) st_relaxed_gpu_u64(ch.group_st + grp, word);
    if (!good) {
      // err_word is word 2 of the workspace header; word 3 keeps the first wait that ran out (11: a look-back)
      if (*err_word < (uint32_t)kErrTimeout) atomicCAS((uint32_t*)err_word + 1, 0u, 11u);
      atomicMax((uint32_t*)err_word, (uint32_t)kErrTimeout);
    }
  }
  *ok = good;
  return excl;
}

// bounded wait for a 32-bit flag written by another GPU (uncompressed collective)
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, uint64_t limit_ns, volatile uint32_t* err_word) {
  if (ld_acquire_sys_u32(flag) == want) return true;
  const long long t0 = clock64();
  const long long limit_clk = (long long)limit_ns * 2;
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (ld_acquire_sys_u32(flag) == want) return true;
    if ((it & 7u) == 7u) {
      __nanosleep(64);
      if (clock64() - t0 > limit_clk || *err_word >= (uint32_t)kErrTimeout) return false;
    }
  }
  return false;
}
// bounded wait for a tile's arrival flag of call `call`; returns the flag word, or 0 on time-out
__device__ __forceinline__ uint64_t wait_tile_flag(const uint64_t* flag, uint32_t call, uint64_t limit_ns,
                                                   volatile uint32_t* err_word) {
  uint64_t w = ld_acquire_sys_u64(flag);
  if (flag_matches(w, call)) return w;
  const long long t0 = clock64();
  const long long limit_clk = (long long)limit_ns * 2;
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    w = ld_acquire_sys_u64(flag);
    if (flag_matches(w, call)) return w;
    if ((it & 7u) == 7u) {
      __nanosleep(64);
      if (clock64() - t0 > limit_clk || *err_word >= (uint32_t)kErrTimeout) return 0;
    }
  }
  return 0;
}

// Moves the `tot` payload bytes packed at obuf[0..tot) to global byte offset `goff` of every
// destination, with aligned 16-byte stores wherever a whole unit belongs to this tile (run by
// `nthr` threads, this one being number `t`).  16 readable guard bytes must precede and follow
// obuf.  All destinations share the same 16-byte phase.
// `mc` (optional): multicast alias of ALL n_dst destinations; whole 16-byte units then leave with one
// multimem store instead of n_dst peer stores, the ragged first/last unit still goes to each peer.
__device__ __forceinline__ void copy_out(const uint8_t* obuf, uint8_t* const* outs, uint32_t n_dst, uint64_t goff,
                                         uint32_t tot, uint32_t t, uint32_t nthr, uint8_t* mc = nullptr) {
  if (tot == 0) return;
  const uint32_t phase = (uint32_t)((reinterpret_cast<uintptr_t>(outs[0]) + goff) & 15u);
  const uint32_t nvec = (phase + tot + 15u) >> 4;
  const uint32_t sh = ((16u - phase) & 3u) * 8u;
  const uint32_t lo_valid = phase, hi_valid = phase + tot;
  auto fetch = [&](uint32_t v, uint32_t (&o)[4]) {  // the 16 bytes of unit v, shifted into place
    const int so = (int)(16u * v) - (int)phase;
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(obuf + (so & ~3));
    const uint32_t w0 = wp[0], w1 = wp[1], w2 = wp[2], w3 = wp[3], w4 = sh ? wp[4] : 0u;
    o[0] = __funnelshift_r(w0, w1, sh);
    o[1] = __funnelshift_r(w1, w2, sh);
    o[2] = __funnelshift_r(w2, w3, sh);
    o[3] = __funnelshift_r(w3, w4, sh);
  };
  auto put = [&](uint32_t v, const uint32_t (&o)[4]) {
    const uint32_t lo = 16u * v, hi = lo + 16u;
    const bool full = lo >= lo_valid && hi <= hi_valid;
    if (full && mc != nullptr) {
      multimem_st_v4(mc + goff - phase + lo, o[0], o[1], o[2], o[3]);
      return;
    }
#pragma unroll 1
    for (uint32_t d = 0; d < n_dst; ++d) {
      uint8_t* p = outs[d] + goff - phase + lo;
      if (full) {
        *reinterpret_cast<uint4*>(p) = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (uint32_t b = 0; b < 16; ++b)
          if (lo + b >= lo_valid && lo + b < hi_valid) p[b] = (uint8_t)(o[b >> 2] >> (8 * (b & 3)));
      }
    }
  };
  for (uint32_t v = t; v < nvec; v += nthr) {
    uint32_t a[4];
    fetch(v, a);
    put(v, a);
  }
}

// 1-D bulk copy global -> shared (TMA unit, no tensor map); both addresses 16-byte aligned, size a
// multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

}  // namespace dev
}  // namespace hc
