// Stream format shared by the CPU oracle and the sm_100a kernels.
//
// A compressed stream of n fp32 values (absolute error bound eb) is
//   section A: one "rate" byte per 32-element block, for ceil(n/32768)*1024 blocks
//   section B: the blocks' payloads, concatenated in block order
// The layout is the Outlier-FLE layout of the reference codec
// (HomComp/src/GSZ.cu:33-756 encode, :758-1473 decode), so streams are interchangeable.
//
// Rate byte: bit7 = outlier mode, bits6..5 = outlier byte count - 1, bits4..0 = F (bit planes).
// Plain payload (F > 0):  BE32 sign map, then F planes (LSB plane first), BE32 each.
// Outlier payload:        |d0| in nOut little-endian bytes, BE32 sign map, F planes (element 0's
//                         plane bit is 0).
// In a BE32 map, element i of the block sits at bit (31 - i).
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define HC_HD __host__ __device__ __forceinline__
#else
#define HC_HD inline
#endif

namespace hc {

constexpr int kBlock = 32;             // elements per block
constexpr int kChunk = 32768;          // elements per chunk (section A is padded to whole chunks)
constexpr int kBlocksPerChunk = kChunk / kBlock;
constexpr int kMaxBlockPayload = 128;  // 4 + 4*31 bytes

enum Mode : int {
  kModeOutlier = 0,  // per-block choice between plain and outlier layout (HomComp/src/GSZ.cu:152-164)
  kModePlain = 1,    // always the plain layout (HomComp/src/GSZ.cu:1475-1747)
  kModeVec = 2,      // stride-4 Lorenzo predictor (HomComp/src/homcomp.cu:143-146); own stream family
};

enum Status : int {
  kOk = 0,
  kErrCapacity = 1,     // output buffer too small for the stream
  kErrTruncated = 2,    // input stream shorter than its rate bytes imply
  kErrTimeout = 3,      // a bounded device-side wait ran out
  kErrArgument = 4,
  kErrCuda = 5,
  kErrPeer = 6,         // a peer reported failure or never arrived
};

HC_HD size_t num_chunks(size_t n) { return (n + kChunk - 1) / kChunk; }
HC_HD size_t num_blocks(size_t n) { return (n + kBlock - 1) / kBlock; }
// blocks that own a rate byte (section A length)
HC_HD size_t rate_bytes(size_t n) { return num_chunks(n) * kBlocksPerChunk; }
// capacity that can never overflow: every block at 1 + 128 bytes
HC_HD size_t max_stream_bytes(size_t n) { return rate_bytes(n) + num_blocks(n) * (size_t)kMaxBlockPayload; }

HC_HD int bit_width(uint32_t v) {
#if defined(__CUDA_ARCH__)
  return 32 - __clz((int)v);
#else
  return v ? 32 - __builtin_clz(v) : 0;
#endif
}

// payload length implied by a rate byte
HC_HD uint32_t payload_len(uint32_t rate) {
  uint32_t F = rate & 31u;
  if (rate & 0x80u) return 4u + 4u * F + ((rate >> 5) & 3u) + 1u;
  return F ? 4u + 4u * F : 0u;
}

// Mode choice and rate byte from the OR of the magnitudes (same top bit as the max):
//   or_all  = OR of |d_0..d_31|,  or_tail = OR of |d_1..d_31|,  a0 = |d_0|.
// mode kModePlain forces the plain layout.
HC_HD uint32_t choose_rate(uint32_t or_all, uint32_t or_tail, uint32_t a0, bool allow_outlier) {
  uint32_t fr1 = (uint32_t)bit_width(or_all);
  uint32_t fr2 = (uint32_t)bit_width(or_tail);
  uint32_t nout = ((uint32_t)bit_width(a0) + 7u) >> 3;
  uint32_t s1 = fr1 ? 4u + 4u * fr1 : 0u;
  uint32_t s2 = 4u + 4u * fr2 + nout;
  if (!allow_outlier || s1 <= s2) return fr1;
  return 0x80u | ((nout - 1u) << 5) | fr2;
}

// Magnitude and sign of a delta.  Deltas live in wrapping int32; the magnitude keeps 31 bits so F
// never reaches 32 (INT_MIN folds to -0).  Inputs with |x| / (2 eb) >= 2^30 are outside the contract.
HC_HD uint32_t delta_mag(int32_t d) {
  uint32_t u = (uint32_t)d;
  uint32_t a = d < 0 ? (0u - u) : u;
  return a & 0x7fffffffu;
}

}  // namespace hc
