// In-register bit-plane transposition for one 32-element block held by ONE thread.
//
// The stream stores a block's magnitudes as F bit planes: plane p is a big-endian 32-bit map in
// which element i sits at bit 31 - i.  Read as a little-endian machine word, element i therefore
// sits at bit (i ^ 7).  With rows A[j] = mag[j ^ 7] (a compile-time renaming of registers) the
// planes are exactly the 32x32 bit-matrix transpose:  T[p] bit j = A[j] bit p.
//
// The transpose is five independent stages (one per index bit); stage `s` swaps bit s of the row
// index with bit s of the column index.  Stages 16 and 8 are byte permutes (PRMT), stages 4, 2, 1
// are shift-xor swaps.  When every magnitude of the block fits W bits (W = 4, 8, 16) the upper rows
// of the result are known zero and most of the network disappears, which is what makes the
// thread-per-block layout cheaper than one warp ballot per plane: cost is ~2.6 (W=8) to ~9.5 (W=32)
// integer instructions per element, independent of F.
//
// The reference packs planes with 32 shift/or pairs per output byte (HomComp/src/GSZ.cu:1698-1735).
#pragma once
#include "hc_format.h"

namespace hc {

HC_HD uint32_t perm(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(a, b, sel);
#else
  uint64_t v = ((uint64_t)b << 32) | a;
  uint32_t r = 0;
  for (int k = 0; k < 4; ++k) r |= (uint32_t)((v >> (8 * ((sel >> (4 * k)) & 7))) & 0xff) << (8 * k);
  return r;
#endif
}

// swap the bits of A[k] selected by (m << s) with the bits of A[k + s] selected by m
template <int S>
HC_HD void swap_stage(uint32_t& lo, uint32_t& hi) {
  constexpr uint32_t m = S == 4 ? 0x0f0f0f0fu : (S == 2 ? 0x33333333u : 0x55555555u);
  uint32_t t = ((lo >> S) ^ hi) & m;
  hi ^= t;
  lo ^= t << S;
}

// Forward: rows A[0..31] hold values below 2^W; on return A[0..W-1] hold planes 0..W-1.
// Rows W..31 are unspecified afterwards.
template <int W>
HC_HD void planes_from_rows(uint32_t (&A)[32]) {
  static_assert(W == 4 || W == 8 || W == 16 || W == 32, "W");
  // stage 16
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    uint32_t lo = A[k], hi = A[k + 16];
    A[k] = perm(lo, hi, 0x5410);
    if (W > 16) A[k + 16] = perm(lo, hi, 0x7632);
  }
  // stage 8
#pragma unroll
  for (int h = 0; h < (W > 16 ? 32 : 16); h += 16) {
#pragma unroll
    for (int k = h; k < h + 8; ++k) {
      uint32_t lo = A[k], hi = A[k + 8];
      A[k] = perm(lo, hi, 0x6240);
      if (W > 8) A[k + 8] = perm(lo, hi, 0x7351);
    }
  }
  constexpr int R = W;  // live rows from here on
  // stage 4
  if (W == 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k) A[k] = (A[k] & 0x0f0f0f0fu) | ((A[k + 4] << 4) & 0xf0f0f0f0u);
  } else {
#pragma unroll
    for (int k = 0; k < R; ++k)
      if ((k & 4) == 0) swap_stage<4>(A[k], A[k + 4]);
  }
#pragma unroll
  for (int k = 0; k < R; ++k)
    if ((k & 2) == 0) swap_stage<2>(A[k], A[k + 2]);
#pragma unroll
  for (int k = 0; k < R; ++k)
    if ((k & 1) == 0) swap_stage<1>(A[k], A[k + 1]);
}

// Inverse: A[0..W-1] hold planes 0..W-1 (planes >= F are zero); on return A[0..31] are the rows.
// Entries A[W..31] are ignored on input.
template <int W>
HC_HD void rows_from_planes(uint32_t (&A)[32]) {
  static_assert(W == 4 || W == 8 || W == 16 || W == 32, "W");
  constexpr int R = W;
#pragma unroll
  for (int k = 0; k < R; ++k)
    if ((k & 1) == 0) swap_stage<1>(A[k], A[k + 1]);
#pragma unroll
  for (int k = 0; k < R; ++k)
    if ((k & 2) == 0) swap_stage<2>(A[k], A[k + 2]);
  if (W == 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t v = A[k];
      A[k] = v & 0x0f0f0f0fu;
      A[k + 4] = (v >> 4) & 0x0f0f0f0fu;
    }
  } else {
#pragma unroll
    for (int k = 0; k < R; ++k)
      if ((k & 4) == 0) swap_stage<4>(A[k], A[k + 4]);
  }
  // stage 8
#pragma unroll
  for (int h = 0; h < (W > 16 ? 32 : 16); h += 16) {
#pragma unroll
    for (int k = h; k < h + 8; ++k) {
      uint32_t lo = A[k], hi = (W > 8) ? A[k + 8] : 0u;
      A[k] = perm(lo, hi, 0x6240);
      A[k + 8] = perm(lo, hi, 0x7351);
    }
  }
  // stage 16
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    uint32_t lo = A[k], hi = (W > 16) ? A[k + 16] : 0u;
    A[k] = perm(lo, hi, 0x5410);
    A[k + 16] = perm(lo, hi, 0x7632);
  }
}

// smallest supported width that holds F planes (F in 0..31); 0 means "no planes at all"
HC_HD int plane_width(uint32_t F) { return F == 0 ? 0 : (F <= 4 ? 4 : (F <= 8 ? 8 : (F <= 16 ? 16 : 32))); }

}  // namespace hc
