// Portable C++ statement of the codec arithmetic: the oracle every GPU kernel is compared with,
// and the codec of the host-rank collectives.  The reference has no CPU codec; this follows the
// behaviour of its kernels (quantiser HomComp/src/GSZ.cu:6-25, block encoder :75-167 and :245-747,
// decoder :883-1469, fused homomorphic add HomComp/src/homcomp.cu:3054-3681) with the defects on
// zero blocks and on "outlier with F = 0" blocks replaced by the intended semantics.
#include <math.h>
#include <string.h>

#include <vector>

#include "hc_format.h"
#include "homcomp_b200.h"

#pragma STDC FP_CONTRACT OFF

namespace {

using namespace hc;

inline int32_t cvt_rzi_sat(float u) {
  if (u != u) return 0;
  if (u >= 2147483648.0f) return INT32_MAX;
  if (u <= -2147483648.0f) return INT32_MIN;
  return (int32_t)u;
}

inline int32_t quantise(float x, float recip) {
  volatile float t = x * recip;  // two roundings, never an FMA
  volatile float u = t + 0.5f;
  int32_t s = (t >= -0.5f) ? 0 : 1;
  return (int32_t)((uint32_t)cvt_rzi_sat(u) - (uint32_t)s);
}

inline int lorenzo_stride(int mode) { return mode == kModeVec ? 4 : 1; }

// deltas of one block of quantised values (wrapping int32)
inline void block_deltas(const int32_t* q, int stride, int32_t* d) {
  for (int i = 0; i < kBlock; ++i) {
    uint32_t prev = i >= stride ? (uint32_t)q[i - stride] : 0u;
    d[i] = (int32_t)((uint32_t)q[i] - prev);
  }
}

inline void put_be32(uint8_t* p, uint32_t w) {
  p[0] = (uint8_t)(w >> 24); p[1] = (uint8_t)(w >> 16); p[2] = (uint8_t)(w >> 8); p[3] = (uint8_t)w;
}
inline uint32_t get_be32(const uint8_t* p) {
  return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | (uint32_t)p[3];
}

// Encodes 32 deltas; returns the rate byte and appends the payload at `out` (>= 128 bytes free).
inline uint32_t encode_block(const int32_t* d, bool allow_outlier, uint8_t* out, uint32_t* len) {
  uint32_t a[kBlock];
  uint32_t sign = 0, or_all = 0, or_tail = 0;
  for (int i = 0; i < kBlock; ++i) {
    a[i] = delta_mag(d[i]);
    if (d[i] < 0) sign |= 1u << (31 - i);
    or_all |= a[i];
    if (i) or_tail |= a[i];
  }
  uint32_t rate = choose_rate(or_all, or_tail, a[0], allow_outlier);
  uint32_t F = rate & 31u;
  uint8_t* p = out;
  bool outl = (rate & 0x80u) != 0;
  if (outl) {
    uint32_t nout = ((rate >> 5) & 3u) + 1u;
    for (uint32_t k = 0; k < nout; ++k) *p++ = (uint8_t)(a[0] >> (8 * k));
    a[0] = 0;
  }
  if (outl || F) {
    put_be32(p, sign);
    p += 4;
    for (uint32_t pl = 0; pl < F; ++pl) {
      uint32_t w = 0;
      for (int i = 0; i < kBlock; ++i) w |= ((a[i] >> pl) & 1u) << (31 - i);
      put_be32(p, w);
      p += 4;
    }
  }
  *len = (uint32_t)(p - out);
  return rate;
}

// Decodes one block's payload to signed deltas.  `avail` = bytes readable at `p`.
inline bool decode_block_deltas(uint32_t rate, const uint8_t* p, size_t avail, int32_t* d) {
  uint32_t len = payload_len(rate);
  if (len > avail) return false;
  uint32_t F = rate & 31u;
  bool outl = (rate & 0x80u) != 0;
  uint32_t a[kBlock];
  memset(a, 0, sizeof(a));
  if (!outl && F == 0) {
    memset(d, 0, kBlock * sizeof(int32_t));
    return true;
  }
  uint32_t a0 = 0;
  if (outl) {
    uint32_t nout = ((rate >> 5) & 3u) + 1u;
    for (uint32_t k = 0; k < nout; ++k) a0 |= (uint32_t)(*p++) << (8 * k);
  }
  uint32_t sign = get_be32(p);
  p += 4;
  for (uint32_t pl = 0; pl < F; ++pl) {
    uint32_t w = get_be32(p);
    p += 4;
    for (int i = 0; i < kBlock; ++i) a[i] |= ((w >> (31 - i)) & 1u) << pl;
  }
  if (outl) a[0] = a0 & 0x7fffffffu;
  for (int i = 0; i < kBlock; ++i) {
    uint32_t neg = (sign >> (31 - i)) & 1u;
    d[i] = (int32_t)(neg ? (0u - a[i]) : a[i]);
  }
  return true;
}

inline void deltas_to_quant(const int32_t* d, int stride, int32_t* q) {
  for (int i = 0; i < kBlock; ++i) {
    uint32_t prev = i >= stride ? (uint32_t)q[i - stride] : 0u;
    q[i] = (int32_t)((uint32_t)d[i] + prev);
  }
}

struct StreamWriter {
  uint8_t* base;
  size_t cap;
  size_t nrate;
  size_t cursor;  // absolute byte position of the next payload
  bool overflow = false;
  StreamWriter(uint8_t* b, size_t c, size_t n) : base(b), cap(c), nrate(rate_bytes(n)), cursor(rate_bytes(n)) {
    if (cap < nrate) overflow = true;
    else memset(base, 0, nrate);
  }
  void emit(size_t blk, uint32_t rate, const uint8_t* payload, uint32_t len) {
    if (overflow) return;
    if (cursor + len > cap) { overflow = true; return; }
    base[blk] = (uint8_t)rate;
    memcpy(base + cursor, payload, len);
    cursor += len;
  }
};

struct StreamReader {
  const uint8_t* base;
  size_t size;
  size_t cursor;
  bool bad = false;
  StreamReader(const uint8_t* b, size_t s, size_t n) : base(b), size(s), cursor(rate_bytes(n)) {
    if (size < cursor) bad = true;
  }
  // signed deltas of block blk; blocks must be read in increasing order
  void next(size_t blk, int32_t* d) {
    if (bad) { memset(d, 0, kBlock * sizeof(int32_t)); return; }
    uint32_t rate = base[blk];
    if (!decode_block_deltas(rate, base + cursor, size - cursor, d)) {
      bad = true;
      memset(d, 0, kBlock * sizeof(int32_t));
      return;
    }
    cursor += payload_len(rate);
  }
};

inline void load_block(const float* x, size_t n, size_t blk, float* v) {
  size_t o = blk * kBlock;
  for (int i = 0; i < kBlock; ++i) v[i] = (o + i < n) ? x[o + i] : 0.0f;
}

}  // namespace

extern "C" {

size_t hc_max_compressed_bytes(size_t n) { return hc::max_stream_bytes(n); }
size_t hc_rate_bytes(size_t n) { return hc::rate_bytes(n); }

int hc_cpu_quantize(const float* x, size_t n, float eb, int32_t* q) {
  float recip = 0.5f / eb;
  for (size_t i = 0; i < n; ++i) q[i] = quantise(x[i], recip);
  return kOk;
}

int hc_cpu_dequantize(const int32_t* q, size_t n, float eb, float* x) {
  for (size_t i = 0; i < n; ++i) {
    volatile float t = (float)q[i] * eb;
    x[i] = t * 2.0f;
  }
  return kOk;
}

// Quantise + Lorenzo only: writes num_blocks(n)*32 int32 deltas (tail of the last block = zeros
// as padding).  Counterpart of kernel_quant_prediction (HomComp/src/homcomp.cu:1553-1602).
int hc_cpu_quant_pred(const float* x, size_t n, float eb, int mode, int32_t* deltas) {
  float recip = 0.5f / eb;
  int stride = lorenzo_stride(mode);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb; ++b) {
    float v[kBlock];
    int32_t q[kBlock];
    load_block(x, n, b, v);
    for (int i = 0; i < kBlock; ++i) q[i] = quantise(v[i], recip);
    block_deltas(q, stride, deltas + b * kBlock);
  }
  return kOk;
}

int hc_cpu_compress(const float* x, size_t n, float eb, int mode, uint8_t* out, size_t cap, size_t* size) {
  if (!(eb > 0.0f) || !out || !size) return kErrArgument;
  float recip = 0.5f / eb;
  int stride = lorenzo_stride(mode);
  StreamWriter w(out, cap, n);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb && !w.overflow; ++b) {
    float v[kBlock];
    int32_t q[kBlock], d[kBlock];
    uint8_t payload[kMaxBlockPayload + 8];
    uint32_t len;
    load_block(x, n, b, v);
    for (int i = 0; i < kBlock; ++i) q[i] = quantise(v[i], recip);
    block_deltas(q, stride, d);
    uint32_t rate = encode_block(d, mode != kModePlain, payload, &len);
    w.emit(b, rate, payload, len);
  }
  if (w.overflow) return kErrCapacity;
  *size = w.cursor;
  return kOk;
}

int hc_cpu_decompress(const uint8_t* in, size_t size, size_t n, float eb, int mode, float* x) {
  if (!in || !x) return kErrArgument;
  int stride = lorenzo_stride(mode);
  StreamReader r(in, size, n);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb; ++b) {
    int32_t d[kBlock], q[kBlock];
    r.next(b, d);
    deltas_to_quant(d, stride, q);
    size_t o = b * kBlock;
    for (int i = 0; i < kBlock && o + i < n; ++i) {
      volatile float t = (float)q[i] * eb;
      x[o + i] = t * 2.0f;
    }
  }
  return r.bad ? kErrTruncated : kOk;
}

// Decode to quantised integers (inverse Lorenzo applied, no dequantisation).
int hc_cpu_decode_quant(const uint8_t* in, size_t size, size_t n, int mode, int32_t* q_out) {
  int stride = lorenzo_stride(mode);
  StreamReader r(in, size, n);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb; ++b) {
    int32_t d[kBlock], q[kBlock];
    r.next(b, d);
    deltas_to_quant(d, stride, q);
    size_t o = b * kBlock;
    for (int i = 0; i < kBlock && o + i < n; ++i) q_out[o + i] = q[i];
  }
  return r.bad ? kErrTruncated : kOk;
}

// stream (+) fp32 -> stream, in the delta domain.  Intended semantics of kernel_homomophic_sum_F.
int hc_cpu_hom_add_f32(const uint8_t* in, size_t in_size, const float* local, size_t n, float eb, int mode,
                       uint8_t* out, size_t cap, size_t* size) {
  if (!(eb > 0.0f)) return kErrArgument;
  float recip = 0.5f / eb;
  int stride = lorenzo_stride(mode);
  StreamReader r(in, in_size, n);
  StreamWriter w(out, cap, n);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb && !w.overflow; ++b) {
    float v[kBlock];
    int32_t q[kBlock], dl[kBlock], di[kBlock];
    uint8_t payload[kMaxBlockPayload + 8];
    uint32_t len;
    r.next(b, di);
    load_block(local, n, b, v);
    for (int i = 0; i < kBlock; ++i) q[i] = quantise(v[i], recip);
    block_deltas(q, stride, dl);
    for (int i = 0; i < kBlock; ++i) di[i] = (int32_t)((uint32_t)di[i] + (uint32_t)dl[i]);
    uint32_t rate = encode_block(di, mode != kModePlain, payload, &len);
    w.emit(b, rate, payload, len);
  }
  if (w.overflow) return kErrCapacity;
  *size = w.cursor;
  return r.bad ? kErrTruncated : kOk;
}

// stream (+) precomputed int32 deltas -> stream.  Intended semantics of kernel_homomophic_sum
// (HomComp/src/homcomp.cu:1604-2921, add step :2249-2268).
int hc_cpu_hom_add_i32(const uint8_t* in, size_t in_size, const int32_t* deltas, size_t n, int mode, uint8_t* out,
                       size_t cap, size_t* size) {
  StreamReader r(in, in_size, n);
  StreamWriter w(out, cap, n);
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb && !w.overflow; ++b) {
    int32_t di[kBlock];
    uint8_t payload[kMaxBlockPayload + 8];
    uint32_t len;
    r.next(b, di);
    const int32_t* dl = deltas + b * kBlock;
    for (int i = 0; i < kBlock; ++i) di[i] = (int32_t)((uint32_t)di[i] + (uint32_t)dl[i]);
    uint32_t rate = encode_block(di, mode != kModePlain, payload, &len);
    w.emit(b, rate, payload, len);
  }
  if (w.overflow) return kErrCapacity;
  *size = w.cursor;
  return r.bad ? kErrTruncated : kOk;
}

// stream (+) stream -> stream (not in the reference; used by the one-shot allreduce).
int hc_cpu_hom_add_stream(const uint8_t* a, size_t a_size, const uint8_t* b, size_t b_size, size_t n, int mode,
                          uint8_t* out, size_t cap, size_t* size) {
  StreamReader ra(a, a_size, n), rb(b, b_size, n);
  StreamWriter w(out, cap, n);
  size_t nb = num_blocks(n);
  for (size_t k = 0; k < nb && !w.overflow; ++k) {
    int32_t da[kBlock], db[kBlock];
    uint8_t payload[kMaxBlockPayload + 8];
    uint32_t len;
    ra.next(k, da);
    rb.next(k, db);
    for (int i = 0; i < kBlock; ++i) da[i] = (int32_t)((uint32_t)da[i] + (uint32_t)db[i]);
    uint32_t rate = encode_block(da, mode != kModePlain, payload, &len);
    w.emit(k, rate, payload, len);
  }
  if (w.overflow) return kErrCapacity;
  *size = w.cursor;
  return (ra.bad || rb.bad) ? kErrTruncated : kOk;
}

// True length of a stream from its rate bytes alone.
int hc_cpu_stream_size(const uint8_t* in, size_t avail, size_t n, size_t* size) {
  size_t nr = rate_bytes(n);
  if (avail < nr) return kErrTruncated;
  size_t total = nr;
  size_t nb = num_blocks(n);
  for (size_t b = 0; b < nb; ++b) total += payload_len(in[b]);
  *size = total;
  return total <= avail ? kOk : kErrTruncated;
}

}  // extern "C"
