// Host-rank ring allreduce over the CPU codec: P ranks simulated in one process.  Same partition,
// hop order and arithmetic as the device ring, so its output is the bit-exact expectation for the
// multi-GPU collectives.  Algorithm of allreduce_ring_comprs_hom_sum_F
// (HomComp/src/cuda_awareallreduce.cu:166-264): compressed ring reduce-scatter with a homomorphic
// add per hop, then distribution of the reduced compressed chunks, decoded once per rank.
#include <string.h>

#include <vector>

#include "hc_format.h"
#include "homcomp_b200.h"

extern "C" {

size_t hc_chunk_elems(size_t count, int P) {
  if (P <= 0) return 0;
  size_t per = (count + (size_t)P - 1) / (size_t)P;
  return (per + hc::kBlock - 1) / hc::kBlock * hc::kBlock;
}

int hc_cpu_ring_allreduce(const float* const* bufs, float* const* outs, int P, size_t count, float eb,
                          size_t* hop_bytes) {
  if (P <= 0 || !(eb > 0.0f)) return hc::kErrArgument;
  const size_t B = hc_chunk_elems(count, P);
  auto chunk_len = [&](int c) -> size_t {
    size_t lo = (size_t)c * B;
    if (lo >= count) return 0;
    size_t hi = lo + B;
    return (hi > count ? count : hi) - lo;
  };
  const size_t cap = hc::max_stream_bytes(B) + 16;
  // inflight[r] = stream rank r produced in the previous step
  std::vector<std::vector<uint8_t>> cur(P, std::vector<uint8_t>(cap)), nxt(P, std::vector<uint8_t>(cap));
  std::vector<size_t> cur_size(P), nxt_size(P);
  int rc = hc::kOk;
  for (int r = 0; r < P; ++r) {
    size_t n = chunk_len(r);
    int e = hc_cpu_compress(bufs[r] + (size_t)r * B, n, eb, hc::kModeOutlier, cur[r].data(), cap, &cur_size[r]);
    if (e) rc = e;
    if (hop_bytes) hop_bytes[(size_t)r * P + 0] = cur_size[r];
  }
  for (int s = 1; s < P; ++s) {
    for (int r = 0; r < P; ++r) {
      int from = (r - 1 + P) % P;
      int c = ((r - s) % P + P) % P;
      size_t n = chunk_len(c);
      int e = hc_cpu_hom_add_f32(cur[from].data(), cur_size[from], bufs[r] + (size_t)c * B, n, eb, hc::kModeOutlier,
                                 nxt[r].data(), cap, &nxt_size[r]);
      if (e) rc = e;
      if (hop_bytes) hop_bytes[(size_t)r * P + s] = nxt_size[r];
    }
    cur.swap(nxt);
    cur_size.swap(nxt_size);
  }
  // rank r now owns the reduced stream of chunk (r + 1) mod P (chunk r when P == 1)
  for (int r = 0; r < P; ++r) {
    int c = (r + 1) % P;
    size_t n = chunk_len(c);
    for (int dst = 0; dst < P; ++dst) {
      int e = hc_cpu_decompress(cur[r].data(), cur_size[r], n, eb, hc::kModeOutlier, outs[dst] + (size_t)c * B);
      if (e) rc = e;
    }
  }
  return rc;
}

}  // extern "C"
