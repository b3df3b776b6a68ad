// Checks of the reference-named entry points (homcomp_compat.h) that need no second GPU:
//   * round trip through GSZ_compress_deviceptr_outlier / GSZ_decompress_deviceptr_outlier and the
//     fused homomorphic_sum_F on compressible data;
//   * incompressible data (finite values whose deltas need 31 bit planes in every block, i.e. 129
//     stream bytes per 128 input bytes) with a canary behind the output buffer: under the default
//     capacity rule (nbEle * 4 bytes, what the reference's callers allocate) the stream is cut off and
//     status 1 reported, with hc_compat_set_capacity_rule(1) it is stored whole; in neither case is a
//     byte written past the assumed capacity.
// Prints one line per check and "ok" at the end; exit code 0 only if everything held.
//
//   compat_check [count]
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "homcomp_compat.h"

static int g_fail = 0;
static void check(bool ok, const char* what) {
  printf("%-72s %s\n", what, ok ? "pass" : "FAIL");
  if (!ok) g_fail = 1;
}

static bool canary_intact(const unsigned char* d_buf, size_t from, size_t len) {
  std::vector<unsigned char> h(len);
  cudaMemcpy(h.data(), d_buf + from, len, cudaMemcpyDeviceToHost);
  for (size_t i = 0; i < len; ++i)
    if (h[i] != 0xA5) return false;
  return true;
}

int main(int argc, char** argv) {
  const size_t n = argc > 1 ? (size_t)atoll(argv[1]) : 1000003;
  const float eb = 1e-4f;
  const size_t cap_max = hc_max_compressed_bytes(n), canary = 4096;
  std::vector<float> h(n), back(n);
  float *d_x = nullptr, *d_y = nullptr;
  unsigned char *d_c = nullptr, *d_c2 = nullptr;
  cudaMalloc(&d_x, n * sizeof(float));
  cudaMalloc(&d_y, n * sizeof(float));
  cudaMalloc(&d_c, cap_max + canary);
  cudaMalloc(&d_c2, cap_max + canary);

  // ---- compressible data: round trip and fused add ---------------------------------------------
  for (size_t i = 0; i < n; ++i) h[i] = 0.5f * sinf(0.001f * (float)i) + 0.001f * (float)((i * 2654435761u) % 1000) / 1000.f;
  cudaMemcpy(d_x, h.data(), n * sizeof(float), cudaMemcpyHostToDevice);
  size_t sz = 0, sz2 = 0;
  GSZ_compress_deviceptr_outlier(d_x, d_c, n, &sz, eb);
  check(sz > hc_rate_bytes(n) && sz < n * sizeof(float), "compress: size between the rate bytes and the input size");
  cudaMemset(d_y, 0x7f, n * sizeof(float));
  GSZ_decompress_deviceptr_outlier(d_y, d_c, n, sz, eb);
  cudaMemcpy(back.data(), d_y, n * sizeof(float), cudaMemcpyDeviceToHost);
  double worst = 0;
  for (size_t i = 0; i < n; ++i) worst = fmax(worst, fabs((double)back[i] - (double)h[i]));
  check(worst <= eb * 1.01, "decompress: every value within the error bound (plus fp32 rounding)");
  homomorphic_sum_F(d_c, d_x, d_c2, n, eb, &sz2, sz);
  GSZ_decompress_deviceptr_outlier(d_y, d_c2, n, sz2, eb);
  cudaMemcpy(back.data(), d_y, n * sizeof(float), cudaMemcpyDeviceToHost);
  worst = 0;
  for (size_t i = 0; i < n; ++i) worst = fmax(worst, fabs((double)back[i] - 2.0 * (double)h[i]));
  check(worst <= 2 * eb * 1.01, "homomorphic_sum_F: x (+) x within two error bounds of 2x");
  check(hc_compat_last_status == 0, "no status reported so far");

  // ---- incompressible data -----------------------------------------------------------------------
  // alternating +-(2^29 + noise) * 2 eb: every delta inside a block has a magnitude just above 2^30,
  // 31 bit planes; values stay finite and inside the codec's contract (|x| / (2 eb) < 2^30)
  for (size_t i = 0; i < n; ++i) {
    const float mag = (float)((1u << 29) + 1024 + (unsigned)((i * 40503u) % 4096)) * (2.0f * eb);
    h[i] = (i & 1) ? -mag : mag;
  }
  cudaMemcpy(d_x, h.data(), n * sizeof(float), cudaMemcpyHostToDevice);
  const size_t cap_ref = n * sizeof(float);
  cudaMemset(d_c, 0xA5, cap_max + canary);
  sz = 12345;
  GSZ_compress_deviceptr_outlier(d_x, d_c, n, &sz, eb);  // default rule: the buffer holds nbEle * 4 bytes
  check(hc_compat_last_status == 1, "incompressible input, default rule: status 1 (capacity) reported");
  check(sz == 0, "incompressible input, default rule: *cmpSize is 0");
  check(canary_intact(d_c, cap_ref, cap_max + canary - cap_ref), "incompressible input, default rule: nothing written past nbEle * 4 bytes");
  hc_compat_last_status = 0;
  hc_compat_set_capacity_rule(1);
  cudaMemset(d_c, 0xA5, cap_max + canary);
  GSZ_compress_deviceptr_outlier(d_x, d_c, n, &sz, eb);
  check(hc_compat_last_status == 0, "incompressible input, rule 1: stored without an error");
  check(sz > n * sizeof(float) && sz <= cap_max, "incompressible input, rule 1: stream longer than the input, within the bound");
  check(canary_intact(d_c, cap_max, canary), "incompressible input, rule 1: nothing written past hc_max_compressed_bytes");
  cudaMemset(d_y, 0, n * sizeof(float));
  GSZ_decompress_deviceptr_outlier(d_y, d_c, n, sz, eb);
  cudaMemcpy(back.data(), d_y, n * sizeof(float), cudaMemcpyDeviceToHost);
  worst = 0;
  for (size_t i = 0; i < n; ++i) worst = fmax(worst, fabs((double)back[i] - (double)h[i]) / fabs((double)h[i]));
  check(worst <= 1e-6, "incompressible input: decodes to the input within fp32 rounding of the large values");
  hc_compat_set_capacity_rule(0);

  cudaFree(d_x);
  cudaFree(d_y);
  cudaFree(d_c);
  cudaFree(d_c2);
  if (cudaDeviceSynchronize() != cudaSuccess) g_fail = 1;
  printf("%s\n", g_fail ? "FAILED" : "ok");
  return g_fail;
}
