// Single-GPU evaluation tool: compress a float32 data set, add it to itself on the compressed
// stream (fused homomorphic add) and by decompress-operate-compress, report timings, compression
// ratio and error metrics.  Counterpart of HomComp/src/homcomp_eval.cu:135-236, written against the
// reference-named API (homcomp_compat.h) with CUDA-event timing.
//
//   homcomp_eval <file.bin | gen:N> [eb] [REL|ABS] [iterations]
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "homcomp_compat.h"

static void error_evaluation(const std::vector<float>& ref, const std::vector<float>& rec, size_t cmp_bytes) {
  double maxerr = 0, maxrel = 0, mse = 0, mn = ref[0], mx = ref[0], sa = 0, sb = 0;
  const size_t n = ref.size();
  for (size_t i = 0; i < n; ++i) {
    double a = ref[i], b = rec[i], e = fabs(a - b);
    if (e > maxerr) maxerr = e;
    if (a != 0 && e / fabs(a) > maxrel) maxrel = e / fabs(a);
    mse += e * e;
    if (a < mn) mn = a;
    if (a > mx) mx = a;
    sa += a;
    sb += b;
  }
  mse /= n;
  const double range = mx - mn, ma = sa / n, mb = sb / n;
  double cov = 0, va = 0, vb = 0;
  for (size_t i = 0; i < n; ++i) {
    cov += (ref[i] - ma) * (rec[i] - mb);
    va += (ref[i] - ma) * (ref[i] - ma);
    vb += (rec[i] - mb) * (rec[i] - mb);
  }
  printf("max abs err %.6g | max rel err %.6g | PSNR %.3f dB | NRMSE %.6g | Pearson %.9f | CR %.3f\n", maxerr, maxrel,
         20 * log10(range) - 10 * log10(mse), sqrt(mse) / range, cov / sqrt(va * vb), 4.0 * n / cmp_bytes);
}

__global__ void add_arrays(float* a, const float* b, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) a[i] += b[i];
}

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "usage: %s <file.bin | gen:N> [eb=1e-4] [ABS|REL] [iterations=10]\n", argv[0]);
    return 2;
  }
  std::vector<float> host;
  if (strncmp(argv[1], "gen:", 4) == 0) {
    size_t n = (size_t)atoll(argv[1] + 4);
    host.resize(n);
    unsigned s = 12345u;
    double walk = 0;
    for (size_t i = 0; i < n; ++i) {  // smooth random walk
      s = s * 1664525u + 1013904223u;
      walk += ((double)(s >> 8) / (1 << 24) - 0.5) * 1e-2;
      host[i] = (float)(sin(i * 1e-4) + walk * 1e-2);
    }
  } else {
    size_t n = 0;
    float* p = read_binary_floats(argv[1], &n);
    if (!p) {
      fprintf(stderr, "cannot read %s\n", argv[1]);
      return 1;
    }
    host.assign(p, p + n);
    free(p);
  }
  float eb = argc > 2 ? (float)atof(argv[2]) : 1e-4f;
  if (argc > 3 && strcmp(argv[3], "REL") == 0) {
    float mn = host[0], mx = host[0];
    for (float v : host) { mn = v < mn ? v : mn; mx = v > mx ? v : mx; }
    eb *= (mx - mn);
  }
  const int iters = argc > 4 ? atoi(argv[4]) : 10;
  const size_t n = host.size(), cap = hc_max_compressed_bytes(n);
  float *d_x, *d_tmp;
  unsigned char *d_c, *d_c2;
  cudaMalloc(&d_x, n * 4);
  cudaMalloc(&d_tmp, n * 4);
  cudaMalloc(&d_c, cap);
  cudaMalloc(&d_c2, cap);
  cudaMemcpy(d_x, host.data(), n * 4, cudaMemcpyHostToDevice);
  size_t sz = 0, sz2 = 0;
  GSZ_compress_deviceptr_outlier(d_x, d_c, n, &sz, eb);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float ms_fused = 0, ms_doc = 0, ms;
  for (int it = 0; it < iters + 1; ++it) {
    cudaEventRecord(e0);
    homomorphic_sum_F(d_c, d_x, d_c2, n, eb, &sz2, sz);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    if (it) ms_fused += ms;
    cudaEventRecord(e0);
    GSZ_decompress_deviceptr_outlier(d_tmp, d_c, n, sz, eb);
    add_arrays<<<1184, 256>>>(d_tmp, d_x, n);
    size_t sz3 = 0;
    GSZ_compress_deviceptr_outlier(d_tmp, d_c2, n, &sz3, eb);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    if (it) ms_doc += ms;
  }
  homomorphic_sum_F(d_c, d_x, d_c2, n, eb, &sz2, sz);
  GSZ_decompress_deviceptr_outlier(d_tmp, d_c2, n, sz2, eb);
  std::vector<float> rec(n), twice(n);
  cudaMemcpy(rec.data(), d_tmp, n * 4, cudaMemcpyDeviceToHost);
  for (size_t i = 0; i < n; ++i) twice[i] = 2 * host[i];
  printf("n %zu eb %g | compressed %zu B | hom-add stream %zu B\n", n, eb, sz, sz2);
  printf("fused homomorphic add: %.3f ms (%.1f GB/s) | decompress+add+compress: %.3f ms (%.1f GB/s) | speedup %.2fx\n",
         ms_fused / iters, 4e-6 * n / (ms_fused / iters), ms_doc / iters, 4e-6 * n / (ms_doc / iters), ms_doc / ms_fused);
  error_evaluation(twice, rec, sz2);
  cudaError_t err = cudaDeviceSynchronize();
  printf("status %s\n", cudaGetErrorString(err));
  return err == cudaSuccess ? 0 : 1;
}
