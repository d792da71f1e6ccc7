// SPDX-License-Identifier: MIT
//
// stock_d2d -- library baselines for a GPU-to-GPU copy: cudaMemcpyPeerAsync
// (copy engine over NVLink) and staging through pinned host memory, both
// directions, 4 KiB .. 256 MiB.  Counterpart of the reference's
// bench/stock-d2d/stock-d2d.cu:27-62 (what a stock driver offers without the
// library).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      exit(1);                                                                         \
    }                                                                                  \
  } while (0)

int main() {
  int n = 0;
  CK(cudaGetDeviceCount(&n));
  if (n < 2) {
    fprintf(stderr, "stock_d2d needs two GPUs\n");
    return 2;
  }
  const size_t maxb = 256u << 20;
  void *d0, *d1, *h;
  CK(cudaSetDevice(0));
  CK(cudaMalloc(&d0, maxb));
  cudaDeviceEnablePeerAccess(1, 0);
  CK(cudaSetDevice(1));
  CK(cudaMalloc(&d1, maxb));
  cudaDeviceEnablePeerAccess(0, 0);
  cudaGetLastError();
  CK(cudaMallocHost(&h, maxb));
  CK(cudaSetDevice(0));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));
  cudaEvent_t a, b;
  CK(cudaEventCreate(&a));
  CK(cudaEventCreate(&b));
  printf("%12s %16s %16s %18s\n", "bytes", "peer 0->1", "peer 1->0", "pinned staging 0->1");
  for (size_t bytes = 4096; bytes <= maxb; bytes *= 4) {
    const int iters = bytes >= (64u << 20) ? 20 : 200;
    float ms[3];
    for (int mode = 0; mode < 3; ++mode) {
      for (int w = 0; w < 3; ++w) {
        if (mode == 0) CK(cudaMemcpyPeerAsync(d1, 1, d0, 0, bytes, st));
        else if (mode == 1) CK(cudaMemcpyPeerAsync(d0, 0, d1, 1, bytes, st));
        else {
          CK(cudaMemcpyAsync(h, d0, bytes, cudaMemcpyDeviceToHost, st));
          CK(cudaMemcpyAsync(d1, h, bytes, cudaMemcpyHostToDevice, st));
        }
      }
      CK(cudaStreamSynchronize(st));
      CK(cudaEventRecord(a, st));
      for (int i = 0; i < iters; ++i) {
        if (mode == 0) CK(cudaMemcpyPeerAsync(d1, 1, d0, 0, bytes, st));
        else if (mode == 1) CK(cudaMemcpyPeerAsync(d0, 0, d1, 1, bytes, st));
        else {
          CK(cudaMemcpyAsync(h, d0, bytes, cudaMemcpyDeviceToHost, st));
          CK(cudaMemcpyAsync(d1, h, bytes, cudaMemcpyHostToDevice, st));
        }
      }
      CK(cudaEventRecord(b, st));
      CK(cudaEventSynchronize(b));
      CK(cudaEventElapsedTime(&ms[mode], a, b));
      ms[mode] /= iters;
    }
    printf("%12zu %11.1f GB/s %11.1f GB/s %13.1f GB/s\n", bytes, bytes / ms[0] / 1e6, bytes / ms[1] / 1e6,
           bytes / ms[2] / 1e6);
  }
  return 0;
}
