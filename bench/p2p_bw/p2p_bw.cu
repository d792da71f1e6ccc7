// SPDX-License-Identifier: MIT
//
// p2p_bw -- raw NVLink peer-memory benchmark with byte verification.
//
// Role of the reference's bench/bar1-p2p-write/main.cu (link bring-up, Phase-1
// byte proof, Phase-2 bandwidth sweep 4 KiB..64 MiB, --both/--reverse), for a
// box where peer memory is plain CUDA: one process, two GPUs, kernels on the
// writer GPU store straight into (or load straight from) the other GPU's
// memory.  Phases:
//   1. verify: pattern written through the peer mapping, checked by the owner
//   2. bandwidth: kernel P2P write, kernel P2P read, copy-engine peer copy,
//      4 KiB .. 1 GiB, device-timed
//   3. latency: flag ping-pong between the two GPUs (one kernel per GPU,
//      different GPUs, bounded spins)
//
//   p2p_bw [--src A] [--dst B] [--both] [--max-mb N] [--iters N]
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      exit(1);                                                                         \
    }                                                                                  \
  } while (0)

__device__ __forceinline__ uint32_t pat(uint64_t i, uint32_t seed) {
  uint64_t x = i * 0x9E3779B97F4A7C15ull + seed;
  x ^= x >> 31;
  x *= 0xBF58476D1CE4E5B9ull;
  return uint32_t(x >> 16);
}

__global__ void k_write(uint4* dst, size_t n, uint32_t seed) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    dst[i] = make_uint4(pat(4 * i, seed), pat(4 * i + 1, seed), pat(4 * i + 2, seed), pat(4 * i + 3, seed));
}
__global__ void k_check(const uint4* src, size_t n, uint32_t seed, unsigned long long* bad) {
  unsigned long long b = 0;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    b += (v.x != pat(4 * i, seed)) + (v.y != pat(4 * i + 1, seed)) + (v.z != pat(4 * i + 2, seed)) +
         (v.w != pat(4 * i + 3, seed));
  }
  if (b) atomicAdd(bad, b * 4);
}
__global__ void k_copy(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}
// ping-pong on two flags, each in the memory of the GPU that waits on it
__global__ void k_pingpong(volatile uint32_t* mine, volatile uint32_t* theirs, int iters, int first,
                           unsigned long long* ns, int* gave_up) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (int i = 1; i <= iters; ++i) {
    if (first) {
      *theirs = uint32_t(i);
      __threadfence_system();
    }
    unsigned spins = 0;
    while (*mine < uint32_t(i)) {
      if (++spins > (1u << 26)) {  // bounded: report and leave
        *gave_up = i;
        return;
      }
    }
    if (!first) {
      *theirs = uint32_t(i);
      __threadfence_system();
    }
  }
  unsigned long long t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  *ns = (t1 - t0) / (unsigned long long)iters;
}

static float time_ms(cudaStream_t st, int iters, void (*fn)(void*), void* arg) {
  cudaEvent_t a, b;
  CK(cudaEventCreate(&a));
  CK(cudaEventCreate(&b));
  for (int i = 0; i < 3; ++i) fn(arg);
  CK(cudaStreamSynchronize(st));
  CK(cudaEventRecord(a, st));
  for (int i = 0; i < iters; ++i) fn(arg);
  CK(cudaEventRecord(b, st));
  CK(cudaEventSynchronize(b));
  float ms = 0;
  CK(cudaEventElapsedTime(&ms, a, b));
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return ms / iters;
}

struct Job {
  const uint4* src;
  uint4* dst;
  size_t n;
  cudaStream_t st;
  int dst_dev, src_dev;
};
static void run_kernel(void* p) {
  Job* j = (Job*)p;
  size_t blocks = (j->n + 511) / 512;
  if (blocks > 148 * 8) blocks = 148 * 8;
  k_copy<<<(unsigned)blocks, 512, 0, j->st>>>(j->src, j->dst, j->n);
}
static void run_ce(void* p) {
  Job* j = (Job*)p;
  cudaMemcpyPeerAsync(j->dst, j->dst_dev, j->src, j->src_dev, j->n * 16, j->st);
}

static void direction(int a, int b, size_t max_bytes, int iters) {
  printf("\n== GPU %d -> GPU %d ==\n", a, b);
  uint4 *la, *rb;
  unsigned long long* bad;
  CK(cudaSetDevice(a));
  CK(cudaMalloc(&la, max_bytes));
  CK(cudaSetDevice(b));
  CK(cudaMalloc(&rb, max_bytes));
  CK(cudaMallocManaged(&bad, 8));
  *bad = 0;
  // phase 1: byte proof through the peer mapping
  const size_t vn = (max_bytes < (64u << 20) ? max_bytes : (64u << 20)) / 16;
  CK(cudaSetDevice(a));
  k_write<<<148 * 4, 512>>>(rb, vn, 0x1234u + a);
  CK(cudaDeviceSynchronize());
  CK(cudaSetDevice(b));
  k_check<<<148 * 4, 512>>>(rb, vn, 0x1234u + a, bad);
  CK(cudaDeviceSynchronize());
  printf("verify: %zu MiB written by GPU %d into GPU %d: %llu bad bytes\n", vn * 16 >> 20, a, b, *bad);
  if (*bad) exit(2);
  // phase 2: bandwidth
  CK(cudaSetDevice(a));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));
  printf("%12s %14s %14s %14s\n", "bytes", "kernel write", "kernel read", "copy engine");
  for (size_t bytes = 4096; bytes <= max_bytes; bytes *= 4) {
    Job w{la, rb, bytes / 16, st, b, a}, r{rb, la, bytes / 16, st, a, b};
    const int it = bytes >= (256u << 20) ? (iters / 8 > 2 ? iters / 8 : 2) : iters;
    const float tw = time_ms(st, it, run_kernel, &w);
    const float tr = time_ms(st, it, run_kernel, &r);
    const float tc = time_ms(st, it, run_ce, &w);
    printf("%12zu %11.1f GB/s %11.1f GB/s %11.1f GB/s   (%.1f / %.1f / %.1f us)\n", bytes,
           bytes / tw / 1e6, bytes / tr / 1e6, bytes / tc / 1e6, tw * 1e3, tr * 1e3, tc * 1e3);
  }
  CK(cudaStreamDestroy(st));
  CK(cudaFree(la));
  CK(cudaSetDevice(b));
  CK(cudaFree(rb));
  CK(cudaFree(bad));
}

int main(int argc, char** argv) {
  int a = 0, b = 1, both = 0, iters = 50;
  size_t max_mb = 1024;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--src") && i + 1 < argc) a = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--dst") && i + 1 < argc) b = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--both")) both = 1;
    else if (!strcmp(argv[i], "--reverse")) { int t = a; a = b; b = t; }
    else if (!strcmp(argv[i], "--max-mb") && i + 1 < argc) max_mb = strtoul(argv[++i], nullptr, 10);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else {
      fprintf(stderr, "usage: p2p_bw [--src A] [--dst B] [--both] [--reverse] [--max-mb N] [--iters N]\n");
      return 2;
    }
  }
  int n = 0;
  CK(cudaGetDeviceCount(&n));
  if (n < 2 || a >= n || b >= n || a == b) {
    fprintf(stderr, "p2p_bw needs two different GPUs (box has %d)\n", n);
    return 2;
  }
  int ok = 0;
  CK(cudaDeviceCanAccessPeer(&ok, a, b));
  if (!ok) {
    fprintf(stderr, "GPU %d cannot access GPU %d\n", a, b);
    return 2;
  }
  CK(cudaSetDevice(a));
  cudaDeviceEnablePeerAccess(b, 0);
  CK(cudaSetDevice(b));
  cudaDeviceEnablePeerAccess(a, 0);
  cudaGetLastError();
  direction(a, b, max_mb << 20, iters);
  if (both) direction(b, a, max_mb << 20, iters);
  // phase 3: signal latency
  uint32_t *fa, *fb;
  unsigned long long* ns;
  int* gave;
  CK(cudaSetDevice(a));
  CK(cudaMalloc(&fa, 256));
  CK(cudaMemset(fa, 0, 256));
  CK(cudaSetDevice(b));
  CK(cudaMalloc(&fb, 256));
  CK(cudaMemset(fb, 0, 256));
  CK(cudaMallocManaged(&ns, 16));
  CK(cudaMallocManaged(&gave, 8));
  ns[0] = ns[1] = 0;
  gave[0] = gave[1] = 0;
  CK(cudaDeviceSynchronize());
  const int pp = 2000;
  CK(cudaSetDevice(b));
  k_pingpong<<<1, 1>>>(fb, fa, pp, 0, ns + 1, gave + 1);
  CK(cudaSetDevice(a));
  k_pingpong<<<1, 1>>>(fa, fb, pp, 1, ns, gave);
  CK(cudaDeviceSynchronize());
  CK(cudaSetDevice(b));
  CK(cudaDeviceSynchronize());
  if (gave[0] || gave[1]) printf("\nsignal ping-pong gave up at iteration %d/%d\n", gave[0], gave[1]);
  else printf("\nsignal round trip GPU %d <-> GPU %d: %.2f us (one way %.2f us)\n", a, b, ns[0] / 1e3, ns[0] / 2e3);
  return 0;
}
