// SPDX-License-Identifier: MIT
//
// The reference's W8A8-activation decode GEMM API, kept for callers written
// against it (torch_ext/barlink_sm86/w8a16.cu:165-212, binding.cpp:434-490):
//
//   xq, xs = w8a16_quant_act(x)              per-token int8 activations, scale amax/127
//   y = w8a16_gemm(xq, xs, wq_t, sw_t, N, K, S)
//       y[m, n] = xs[m] * sum_g sw_t[g, n] * sum_{k in group g} xq[m, k] * w[n, k]
//       wq_t int8 [K/16, N, 16] (k-chunk major), sw_t fp32 [K/128, N], M <= 16
//
// The product path of this library is bl_w8a16_linear (gemm_kernels.cu: bf16
// activations, int8 weights widened inside a tcgen05 main loop); the pair
// here exists for API parity and as the numerics cross-check of that kernel.
// Differences from the reference's kernels: activations of a k-group are
// staged in shared memory once per block, and the split over k-groups is
// reduced in a fixed order (workspace + second kernel) instead of with
// floating-point atomics, so results are reproducible run to run.
#include <stdint.h>
#include <stdio.h>

#include "bl_ops.h"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

constexpr int kQThreads = 256;
constexpr int kGroup = 128;
constexpr int kMaxM = 16;

__global__ void __launch_bounds__(kQThreads) k_quant_act(const __nv_bfloat16* __restrict__ x,
                                                          int8_t* __restrict__ xq,
                                                          float* __restrict__ xs, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_red[kQThreads / 32];
  __shared__ float s_scale;
  const __nv_bfloat16* row = x + size_t(blockIdx.x) * K;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
                 d = unpack_bf16x2(v.w);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kQThreads / 32 ? s_red[threadIdx.x] : 0.f;
    t = warp_max(t);
    if (threadIdx.x == 0) {
      s_scale = fmaxf(t / 127.f, 1e-12f);
      xs[blockIdx.x] = s_scale;
    }
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  int8_t* out = xq + size_t(blockIdx.x) * K;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
                 d = unpack_bf16x2(v.w);
    const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int q = __float2int_rn(f[j] * inv);
      q = max(-127, min(127, q));
      w[j >> 2] |= (uint32_t(q) & 0xffu) << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(out + i) = make_uint2(w[0], w[1]);
  }
}

// grid (ceil(N/256), S); thread = output feature n; group range of this split
template <int MT>
__global__ void __launch_bounds__(kQThreads) k_w8a8_gemm(const int8_t* __restrict__ wq_t,
                                                         const float* __restrict__ sw_t,
                                                         const int8_t* __restrict__ xq,
                                                         const float* __restrict__ xs,
                                                         __nv_bfloat16* __restrict__ out,
                                                         float* __restrict__ ws, int M, int N, int K,
                                                         int gper) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_x[MT][kGroup / 4];  // one k-group of every activation row, as dp4a words
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int G = K / kGroup;
  const int g0 = blockIdx.y * gper, g1 = min(G, g0 + gper);
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  for (int g = g0; g < g1; ++g) {
    __syncthreads();
    for (int t = threadIdx.x; t < MT * (kGroup / 4); t += blockDim.x) {
      const int m = t / (kGroup / 4), w = t % (kGroup / 4);
      s_x[m][w] = m < M ? *reinterpret_cast<const int*>(xq + size_t(m) * K + g * kGroup + w * 4) : 0;
    }
    __syncthreads();
    if (n < N) {
      int isum[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) isum[m] = 0;
#pragma unroll
      for (int c = 0; c < kGroup / 16; ++c) {
        const int4 w = *reinterpret_cast<const int4*>(wq_t + (size_t(g * (kGroup / 16) + c) * N + n) * 16);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          isum[m] = __dp4a(w.x, s_x[m][c * 4], isum[m]);
          isum[m] = __dp4a(w.y, s_x[m][c * 4 + 1], isum[m]);
          isum[m] = __dp4a(w.z, s_x[m][c * 4 + 2], isum[m]);
          isum[m] = __dp4a(w.w, s_x[m][c * 4 + 3], isum[m]);
        }
      }
      const float sw = sw_t[size_t(g) * N + n];
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] += sw * float(isum[m]);
    }
  }
  if (n >= N) return;
  if (gridDim.y == 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M) out[size_t(m) * N + n] = __float2bfloat16(acc[m] * xs[m]);
  } else {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M) ws[(size_t(blockIdx.y) * M + m) * N + n] = acc[m];
  }
}

__global__ void k_w8a8_reduce(const float* __restrict__ ws, const float* __restrict__ xs,
                              __nv_bfloat16* __restrict__ out, int M, int N, int S) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M * N) return;
  float a = 0.f;
  for (int s = 0; s < S; ++s) a += ws[size_t(s) * M * N + t];
  out[t] = __float2bfloat16(a * xs[t / N]);
}

}  // namespace bl

using namespace bl;

extern "C" int bl_w8a16_quant_act(const void* x, int m, int k, void* xq, void* xs, void* stream,
                                  char* err, size_t errlen) {
  if (!x || !xq || !xs || m < 1 || k < 8 || (k & 7)) {
    set_err(err, errlen, "barlink: w8a16_quant_act needs K a multiple of 8");
    return -1;
  }
  cudaError_t e = launch_k(k_quant_act, dim3(m), dim3(kQThreads), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const __nv_bfloat16*>(x), static_cast<int8_t*>(xq),
                           static_cast<float*>(xs), k);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w8a16_quant_act launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

extern "C" int bl_w8a16_gemm(const void* xq, const void* xs, const void* wq_t, const void* sw_t,
                             void* out, int m, int n, int k, int splits, void* ws, void* stream,
                             char* err, size_t errlen) {
  if (m < 1 || m > kMaxM) {
    set_err(err, errlen, "barlink: w8a16_gemm is the decode kernel of the reference API: 1..%d rows (got %d)",
            kMaxM, m);
    return -2;
  }
  if (k < kGroup || k % kGroup || n < 1) {
    set_err(err, errlen, "barlink: w8a16_gemm needs K a multiple of %d", kGroup);
    return -1;
  }
  const int G = k / kGroup;
  if (splits < 1) splits = 1;
  if (splits > G) splits = G;
  const int gper = (G + splits - 1) / splits;
  splits = (G + gper - 1) / gper;
  if (splits > 1 && !ws) {
    set_err(err, errlen, "barlink: w8a16_gemm with a k-split needs a workspace of S*M*N floats");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((n + kQThreads - 1) / kQThreads, splits);
  cudaError_t e;
#define BL_W8A8(MT)                                                                                   \
  e = launch_k(k_w8a8_gemm<MT>, grid, dim3(kQThreads), 0, st, static_cast<const int8_t*>(wq_t),       \
               static_cast<const float*>(sw_t), static_cast<const int8_t*>(xq),                       \
               static_cast<const float*>(xs), static_cast<__nv_bfloat16*>(out), static_cast<float*>(ws), \
               m, n, k, gper)
  if (m <= 1) BL_W8A8(1);
  else if (m <= 4) BL_W8A8(4);
  else BL_W8A8(16);
#undef BL_W8A8
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess && splits > 1) {
    e = launch_k(k_w8a8_reduce, dim3((m * n + 255) / 256), dim3(256), 0, st,
                 static_cast<const float*>(ws), static_cast<const float*>(xs),
                 static_cast<__nv_bfloat16*>(out), m, n, splits);
    if (e == cudaSuccess) e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w8a16_gemm launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
