// SPDX-License-Identifier: MIT
//
// Weight-only int4 linear for decode (1..16 tokens) on GPTQ-v1 tensors, the
// format of the reference's Triton GEMV (demos/qwen_tp/int4linear.py:5-12,
// kernel :22-44):
//
//   qweight int32 [K/8, N]   8 consecutive k per word, nibble j = k % 8
//   scales  fp16  [G, N]     one scale per (group of `group` inputs, output)
//   qzeros  int32 [G, N/8]   8 consecutive outputs per word
//   w[n, k] = (nibble - zero) * scale
//
// One thread owns four adjacent outputs and reads one 16-byte vector per
// 8 inputs, so a warp reads 512 contiguous bytes; nibbles become fp16 with
// the 0x6400 exponent trick (1024 + nibble, exact), the zero point is
// subtracted in fp16 (exact) and products accumulate in fp32 per group, then
// per-group sums are scaled.  The split over k is reduced in a fixed order by
// a second kernel (the reference adds with floating-point atomics), so results
// repeat run to run.  More than 16 tokens: widen the weight to bf16 once
// (k_w4_dequant) and use the tcgen05 GEMM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "bl_ops.h"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

constexpr int kW4Threads = 128;
constexpr int kW4MaxM = 16;
constexpr int kW4MaxGroup = 128;

template <int MT>
__global__ void __launch_bounds__(kW4Threads) k_w4a16_gemv(const __nv_bfloat16* __restrict__ x,
                                                           const uint32_t* __restrict__ qw,
                                                           const __half* __restrict__ sc,
                                                           const uint32_t* __restrict__ qz,
                                                           __nv_bfloat16* __restrict__ out,
                                                           float* __restrict__ ws, int M, int N, int K,
                                                           int group, int gper) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_x[MT][kW4MaxGroup];
  const int n = (blockIdx.x * kW4Threads + threadIdx.x) * 4;
  const int G = K / group;
  const int g0 = blockIdx.y * gper, g1 = min(G, g0 + gper);
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0.f;
  for (int g = g0; g < g1; ++g) {
    __syncthreads();
    for (int t = threadIdx.x; t < MT * group; t += kW4Threads) {
      const int m = t / group, k = t - m * group;
      s_x[m][k] = m < M ? __bfloat162float(x[size_t(m) * K + g * group + k]) : 0.f;
    }
    __syncthreads();
    if (n < N) {
      const uint2 sraw = *reinterpret_cast<const uint2*>(sc + size_t(g) * N + n);
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sraw.x));
      const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sraw.y));
      const float scl[4] = {s01.x, s01.y, s23.x, s23.y};
      const uint32_t zw = qz[size_t(g) * (N / 8) + (n >> 3)] >> ((n & 7) * 4);
      float part[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[m][c] = 0.f;
      const uint32_t* wp = qw + (size_t(g) * (group / 8)) * N + n;
#pragma unroll 4
      for (int kk = 0; kk < group / 8; ++kk) {
        const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(wp + size_t(kk) * N));
        const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          // 1024 + zero as fp16 in both halves
          const uint32_t zbits = 0x6400u | ((zw >> (4 * c)) & 15u);
          const __half2 z2 = __halves2half2(__ushort_as_half(zbits), __ushort_as_half(zbits));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // nibbles j (low half) and j + 4 (high half)
            const uint32_t bits = ((wv[c] >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
            const float2 v = __half22float2(__hsub2(*reinterpret_cast<const __half2*>(&bits), z2));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              part[m][c] = fmaf(s_x[m][kk * 8 + j], v.x, part[m][c]);
              part[m][c] = fmaf(s_x[m][kk * 8 + j + 4], v.y, part[m][c]);
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][c] = fmaf(part[m][c], scl[c], acc[m][c]);
    }
  }
  if (n >= N) return;
  if (gridDim.y == 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M)
        *reinterpret_cast<uint2*>(out + size_t(m) * N + n) =
            make_uint2(pack_bf16x2(acc[m][0], acc[m][1]), pack_bf16x2(acc[m][2], acc[m][3]));
  } else {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M)
        *reinterpret_cast<float4*>(ws + (size_t(blockIdx.y) * M + m) * N + n) =
            make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  }
}

__global__ void k_w4_reduce(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int MN, int S) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= MN) return;
  float a = 0.f;
  for (int s = 0; s < S; ++s) a += ws[size_t(s) * MN + t];
  out[t] = __float2bfloat16(a);
}

// w [N, K] bf16 from the packed tensors; one thread per (8 k, 1 n) word
__global__ void k_w4_dequant(const uint32_t* __restrict__ qw, const __half* __restrict__ sc,
                             const uint32_t* __restrict__ qz, __nv_bfloat16* __restrict__ w, int N, int K,
                             int group) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(K / 8) * N) return;
  const int kw = int(t / N), n = int(t % N);
  const int g = kw * 8 / group;
  const float s = __half2float(sc[size_t(g) * N + n]);
  const int z = int((qz[size_t(g) * (N / 8) + (n >> 3)] >> ((n & 7) * 4)) & 15u);
  const uint32_t v = qw[t];
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = float(int((v >> (4 * j)) & 15u) - z) * s;
  *reinterpret_cast<uint4*>(w + size_t(n) * K + kw * 8) =
      make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                 pack_bf16x2(f[6], f[7]));
}

}  // namespace bl

using namespace bl;

static int w4_check(int n, int k, int group, char* err, size_t errlen) {
  if (group < 8 || group > kW4MaxGroup || (group & 7) || k < group || k % group || n < 8 || (n & 7)) {
    set_err(err, errlen,
            "barlink: w4a16 needs group in {8..%d, multiple of 8}, K a multiple of the group and N a multiple of 8 "
            "(got N %d, K %d, group %d)", kW4MaxGroup, n, k, group);
    return -1;
  }
  return 0;
}

extern "C" int bl_w4a16_gemv(const void* x, const void* qweight, const void* scales, const void* qzeros,
                             void* out, int m, int n, int k, int group, int splits, void* ws,
                             size_t ws_bytes, void* stream, char* err, size_t errlen) {
  if (m < 1 || m > kW4MaxM) {
    set_err(err, errlen, "barlink: w4a16_gemv is the decode kernel: 1..%d rows (got %d)", kW4MaxM, m);
    return -2;
  }
  if (w4_check(n, k, group, err, errlen)) return -1;
  const int G = k / group;
  const int nblocks = (n / 4 + kW4Threads - 1) / kW4Threads;
  if (splits <= 0) {
    // enough blocks for every SM a few times over, every split at least two groups
    splits = (148 * 8 + nblocks - 1) / nblocks;
    if (splits > G / 2) splits = G / 2;
  }
  if (splits < 1) splits = 1;
  if (splits > G) splits = G;
  const int gper = (G + splits - 1) / splits;
  splits = (G + gper - 1) / gper;
  if (splits > 1 && (!ws || ws_bytes < size_t(splits) * m * n * sizeof(float))) {
    splits = 1;
  }
  const int gper2 = splits == 1 ? G : gper;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(nblocks, splits);
  cudaError_t e;
#define BL_W4(MT)                                                                                      \
  e = launch_k(k_w4a16_gemv<MT>, grid, dim3(kW4Threads), 0, st, static_cast<const __nv_bfloat16*>(x),  \
               static_cast<const uint32_t*>(qweight), static_cast<const __half*>(scales),              \
               static_cast<const uint32_t*>(qzeros), static_cast<__nv_bfloat16*>(out),                 \
               static_cast<float*>(ws), m, n, k, group, gper2)
  if (m <= 1) BL_W4(1);
  else if (m <= 2) BL_W4(2);
  else if (m <= 4) BL_W4(4);
  else if (m <= 8) BL_W4(8);
  else BL_W4(16);
#undef BL_W4
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess && splits > 1) {
    e = launch_k(k_w4_reduce, dim3((m * n + 255) / 256), dim3(256), 0, st, static_cast<const float*>(ws),
                 static_cast<__nv_bfloat16*>(out), m * n, splits);
    if (e == cudaSuccess) e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w4a16_gemv launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

extern "C" int bl_w4_dequant(const void* qweight, const void* scales, const void* qzeros, void* w, int n,
                             int k, int group, void* stream, char* err, size_t errlen) {
  if (w4_check(n, k, group, err, errlen)) return -1;
  const size_t total = size_t(k / 8) * n;
  cudaError_t e = launch_k(k_w4_dequant, dim3(unsigned((total + 255) / 256)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const uint32_t*>(qweight),
                           static_cast<const __half*>(scales), static_cast<const uint32_t*>(qzeros),
                           static_cast<__nv_bfloat16*>(w), n, k, group);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w4 dequant launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
