// SPDX-License-Identifier: MIT
//
// Dense attention for prefill (causal, grouped-query) and for the joint
// text+image attention of the MMDiT blocks (non-causal): one CTA per 64-query
// tile and head, K/V streamed in 64-key tiles through a cp.async double
// buffer, QK^T and PV on tensor cores with an online softmax.  Sequences are
// packed and described by cumulative lengths.  This mma.sync kernel is the
// fallback (BL_ATTN_TC=0, or callers that do not pass the longest key length);
// attn_tc_kernels.cu is the tcgen05 kernel used otherwise.  The reference takes this op
// from HF transformers / diffusers attention (demos/flux2_tp/worker.py:96-123,
// demos/qwen_tp/qwen38_int8/worker.py:282-291).
#include <stdio.h>

#include "bl_ops.h"
#include "heap.h"
#include "ptx.cuh"

namespace bl {

constexpr int kAHd = 128;
constexpr int kAPitch = kAHd * 2 + 16;  // bytes per shared-memory row
constexpr int kQTile = 64;
constexpr int kKTile = 64;
constexpr int kATileBytes = kKTile * kAPitch;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n)
               : "memory");
}
__device__ __forceinline__ void a_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void a_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void a_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                       uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void a_ldsm_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                         uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void a_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                      uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (q tiles of the longest sequence, nq, batch), 128 threads
__global__ void __launch_bounds__(128)
    k_attn_fwd(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
               const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
               const int* __restrict__ cu_q, const int* __restrict__ cu_k, int nq, int nkv,
               int q_stride, int k_stride, int v_stride, int o_stride, float scale_log2,
               int causal) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = cu_q[b], lq = cu_q[b + 1] - q0;
  const int k0 = cu_k[b], lk = cu_k[b + 1] - k0;
  const int qt = blockIdx.x * kQTile;
  if (qt >= lq) return;
  const int hk = h / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int shift = causal ? lk - lq : 0;  // query i sees keys j <= i + shift

  // Q fragments straight from global memory (rows beyond the sequence are zero)
  uint32_t qa[kAHd / 16][4];
  {
    const int r0 = qt + warp * 16 + g, r1 = r0 + 8;
    const __nv_bfloat16* p0 = q + size_t(q0 + r0) * q_stride + size_t(h) * kAHd;
    const __nv_bfloat16* p1 = q + size_t(q0 + r1) * q_stride + size_t(h) * kAHd;
#pragma unroll
    for (int ks = 0; ks < kAHd / 16; ++ks) {
      const int c = ks * 16 + 2 * t;
      qa[ks][0] = r0 < lq ? *reinterpret_cast<const uint32_t*>(p0 + c) : 0u;
      qa[ks][1] = r1 < lq ? *reinterpret_cast<const uint32_t*>(p1 + c) : 0u;
      qa[ks][2] = r0 < lq ? *reinterpret_cast<const uint32_t*>(p0 + c + 8) : 0u;
      qa[ks][3] = r1 < lq ? *reinterpret_cast<const uint32_t*>(p1 + c + 8) : 0u;
    }
  }
  float o[kAHd / 8][4];
#pragma unroll
  for (int d = 0; d < kAHd / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  int kend = lk;
  if (causal) {
    const int last = qt + kQTile - 1 + shift;  // last key any row of this tile may see
    kend = last + 1 < lk ? last + 1 : lk;
    if (kend < 0) kend = 0;
  }
  const int ntiles = (kend + kKTile - 1) / kKTile;
  const uint32_t sbase = smem_u32(smem);

  auto issue = [&](int tile, int buf) {
    const int j0 = tile * kKTile;
    const uint32_t kd = sbase + buf * 2 * kATileBytes, vd = kd + kATileBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = threadIdx.x + i * 128;  // 1024 chunks of 16 B per tile
      const int r = c >> 4, cc = c & 15;
      const bool ok = j0 + r < lk;
      const size_t row = size_t(k0 + (ok ? j0 + r : 0));
      cp_async16_zfill(kd + r * kAPitch + cc * 16, k + row * k_stride + size_t(hk) * kAHd + cc * 8, ok);
      cp_async16_zfill(vd + r * kAPitch + cc * 16, v + row * v_stride + size_t(hk) * kAHd + cc * 8, ok);
    }
    a_commit();
  };

  if (ntiles > 0) issue(0, 0);
  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) {
      issue(tile + 1, buf ^ 1);
      a_wait<1>();
    } else {
      a_wait<0>();
    }
    __syncthreads();
    const uint32_t kd = sbase + buf * 2 * kATileBytes, vd = kd + kATileBytes;
    const int j0 = tile * kKTile;
    // S = Q K^T: 16 rows x 64 keys per warp
    float s[kKTile / 8][4];
#pragma unroll
    for (int n = 0; n < kKTile / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int np = 0; np < kKTile / 16; ++np) {
        const uint32_t a0 = kd + (np * 16 + (mi >> 1) * 8 + r) * kAPitch + (mi & 1) * 16;
#pragma unroll
        for (int ks = 0; ks < kAHd / 16; ++ks) {
          uint32_t b0, b1, b2, b3;
          a_ldsm(a0 + ks * 32, b0, b1, b2, b3);
          a_mma(s[2 * np], qa[ks], b0, b1);
          a_mma(s[2 * np + 1], qa[ks], b2, b3);
        }
      }
    }
    // mask + online softmax (rows g and g+8 of this warp's 16)
    const int i0 = qt + warp * 16 + g, i1 = i0 + 8;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < kKTile / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + 2 * t + (e & 1);
        const int i = e < 2 ? i0 : i1;
        float x = s[n][e] * scale_log2;
        if (j >= lk || (causal && j > i + shift)) x = -INFINITY;
        s[n][e] = x;
        if (e < 2) mx0 = fmaxf(mx0, x);
        else mx1 = fmaxf(mx1, x);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    // a row that has seen no key yet keeps m = -inf; avoid inf - inf
    const float b0m = n0 == -INFINITY ? 0.f : n0, b1m = n1 == -INFINITY ? 0.f : n1;
    const float al0 = exp2f(m0 - b0m), al1 = exp2f(m1 - b1m);
    m0 = n0;
    m1 = n1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int n = 0; n < kKTile / 8; ++n) {
      s[n][0] = exp2f(s[n][0] - b0m);
      s[n][1] = exp2f(s[n][1] - b0m);
      s[n][2] = exp2f(s[n][2] - b1m);
      s[n][3] = exp2f(s[n][3] - b1m);
      ps0 += s[n][0] + s[n][1];
      ps1 += s[n][2] + s[n][3];
    }
    l0 = l0 * al0 + ps0;
    l1 = l1 * al1 + ps1;
#pragma unroll
    for (int d = 0; d < kAHd / 8; ++d) {
      o[d][0] *= al0;
      o[d][1] *= al0;
      o[d][2] *= al1;
      o[d][3] *= al1;
    }
    // O += P V, 16 keys per k-step
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int kk = 0; kk < kKTile / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        const uint32_t a0 = vd + (kk * 16 + (mi & 1) * 8 + r) * kAPitch + (mi >> 1) * 16;
#pragma unroll
        for (int d = 0; d < kAHd / 8; d += 2) {
          uint32_t b0, b1, b2, b3;
          a_ldsm_t(a0 + d * 16, b0, b1, b2, b3);
          a_mma(o[d], pa, b0, b1);
          a_mma(o[d + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = qt + warp * 16 + g, r1 = r0 + 8;
  __nv_bfloat16* o0 = out + size_t(q0 + r0) * o_stride + size_t(h) * kAHd;
  __nv_bfloat16* o1 = out + size_t(q0 + r1) * o_stride + size_t(h) * kAHd;
#pragma unroll
  for (int d = 0; d < kAHd / 8; ++d) {
    const int c = d * 8 + 2 * t;
    if (r0 < lq) *reinterpret_cast<uint32_t*>(o0 + c) = pack_bf16x2(o[d][0] * inv0, o[d][1] * inv0);
    if (r1 < lq) *reinterpret_cast<uint32_t*>(o1 + c) = pack_bf16x2(o[d][2] * inv1, o[d][3] * inv1);
  }
}

}  // namespace bl

using namespace bl;

extern "C" int bl_attn_fwd(const void* q, const void* k, const void* v, void* out, const int* cu_q,
                           const int* cu_k, int batch, int max_q, int nq, int nkv, int hd,
                           int q_stride, int k_stride, int v_stride, int o_stride, float scale,
                           int causal, void* stream, char* err, size_t errlen) {
  if (hd != kAHd) {
    set_err(err, errlen, "barlink: dense attention is built for head_dim %d", kAHd);
    return -1;
  }
  if (nkv < 1 || nq % nkv) {
    set_err(err, errlen, "barlink: dense attention needs nq %% nkv == 0");
    return -1;
  }
  if ((q_stride | k_stride | v_stride | o_stride) & 7) {
    set_err(err, errlen, "barlink: dense attention needs token strides that are multiples of 8 elements");
    return -1;
  }
  if (batch < 1 || max_q < 1) return 0;
  static bool attr = false;
  const int smem = 4 * kATileBytes;
  if (!attr) {
    cudaError_t e =
        cudaFuncSetAttribute(k_attn_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: dense attention shared memory opt-in failed: %s",
              cudaGetErrorString(e));
      return -1;
    }
    attr = true;
  }
  dim3 grid((max_q + kQTile - 1) / kQTile, nq, batch);
  k_attn_fwd<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
      static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(out), cu_q, cu_k, nq, nkv,
      q_stride, k_stride, v_stride, o_stride, scale * 1.4426950408889634f, causal);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: dense attention launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
