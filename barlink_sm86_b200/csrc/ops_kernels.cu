// SPDX-License-Identifier: MIT
//
// Decode-path kernels for sm_100a that are bandwidth bound rather than GEMM
// shaped: RMSNorm (+residual), RoPE fused with the paged-KV write, SiLU*mul,
// embedding gather, arg max, and paged-KV decode attention (tensor-core
// QK^T/PV on 16-token pages, split over the context, log-sum-exp merge).
// The reference takes all of these from HF transformers / vLLM eager kernels
// (about 29 k launches per token, BUILD_AND_TEST.md:373-376); here each is
// one launch per layer.
#include <stdio.h>

#include <mutex>

#include <stdlib.h>

#include "bl_ops.h"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

#define OPS_LAUNCH_CHECK(what)                                                         \
  do {                                                                                 \
    cudaError_t _e = cudaGetLastError();                                               \
    if (_e != cudaSuccess) {                                                           \
      set_err(err, errlen, "barlink: %s launch failed: %s", what, cudaGetErrorString(_e)); \
      return -1;                                                                       \
    }                                                                                  \
  } while (0)

// ---------------------------------------------------------------------------
// RMSNorm (+ residual add)
// ---------------------------------------------------------------------------
constexpr int kNormMaxVpt = 4;

__global__ void __launch_bounds__(512) k_rmsnorm(const uint4* __restrict__ x,
                                                 const uint4* __restrict__ residual,
                                                 const uint4* __restrict__ gamma,
                                                 uint4* __restrict__ out,
                                                 uint4* __restrict__ residual_out, int vpr,
                                                 float eps, const float* __restrict__ partials,
                                                 int nsplit, size_t slab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_part[16];
  __shared__ float s_rstd;
  const size_t row = blockIdx.x;
  float v[kNormMaxVpt][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kNormMaxVpt; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < vpr) {
      uint4 a;
      if (partials) {
        // x is the sum of the k-split slabs of the linear before this norm,
        // rounded to bf16 as that linear's output would have been
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        sum_slabs8(partials + (row * vpr + i) * 8, slab, nsplit, acc);
        a = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                       pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      } else {
        a = x[row * vpr + i];
      }
      float2 p0 = unpack_bf16x2(a.x), p1 = unpack_bf16x2(a.y), p2 = unpack_bf16x2(a.z),
             p3 = unpack_bf16x2(a.w);
      float f[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
      if (residual) {
        const uint4 b = residual[row * vpr + i];
        float2 q0 = unpack_bf16x2(b.x), q1 = unpack_bf16x2(b.y), q2 = unpack_bf16x2(b.z),
               q3 = unpack_bf16x2(b.w);
        const float r[8] = {q0.x, q0.y, q1.x, q1.y, q2.x, q2.y, q3.x, q3.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
        const uint4 packed = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                        pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        residual_out[row * vpr + i] = packed;
        // the norm sees the stored (rounded) sum
        p0 = unpack_bf16x2(packed.x); p1 = unpack_bf16x2(packed.y);
        p2 = unpack_bf16x2(packed.z); p3 = unpack_bf16x2(packed.w);
        f[0] = p0.x; f[1] = p0.y; f[2] = p1.x; f[3] = p1.y;
        f[4] = p2.x; f[5] = p2.y; f[6] = p3.x; f[7] = p3.y;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = f[j];
        ss += f[j] * f[j];
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_rstd = rsqrtf(t / float(vpr * 8) + eps);
  }
  __syncthreads();
  const float rstd = s_rstd;
#pragma unroll
  for (int k = 0; k < kNormMaxVpt; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < vpr) {
      const uint4 gm = gamma[i];
      const float2 g0 = unpack_bf16x2(gm.x), g1 = unpack_bf16x2(gm.y), g2 = unpack_bf16x2(gm.z),
                   g3 = unpack_bf16x2(gm.w);
      const float gg[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o[j] = __bfloat162float(__float2bfloat16(v[k][j] * rstd)) * gg[j];
      out[row * vpr + i] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                      pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
  }
}

// ---------------------------------------------------------------------------
// RoPE (rotate-half) on q and k of a fused qkv row + paged KV write
// ---------------------------------------------------------------------------
// grid (rows, ceil((nq+nkv+nkv)/kRopeHeads)): each block rotates kRopeHeads
// heads of one row, one (head, pair) per thread; V heads are copied.
constexpr int kRopeHeads = 4;
__global__ void __launch_bounds__(256) k_rope_kv_write(__nv_bfloat16* __restrict__ qkv,
                                                       const float* __restrict__ partials,
                                                       int nsplit, size_t slab,
                                                       const __nv_bfloat16* __restrict__ bias,
                                                       const int* __restrict__ positions,
                                                       const int* __restrict__ slots,
                                                       __nv_bfloat16* __restrict__ k_cache,
                                                       __nv_bfloat16* __restrict__ v_cache, int nq,
                                                       int nkv, int hd, int block_size,
                                                       float log2_theta) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int half = hd >> 1;
  const int i = threadIdx.x % half;
  const int hpb = blockDim.x / half;  // heads per block
  const int h = blockIdx.y * hpb + threadIdx.x / half;
  if (threadIdx.x / half >= hpb || h >= nq + 2 * nkv) return;
  __nv_bfloat16* p = qkv + (size_t(row) * (nq + 2 * nkv) + h) * hd;
  // input: the qkv buffer itself, or the k-split slabs of the QKV linear (+ bias)
  float in1, in2;
  if (partials) {
    const size_t e = (size_t(row) * (nq + 2 * nkv) + h) * hd;
    float a1 = 0.f, a2 = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      a1 += __ldcg(partials + sp * slab + e + i);
      a2 += __ldcg(partials + sp * slab + e + i + half);
    }
    if (bias) {
      a1 += __bfloat162float(bias[h * hd + i]);
      a2 += __bfloat162float(bias[h * hd + i + half]);
    }
    in1 = __bfloat162float(__float2bfloat16(a1));
    in2 = __bfloat162float(__float2bfloat16(a2));
  } else {
    in1 = __bfloat162float(p[i]);
    in2 = __bfloat162float(p[i + half]);
  }
  const int slot = slots ? slots[row] : -1;
  const int blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? slot % block_size : 0;
  if (h < nq + nkv) {
    const float pos = float(positions[row]);
    const float inv = exp2f(-log2_theta * (2.f * float(i) / float(hd)));
    float sn, cs;
    sincosf(pos * inv, &sn, &cs);
    const float x1 = in1, x2 = in2;
    const __nv_bfloat16 o1 = __float2bfloat16(x1 * cs - x2 * sn);
    const __nv_bfloat16 o2 = __float2bfloat16(x2 * cs + x1 * sn);
    p[i] = o1;
    p[i + half] = o2;
    if (h >= nq && slot >= 0) {
      __nv_bfloat16* c = k_cache + ((size_t(blk) * nkv + (h - nq)) * block_size + off) * hd;
      c[i] = o1;
      c[i + half] = o2;
    }
  } else {
    const __nv_bfloat16 v1 = __float2bfloat16(in1), v2 = __float2bfloat16(in2);
    if (partials) {
      p[i] = v1;
      p[i + half] = v2;
    }
    if (slot >= 0) {
      __nv_bfloat16* c = v_cache + ((size_t(blk) * nkv + (h - nq - nkv)) * block_size + off) * hd;
      c[i] = v1;
      c[i + half] = v2;
    }
  }
}

// plain RoPE; axes = 2 rotates each half of the head by its own position
__global__ void __launch_bounds__(128) k_rope(__nv_bfloat16* __restrict__ x,
                                              const int* __restrict__ positions, int heads, int hd,
                                              int row_stride, float log2_theta, int axes) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int sub = hd / axes;   // dims rotated by one axis
  const int half = sub >> 1;
  const int pairs = half * axes;
  for (int t = threadIdx.x; t < heads * pairs; t += blockDim.x) {
    const int h = t / pairs, r = t % pairs;
    const int ax = r / half, i = r % half;
    const float pos = float(positions[row * axes + ax]);
    const float inv = exp2f(-log2_theta * (2.f * float(i) / float(sub)));
    float sn, cs;
    sincosf(pos * inv, &sn, &cs);
    __nv_bfloat16* p = x + size_t(row) * row_stride + size_t(h) * hd + ax * sub;
    const float x1 = __bfloat162float(p[i]), x2 = __bfloat162float(p[i + half]);
    p[i] = __float2bfloat16(x1 * cs - x2 * sn);
    p[i + half] = __float2bfloat16(x2 * cs + x1 * sn);
  }
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up
// ---------------------------------------------------------------------------
__global__ void k_silu_mul(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                           int rows, int inter, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = size_t(rows) * inter;
  for (size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += size_t(gridDim.x) * blockDim.x) {
    const size_t r = t / inter, c = t % inter;
    float g, u;
    if (interleaved) {
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * inter + 2 * c);
      g = __bfloat162float(p.x);
      u = __bfloat162float(p.y);
    } else {
      g = __bfloat162float(gu[r * 2 * inter + c]);
      u = __bfloat162float(gu[r * 2 * inter + inter + c]);
    }
    out[t] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
  }
}

// Same on the fp32 k-split slabs [split][row][2*inter] of the gate/up linear
// (interleaved gate/up columns): sums the slabs while reading, 4 outputs per thread.
__global__ void k_silu_mul_slabs(const float* __restrict__ slabs, size_t slab_stride, int nsplit,
                                 __nv_bfloat16* __restrict__ out, size_t total4) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total4;
       t += size_t(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    sum_slabs8(slabs + t * 8, slab_stride, nsplit, acc);
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = acc[2 * j], u = acc[2 * j + 1];
      o[j] = g / (1.f + __expf(-g)) * u;
    }
    *reinterpret_cast<uint2*>(out + t * 4) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
  }
}

__global__ void k_embedding(const int* __restrict__ ids, const uint4* __restrict__ table,
                            uint4* __restrict__ out, int vpr, int lo, int hi) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool mine = id >= lo && id < hi;
  for (int i = threadIdx.x; i < vpr; i += blockDim.x)
    out[size_t(row) * vpr + i] = mine ? table[size_t(id - lo) * vpr + i] : make_uint4(0, 0, 0, 0);
}

// ---------------------------------------------------------------------------
// arg max (ties: lowest index)
// ---------------------------------------------------------------------------
// grid (rows, chunks): each block scans one slice of a row with 16-byte
// loads and leaves (value, index) in part[chunk][row]; k_argmax_merge picks.
constexpr int kArgmaxChunks = 16;
__global__ void __launch_bounds__(256) k_argmax(const __nv_bfloat16* __restrict__ logits, int n,
                                                int ld, int offset, float2* __restrict__ part,
                                                int rows) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  const int row = blockIdx.x, chunk = blockIdx.y;
  const __nv_bfloat16* p = logits + size_t(row) * ld;
  const int per = ((n + kArgmaxChunks - 1) / kArgmaxChunks + 7) & ~7;
  const int lo = chunk * per, hi = min(n, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) && ((ld & 7) == 0);
  if (vec_ok) {
    for (int i = lo + threadIdx.x * 8; i < hi; i += blockDim.x * 8) {
      if (i + 8 <= hi) {
        const uint4 v = *reinterpret_cast<const uint4*>(p + i);
        const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
                     d = unpack_bf16x2(v.w);
        const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (f[j] > best) {  // ascending index inside a thread: first maximum wins
            best = f[j];
            bi = i + j;
          }
      } else {
        for (int j = i; j < hi; ++j) {
          const float f = __bfloat162float(p[j]);
          if (f > best) {
            best = f;
            bi = j;
          }
        }
      }
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float f = __bfloat162float(p[i]);
      if (f > best || (f == best && i < bi)) {
        best = f;
        bi = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = best;
    s_i[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? s_v[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < (blockDim.x >> 5) ? s_i[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0)
      part[size_t(chunk) * rows + row] =
          make_float2(best, __int_as_float(bi == 0x7fffffff ? bi : bi + offset));
  }
}

// ---------------------------------------------------------------------------
// paged decode attention
// ---------------------------------------------------------------------------
constexpr int kPageTokens = 16;
constexpr int kHd = 128;
constexpr int kRowPitch = kHd * 2 + 16;               // bytes, padded against bank conflicts
constexpr int kPageBytes = kPageTokens * kRowPitch;   // one K or V page in shared memory
constexpr int kAttnStages = 3;                        // pages in flight per warp: kAttnStages - 1
constexpr int kWarpSmem = kAttnStages * 2 * kPageBytes;  // (K, V) x stages
constexpr int kAttnWarps = 4;

__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (nkv, batch, splits), 128 threads.  Each warp walks its own pages with
// a private ring of kAttnStages page buffers (cp.async, two pages in flight
// while one is consumed); the warp's block-table entries are fetched 32 at a
// time into registers so that no page address waits on a dependent load.  The
// four warps are merged through shared memory, splits through `scratch` and
// k_attn_merge.
__global__ void __launch_bounds__(kAttnWarps * 32)
    k_paged_attn_decode(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_tables, const int* __restrict__ ctx_lens,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ scratch, int nq,
                        int nkv, int max_blocks, float scale_log2) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, sp = blockIdx.z, nsplit = gridDim.z;
  const int G = nq / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ctx = ctx_lens[b];
  const int n_pages = (ctx + kPageTokens - 1) / kPageTokens;
  const int per = (n_pages + nsplit - 1) / nsplit;
  const int p0 = sp * per;
  const int p1 = min(n_pages, p0 + per);
  const int* table = block_tables + size_t(b) * max_blocks;

  // Q fragments (rows = heads of this group, zero beyond G)
  uint32_t qa[kHd / 16][4];
  {
    const __nv_bfloat16* qb = q + size_t(b) * q_stride + size_t(h) * G * kHd;
#pragma unroll
    for (int ks = 0; ks < kHd / 16; ++ks) {
      const int c = ks * 16 + 2 * t;
      qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * kHd + c) : 0u;
      qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kHd + c) : 0u;
      qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * kHd + c + 8) : 0u;
      qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kHd + c + 8) : 0u;
    }
  }
  float o[kHd / 8][4];
#pragma unroll
  for (int d = 0; d < kHd / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const uint32_t wbase = smem_u32(smem) + warp * kWarpSmem;
  // pages of this warp: p0 + warp + i * kAttnWarps, i in [0, count)
  const int count = p1 > p0 + warp ? (p1 - p0 - warp + kAttnWarps - 1) / kAttnWarps : 0;
  int tbl = 0;        // lane l holds the table entry of page index (chunk * 32 + l)
  int tbl_chunk = -1;
  auto issue = [&](int i, int buf) {
    if ((i >> 5) != tbl_chunk) {
      tbl_chunk = i >> 5;
      const int mine = tbl_chunk * 32 + lane;
      tbl = mine < count ? table[p0 + warp + mine * kAttnWarps] : 0;
    }
    const int blk = __shfl_sync(0xffffffffu, tbl, i & 31);
    const uint8_t* ks = reinterpret_cast<const uint8_t*>(k_cache) +
                        (size_t(blk) * nkv + h) * (kPageTokens * kHd * 2);
    const uint8_t* vs = reinterpret_cast<const uint8_t*>(v_cache) +
                        (size_t(blk) * nkv + h) * (kPageTokens * kHd * 2);
    const uint32_t kd = wbase + buf * 2 * kPageBytes, vd = kd + kPageBytes;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = lane + j * 32;  // 256 chunks of 16 B per page
      const int r = c >> 4, cc = c & 15;
      cp_async16(kd + r * kRowPitch + cc * 16, ks + c * 16);
      cp_async16(vd + r * kRowPitch + cc * 16, vs + c * 16);
    }
  };

  // prologue: kAttnStages - 1 pages in flight (one commit group per slot, empty when past the end)
#pragma unroll
  for (int i = 0; i < kAttnStages - 1; ++i) {
    if (i < count) issue(i, i);
    cp_async_commit();
  }
  int buf = 0;
  for (int i = 0; i < count; ++i) {
    const int page = p0 + warp + i * kAttnWarps;
    {
      const int nxt = i + kAttnStages - 1;
      int nbuf = buf + kAttnStages - 1;
      if (nbuf >= kAttnStages) nbuf -= kAttnStages;
      if (nxt < count) issue(nxt, nbuf);
      cp_async_commit();
      cp_async_wait<kAttnStages - 1>();
    }
    __syncwarp();
    const uint32_t kd = wbase + buf * 2 * kPageBytes, vd = kd + kPageBytes;
    // S = Q K^T for 16 tokens (two n8 tiles)
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      // two accumulator sets (even / odd k-steps) halve the dependent MMA chain
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a0 = kd + ((mi >> 1) * 8 + r) * kRowPitch + (mi & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < kHd / 16; ks += 2) {
        uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
        ldsm_x4(a0 + ks * 32, b0, b1, b2, b3);
        ldsm_x4(a0 + ks * 32 + 32, c0, c1, c2, c3);
        mma_bf16_16816(s[0], qa[ks], b0, b1);
        mma_bf16_16816(s[1], qa[ks], b2, b3);
        mma_bf16_16816(s2[0], qa[ks + 1], c0, c1);
        mma_bf16_16816(s2[1], qa[ks + 1], c2, c3);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
    }
    // mask, online softmax
    const int tok0 = page * kPageTokens;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + nt * 8 + 2 * t + (e & 1);
        float x = s[nt][e] * scale_log2;
        if (tok >= ctx) x = -INFINITY;
        s[nt][e] = x;
        if (e < 2) mx0 = fmaxf(mx0, x);
        else mx1 = fmaxf(mx1, x);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float al0 = fast_ex2(m0 - n0), al1 = fast_ex2(m1 - n1);  // m = -inf -> 0
    m0 = n0;
    m1 = n1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pa[4];
    {
      float pv[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        pv[nt][0] = fast_ex2(s[nt][0] - n0);
        pv[nt][1] = fast_ex2(s[nt][1] - n0);
        pv[nt][2] = fast_ex2(s[nt][2] - n1);
        pv[nt][3] = fast_ex2(s[nt][3] - n1);
        ps0 += pv[nt][0] + pv[nt][1];
        ps1 += pv[nt][2] + pv[nt][3];
      }
      pa[0] = pack_bf16x2(pv[0][0], pv[0][1]);
      pa[1] = pack_bf16x2(pv[0][2], pv[0][3]);
      pa[2] = pack_bf16x2(pv[1][0], pv[1][1]);
      pa[3] = pack_bf16x2(pv[1][2], pv[1][3]);
    }
    l0 = l0 * al0 + ps0;
    l1 = l1 * al1 + ps1;
#pragma unroll
    for (int d = 0; d < kHd / 8; ++d) {
      o[d][0] *= al0;
      o[d][1] *= al0;
      o[d][2] *= al1;
      o[d][3] *= al1;
    }
    // O += P V
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a0 = vd + ((mi & 1) * 8 + r) * kRowPitch + (mi >> 1) * 16;
#pragma unroll
      for (int d = 0; d < kHd / 8; d += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(a0 + d * 16, b0, b1, b2, b3);
        mma_bf16_16816(o[d], pa, b0, b1);
        mma_bf16_16816(o[d + 1], pa, b2, b3);
      }
    }
    __syncwarp();
    if (++buf == kAttnStages) buf = 0;
  }
  cp_async_wait<0>();
  // row sums live spread over the quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the four warps ----------------------------------------------
  float* wo = reinterpret_cast<float*>(smem + warp * kWarpSmem);  // [16][128] + m[16] + l[16]
  float* wm = wo + 16 * kHd;
  float* wl = wm + 16;
#pragma unroll
  for (int d = 0; d < kHd / 8; ++d) {
    *reinterpret_cast<float2*>(wo + g * kHd + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
    *reinterpret_cast<float2*>(wo + (g + 8) * kHd + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
  }
  if (t == 0) {
    wm[g] = m0;
    wm[g + 8] = m1;
    wl[g] = l0;
    wl[g + 8] = l1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * kHd; e += blockDim.x) {
    const int r = e / kHd, d = e % kHd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w)
      M = fmaxf(M, reinterpret_cast<const float*>(smem + w * kWarpSmem)[16 * kHd + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* base = reinterpret_cast<const float*>(smem + w * kWarpSmem);
      const float mw = base[16 * kHd + r];
      const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += base[16 * kHd + 16 + r] * sc;
      acc += base[r * kHd + d] * sc;
    }
    const int head = h * G + r;
    if (nsplit == 1) {
      out[size_t(b) * nq * kHd + size_t(head) * kHd + d] =
          __float2bfloat16(L > 0.f ? acc / L : 0.f);
    } else {
      float* sc = scratch + ((size_t(b) * nq + head) * nsplit + sp) * (kHd + 2);
      sc[d] = acc;
      if (d == 0) {
        sc[kHd] = M;
        sc[kHd + 1] = L;
      }
    }
  }
}

// Source of the raw (pre-RoPE) QKV projection of the decode step: the bf16
// buffer, or the fp32 k-split slabs of the QKV linear (+ bias), summed and
// rounded to bf16 exactly as k_rope_kv_write does.
struct QkvSrc {
  const __nv_bfloat16* qkv;
  int q_stride;
  const float* slabs;
  int nsplit;
  size_t slab;
  const __nv_bfloat16* bias;
  int width;
};
// element `col` of row `row`.  Slabs are added in split order (four loads in flight at a time),
// then the bias, then the sum is rounded to bf16: the same bits as k_rope_kv_write produces.
__device__ __forceinline__ float qkv_elem(const QkvSrc& s, int row, int col) {
  if (s.slabs) {
    const float* p = s.slabs + size_t(row) * s.width + col;
    float acc = 0.f;
    int sp = 0;
    for (; sp + 4 <= s.nsplit; sp += 4) {
      const float a0 = __ldcg(p + size_t(sp) * s.slab), a1 = __ldcg(p + size_t(sp + 1) * s.slab),
                  a2 = __ldcg(p + size_t(sp + 2) * s.slab), a3 = __ldcg(p + size_t(sp + 3) * s.slab);
      acc += a0;
      acc += a1;
      acc += a2;
      acc += a3;
    }
    for (; sp < s.nsplit; ++sp) acc += __ldcg(p + size_t(sp) * s.slab);
    if (s.bias) acc += __bfloat162float(s.bias[col]);
    return __bfloat162float(__float2bfloat16(acc));
  }
  return __bfloat162float(s.qkv[size_t(row) * s.q_stride + col]);
}

// k_paged_attn_decode with the kernel before it folded in: the query heads and
// the new token's key are taken raw from the QKV projection (the bf16 buffer,
// or the k-split slabs of that linear plus bias), rotated here, the new key and
// value are stored to the cache by the block that owns the last page, and that
// block patches the row into its shared-memory copy of the page, so the cache
// write never has to be visible to this kernel's own loads.  Selected with
// BL_FUSE_ROPE_ATTN=1 (one launch less per layer).
__global__ void __launch_bounds__(kAttnWarps * 32)
    k_rope_attn_decode(QkvSrc src, const int* __restrict__ positions, const int* __restrict__ slots,
                       float log2_theta, __nv_bfloat16* __restrict__ k_cache,
                       __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_tables, const int* __restrict__ ctx_lens,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ scratch, int nq,
                        int nkv, int max_blocks, float scale_log2, uint32_t* __restrict__ counters) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, sp = blockIdx.z, nsplit = gridDim.z;
  const int G = nq / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* table = block_tables + size_t(b) * max_blocks;
  const uint32_t wbase = smem_u32(smem) + warp * kWarpSmem;

  // The pages of earlier tokens were written by earlier steps, so their copies may start before
  // the kernels ahead of this one have finished; only the context length could still be the
  // previous step's.  The range of pages is therefore computed from a first read, the first
  // pages are requested, and after the wait the length is read again: in the rare case that the
  // page count changed in between, the requests are drained and issued again.
  int ctx = *reinterpret_cast<const volatile int*>(ctx_lens + b);
  int n_pages, p0, p1, count;
  auto set_range = [&]() {
    n_pages = (ctx + kPageTokens - 1) / kPageTokens;
    if (n_pages > max_blocks) n_pages = max_blocks;
    if (n_pages < 0) n_pages = 0;
    const int per = (n_pages + nsplit - 1) / nsplit;
    p0 = sp * per;
    p1 = min(n_pages, p0 + per);
    // pages of this warp: p0 + warp + i * kAttnWarps, i in [0, count)
    count = p1 > p0 + warp ? (p1 - p0 - warp + kAttnWarps - 1) / kAttnWarps : 0;
  };
  set_range();
  int tbl = 0;        // lane l holds the table entry of page index (chunk * 32 + l)
  int tbl_chunk = -1;
  auto issue = [&](int i, int buf) {
    if ((i >> 5) != tbl_chunk) {
      tbl_chunk = i >> 5;
      const int mine = tbl_chunk * 32 + lane;
      tbl = mine < count ? table[p0 + warp + mine * kAttnWarps] : 0;
    }
    const int blk = __shfl_sync(0xffffffffu, tbl, i & 31);
    const uint8_t* ks = reinterpret_cast<const uint8_t*>(k_cache) +
                        (size_t(blk) * nkv + h) * (kPageTokens * kHd * 2);
    const uint8_t* vs = reinterpret_cast<const uint8_t*>(v_cache) +
                        (size_t(blk) * nkv + h) * (kPageTokens * kHd * 2);
    const uint32_t kd = wbase + buf * 2 * kPageBytes, vd = kd + kPageBytes;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = lane + j * 32;  // 256 chunks of 16 B per page
      const int r = c >> 4, cc = c & 15;
      cp_async16(kd + r * kRowPitch + cc * 16, ks + c * 16);
      cp_async16(vd + r * kRowPitch + cc * 16, vs + c * 16);
    }
  };
  // prologue: kAttnStages - 1 pages in flight (one commit group per slot, empty when past the end)
  auto prologue = [&]() {
#pragma unroll
    for (int i = 0; i < kAttnStages - 1; ++i) {
      if (i < count) issue(i, i);
      cp_async_commit();
    }
  };
  prologue();
  pdl_wait();
  // Everything this block needs from the kernels ahead is requested in one go: the raw query heads
  // and the new key / value (one rotation pair (i, i + 64) per thread and step, consecutive threads
  // on consecutive columns: rows 0..G-1 are the query heads, G the new key, G + 1 the new value),
  // the position and the context length.
  constexpr int kPrepMax = (16 + 2) * (kHd / 2) / (kAttnWarps * 32);
  float px1[kPrepMax], px2[kPrepMax];
#pragma unroll
  for (int it = 0; it < kPrepMax; ++it) {
    const int p = threadIdx.x + it * (kAttnWarps * 32);
    if (p < (G + 2) * (kHd / 2)) {
      const int hh = p / (kHd / 2), i = p % (kHd / 2);
      const int col = hh < G ? (h * G + hh) * kHd : hh == G ? (nq + h) * kHd : (nq + nkv + h) * kHd;
      px1[it] = qkv_elem(src, b, col + i);
      px2[it] = qkv_elem(src, b, col + i + kHd / 2);
    }
  }
  const float pos = float(positions[b]);
  {
    const int pages_before = n_pages;
    ctx = *reinterpret_cast<const volatile int*>(ctx_lens + b);
    const int now = min(max_blocks, (ctx + kPageTokens - 1) / kPageTokens);
    if (now != pages_before) {
      cp_async_wait<0>();
      __syncwarp();
      set_range();
      tbl_chunk = -1;
      prologue();
    } else {
      set_range();
    }
  }
  // cos / sin of this sequence's position for the 64 rotation pairs
  __shared__ float2 s_cs[kHd / 2];
  __shared__ __align__(16) __nv_bfloat16 s_q[16][kHd];   // rotated query heads of this group (rows < G)
  __shared__ __align__(16) __nv_bfloat16 s_new[2][kHd];  // rotated key, value of the new token
  if (threadIdx.x < kHd / 2) {
    const float inv = exp2f(-log2_theta * (2.f * float(threadIdx.x) / float(kHd)));
    float sn, cs;
    sincosf(pos * inv, &sn, &cs);
    s_cs[threadIdx.x] = make_float2(cs, sn);
  }
  __syncthreads();
  const int last_page = n_pages - 1;
  const bool owns_last = last_page >= p0 && last_page < p1;
  {
    const int rows = owns_last ? G + 2 : G;
#pragma unroll
    for (int it = 0; it < kPrepMax; ++it) {
      const int p = threadIdx.x + it * (kAttnWarps * 32);
      if (p >= rows * (kHd / 2)) continue;
      const int hh = p / (kHd / 2), i = p % (kHd / 2);
      const float x1 = px1[it], x2 = px2[it];
      __nv_bfloat16 o1, o2;
      if (hh <= G) {
        const float2 cs = s_cs[i];
        o1 = __float2bfloat16(x1 * cs.x - x2 * cs.y);
        o2 = __float2bfloat16(x2 * cs.x + x1 * cs.y);
      } else {
        o1 = __float2bfloat16(x1);
        o2 = __float2bfloat16(x2);
      }
      __nv_bfloat16* dst = hh < G ? s_q[hh] : s_new[hh - G];
      dst[i] = o1;
      dst[i + kHd / 2] = o2;
    }
  }
  __syncthreads();
  if (owns_last && warp == 0) {
    // the block that owns the last page stores the new row to the cache (8 bytes per lane)
    const int slot = slots[b];
    if (slot >= 0) {
      const size_t row = (size_t(slot / kPageTokens) * nkv + h) * kPageTokens + slot % kPageTokens;
      reinterpret_cast<uint2*>(k_cache + row * kHd)[lane] = reinterpret_cast<const uint2*>(s_new[0])[lane];
      reinterpret_cast<uint2*>(v_cache + row * kHd)[lane] = reinterpret_cast<const uint2*>(s_new[1])[lane];
    }
  }

  // Q fragments (rows = heads of this group, zero beyond G)
  uint32_t qa[kHd / 16][4];
#pragma unroll
  for (int ks = 0; ks < kHd / 16; ++ks) {
    const int c = ks * 16 + 2 * t;
    qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(&s_q[g][c]) : 0u;
    qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(&s_q[g + 8][c]) : 0u;
    qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(&s_q[g][c + 8]) : 0u;
    qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(&s_q[g + 8][c + 8]) : 0u;
  }
  float o[kHd / 8][4];
#pragma unroll
  for (int d = 0; d < kHd / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  int buf = 0;
  for (int i = 0; i < count; ++i) {
    const int page = p0 + warp + i * kAttnWarps;
    {
      const int nxt = i + kAttnStages - 1;
      int nbuf = buf + kAttnStages - 1;
      if (nbuf >= kAttnStages) nbuf -= kAttnStages;
      if (nxt < count) issue(nxt, nbuf);
      cp_async_commit();
      cp_async_wait<kAttnStages - 1>();
    }
    __syncwarp();
    const uint32_t kd = wbase + buf * 2 * kPageBytes, vd = kd + kPageBytes;
    if (page == last_page) {
      // the new token's row comes from this block, not from the cache
      const int r = (ctx - 1) % kPageTokens;
      const uint2 kk = reinterpret_cast<const uint2*>(s_new[0])[lane];
      const uint2 vv = reinterpret_cast<const uint2*>(s_new[1])[lane];
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(kd + r * kRowPitch + lane * 8), "r"(kk.x), "r"(kk.y)
                   : "memory");
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(vd + r * kRowPitch + lane * 8), "r"(vv.x), "r"(vv.y)
                   : "memory");
      __syncwarp();
    }
    // S = Q K^T for 16 tokens (two n8 tiles)
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      // two accumulator sets (even / odd k-steps) halve the dependent MMA chain
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a0 = kd + ((mi >> 1) * 8 + r) * kRowPitch + (mi & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < kHd / 16; ks += 2) {
        uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
        ldsm_x4(a0 + ks * 32, b0, b1, b2, b3);
        ldsm_x4(a0 + ks * 32 + 32, c0, c1, c2, c3);
        mma_bf16_16816(s[0], qa[ks], b0, b1);
        mma_bf16_16816(s[1], qa[ks], b2, b3);
        mma_bf16_16816(s2[0], qa[ks + 1], c0, c1);
        mma_bf16_16816(s2[1], qa[ks + 1], c2, c3);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
    }
    // mask, online softmax
    const int tok0 = page * kPageTokens;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + nt * 8 + 2 * t + (e & 1);
        float x = s[nt][e] * scale_log2;
        if (tok >= ctx) x = -INFINITY;
        s[nt][e] = x;
        if (e < 2) mx0 = fmaxf(mx0, x);
        else mx1 = fmaxf(mx1, x);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float al0 = fast_ex2(m0 - n0), al1 = fast_ex2(m1 - n1);  // m = -inf -> 0
    m0 = n0;
    m1 = n1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pa[4];
    {
      float pv[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        pv[nt][0] = fast_ex2(s[nt][0] - n0);
        pv[nt][1] = fast_ex2(s[nt][1] - n0);
        pv[nt][2] = fast_ex2(s[nt][2] - n1);
        pv[nt][3] = fast_ex2(s[nt][3] - n1);
        ps0 += pv[nt][0] + pv[nt][1];
        ps1 += pv[nt][2] + pv[nt][3];
      }
      pa[0] = pack_bf16x2(pv[0][0], pv[0][1]);
      pa[1] = pack_bf16x2(pv[0][2], pv[0][3]);
      pa[2] = pack_bf16x2(pv[1][0], pv[1][1]);
      pa[3] = pack_bf16x2(pv[1][2], pv[1][3]);
    }
    l0 = l0 * al0 + ps0;
    l1 = l1 * al1 + ps1;
#pragma unroll
    for (int d = 0; d < kHd / 8; ++d) {
      o[d][0] *= al0;
      o[d][1] *= al0;
      o[d][2] *= al1;
      o[d][3] *= al1;
    }
    // O += P V
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a0 = vd + ((mi & 1) * 8 + r) * kRowPitch + (mi >> 1) * 16;
#pragma unroll
      for (int d = 0; d < kHd / 8; d += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(a0 + d * 16, b0, b1, b2, b3);
        mma_bf16_16816(o[d], pa, b0, b1);
        mma_bf16_16816(o[d + 1], pa, b2, b3);
      }
    }
    __syncwarp();
    if (++buf == kAttnStages) buf = 0;
  }
  cp_async_wait<0>();
  // row sums live spread over the quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the four warps ----------------------------------------------
  float* wo = reinterpret_cast<float*>(smem + warp * kWarpSmem);  // [16][128] + m[16] + l[16]
  float* wm = wo + 16 * kHd;
  float* wl = wm + 16;
#pragma unroll
  for (int d = 0; d < kHd / 8; ++d) {
    *reinterpret_cast<float2*>(wo + g * kHd + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
    *reinterpret_cast<float2*>(wo + (g + 8) * kHd + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
  }
  if (t == 0) {
    wm[g] = m0;
    wm[g + 8] = m1;
    wl[g] = l0;
    wl[g + 8] = l1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * kHd; e += blockDim.x) {
    const int r = e / kHd, d = e % kHd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w)
      M = fmaxf(M, reinterpret_cast<const float*>(smem + w * kWarpSmem)[16 * kHd + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* base = reinterpret_cast<const float*>(smem + w * kWarpSmem);
      const float mw = base[16 * kHd + r];
      const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += base[16 * kHd + 16 + r] * sc;
      acc += base[r * kHd + d] * sc;
    }
    const int head = h * G + r;
    if (nsplit == 1) {
      out[size_t(b) * nq * kHd + size_t(head) * kHd + d] =
          __float2bfloat16(L > 0.f ? acc / L : 0.f);
    } else {
      float* sc = scratch + ((size_t(b) * nq + head) * nsplit + sp) * (kHd + 2);
      sc[d] = acc;
      if (d == 0) {
        sc[kHd] = M;
        sc[kHd + 1] = L;
      }
    }
  }
  // Splits are merged by the block of this (sequence, KV head) that finishes last: no second
  // kernel.  The counter goes back to zero for the next launch.
  if (nsplit > 1 && counters) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(&counters[b * nkv + h], 1u);
      s_last = old == uint32_t(nsplit - 1);
      if (s_last) counters[b * nkv + h] = 0u;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int e = threadIdx.x; e < G * kHd; e += blockDim.x) {
        const int r = e / kHd, d = e % kHd;
        const int head = h * G + r;
        const float* base = scratch + (size_t(b) * nq + head) * nsplit * (kHd + 2);
        float M = -INFINITY;
        for (int s2 = 0; s2 < nsplit; ++s2) M = fmaxf(M, __ldcg(base + s2 * (kHd + 2) + kHd));
        float L = 0.f, acc = 0.f;
        for (int s2 = 0; s2 < nsplit; ++s2) {
          const float mw = __ldcg(base + s2 * (kHd + 2) + kHd);
          const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
          L += __ldcg(base + s2 * (kHd + 2) + kHd + 1) * sc;
          acc += __ldcg(base + s2 * (kHd + 2) + d) * sc;
        }
        out[size_t(b) * nq * kHd + size_t(head) * kHd + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
      }
    }
  }
}

__global__ void __launch_bounds__(kHd) k_attn_merge(const float* __restrict__ scratch,
                                                    __nv_bfloat16* __restrict__ out, int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t bh = blockIdx.x;  // batch*nq + head
  const float* base = scratch + bh * nsplit * (kHd + 2);
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, base[s * (kHd + 2) + kHd]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float mw = base[s * (kHd + 2) + kHd];
    const float sc = mw == -INFINITY ? 0.f : exp2f(mw - M);
    L += base[s * (kHd + 2) + kHd + 1] * sc;
    acc += base[s * (kHd + 2) + d] * sc;
  }
  out[bh * kHd + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

// merge per-rank (value, index) pairs of a vocab-parallel arg max:
// pairs [world][rows] as float2(value, index-as-int-bits)
__global__ void k_argmax_merge(const float2* __restrict__ pairs, int world, int rows,
                               int* __restrict__ idx, float* __restrict__ val) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int w = 0; w < world; ++w) {
    const float2 p = pairs[size_t(w) * rows + r];
    const int i = __float_as_int(p.y);
    if (p.x > best || (p.x == best && i < bi)) {
      best = p.x;
      bi = i;
    }
  }
  idx[r] = bi;
  if (val) val[r] = best;
}

// One decode step forward on the device: position += 1, context = position + 1,
// slot = block_table[b][position / bs] * bs + position % bs, next input id =
// the token just sampled.
__global__ void k_decode_advance(int* __restrict__ positions, int* __restrict__ ctx_lens,
                                 int* __restrict__ slots, const int* __restrict__ block_tables,
                                 int* __restrict__ ids, const int* __restrict__ sampled, int batch,
                                 int max_blocks, int block_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int pos = positions[b] + 1;
  positions[b] = pos;
  ctx_lens[b] = pos + 1;
  const int blk = pos / block_size < max_blocks ? block_tables[size_t(b) * max_blocks + pos / block_size] : -1;
  slots[b] = blk >= 0 ? blk * block_size + pos % block_size : -1;
  if (sampled) ids[b] = sampled[b];
}

}  // namespace bl

using namespace bl;

extern "C" int bl_rmsnorm(const void* x, const void* residual, const void* gamma, void* out,
                          void* residual_out, int rows, int hidden, float eps, const void* partials,
                          int nsplit, size_t slab, void* stream, char* err, size_t errlen) {
  if (rows < 1 || hidden < 8 || (hidden & 7) || hidden / 8 > 512 * kNormMaxVpt) {
    set_err(err, errlen, "barlink: rmsnorm needs hidden %% 8 == 0 and hidden <= %d", 512 * kNormMaxVpt * 8);
    return -1;
  }
  const int vpr = hidden / 8;
  int threads = (vpr + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  launch_k(k_rmsnorm, dim3(rows), dim3(threads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const uint4*>(x), static_cast<const uint4*>(residual),
      static_cast<const uint4*>(gamma), static_cast<uint4*>(out), static_cast<uint4*>(residual_out),
      vpr, eps, static_cast<const float*>(partials), nsplit, slab);
  OPS_LAUNCH_CHECK("rmsnorm");
  return 0;
}

extern "C" int bl_rope_kv_write(void* qkv, const void* partials, int nsplit, size_t slab,
                                const void* bias, const int* positions, const int* slots,
                                void* k_cache, void* v_cache, int rows, int nq, int nkv, int hd,
                                int block_size, float theta, void* stream, char* err,
                                size_t errlen) {
  if (rows < 1 || hd < 16 || (hd & 15) || hd > 256) {
    set_err(err, errlen, "barlink: rope_kv_write needs head_dim in 16..256, multiple of 16");
    return -1;
  }
  const int hpb = kRopeHeads * (hd / 2) <= 256 ? kRopeHeads : 256 / (hd / 2);
  launch_k(k_rope_kv_write, dim3(rows, (nq + 2 * nkv + hpb - 1) / hpb), dim3(hpb * (hd / 2)), 0,
           static_cast<cudaStream_t>(stream),
      static_cast<__nv_bfloat16*>(qkv), static_cast<const float*>(partials), nsplit, slab,
      static_cast<const __nv_bfloat16*>(bias), positions, slots, static_cast<__nv_bfloat16*>(k_cache),
      static_cast<__nv_bfloat16*>(v_cache), nq, nkv, hd, block_size, log2f(theta));
  OPS_LAUNCH_CHECK("rope_kv_write");
  return 0;
}

extern "C" int bl_rope(void* x, const int* positions, int rows, int heads, int hd, int row_stride,
                       float theta, int axes, void* stream, char* err, size_t errlen) {
  if (rows < 1 || axes < 1 || axes > 2 || (hd % (2 * axes))) {
    set_err(err, errlen, "barlink: rope needs head_dim divisible by 2*axes (axes 1 or 2)");
    return -1;
  }
  launch_k(k_rope, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<__nv_bfloat16*>(x), positions, heads, hd, row_stride, log2f(theta), axes);
  OPS_LAUNCH_CHECK("rope");
  return 0;
}

extern "C" int bl_silu_mul(const void* gate_up, void* out, int rows, int inter, int interleaved,
                           void* stream, char* err, size_t errlen) {
  const size_t total = size_t(rows) * inter;
  int grid = int((total + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  launch_k(k_silu_mul, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, inter,
      interleaved);
  OPS_LAUNCH_CHECK("silu_mul");
  return 0;
}

extern "C" int bl_silu_mul_slabs(const void* slabs, int nsplit, void* out, int rows, int inter, void* stream,
                                 char* err, size_t errlen) {
  if (nsplit < 1 || rows < 1 || (inter & 3)) {
    set_err(err, errlen, "barlink: silu_mul over slabs needs inter %% 4 == 0");
    return -1;
  }
  const size_t total4 = size_t(rows) * inter / 4;
  size_t grid = (total4 + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  launch_k(k_silu_mul_slabs, dim3(unsigned(grid)), dim3(256), 0, static_cast<cudaStream_t>(stream),
           static_cast<const float*>(slabs), size_t(rows) * 2 * inter, nsplit,
           static_cast<__nv_bfloat16*>(out), total4);
  OPS_LAUNCH_CHECK("silu_mul_slabs");
  return 0;
}

extern "C" int bl_embedding(const int* ids, const void* table, void* out, int rows, int hidden,
                            int vocab_lo, int vocab_hi, void* stream, char* err, size_t errlen) {
  if (hidden & 7) {
    set_err(err, errlen, "barlink: embedding needs hidden %% 8 == 0");
    return -1;
  }
  launch_k(k_embedding, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
      ids, static_cast<const uint4*>(table), static_cast<uint4*>(out), hidden / 8, vocab_lo,
      vocab_hi);
  OPS_LAUNCH_CHECK("embedding");
  return 0;
}

extern "C" int bl_argmax(const void* logits, int rows, int n, int ld, int offset, int* idx,
                         float* val, void* scratch, size_t scratch_bytes, void* stream, char* err,
                         size_t errlen) {
  if (!scratch || scratch_bytes < size_t(rows) * kArgmaxChunks * sizeof(float2)) {
    set_err(err, errlen, "barlink: argmax needs %zu bytes of scratch",
            size_t(rows) * kArgmaxChunks * sizeof(float2));
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  launch_k(k_argmax, dim3(rows, kArgmaxChunks), dim3(256), 0, st,
           static_cast<const __nv_bfloat16*>(logits), n, ld, offset, static_cast<float2*>(scratch),
           rows);
  OPS_LAUNCH_CHECK("argmax");
  launch_k(k_argmax_merge, dim3((rows + 127) / 128), dim3(128), 0, st,
           static_cast<const float2*>(scratch), kArgmaxChunks, rows, idx, val);
  OPS_LAUNCH_CHECK("argmax_merge");
  return 0;
}

extern "C" int bl_argmax_parts(const void* logits, int rows, int n, int ld, int offset, void* parts, void* stream,
                               char* err, size_t errlen) {
  if (!parts || (reinterpret_cast<uintptr_t>(parts) & 7u)) {
    set_err(err, errlen, "barlink: argmax_parts needs an 8-byte aligned output of %d x rows pairs", kArgmaxChunks);
    return -1;
  }
  launch_k(k_argmax, dim3(rows, kArgmaxChunks), dim3(256), 0, static_cast<cudaStream_t>(stream),
           static_cast<const __nv_bfloat16*>(logits), n, ld, offset, static_cast<float2*>(parts), rows);
  OPS_LAUNCH_CHECK("argmax_parts");
  return 0;
}
extern "C" int bl_argmax_chunks(void) { return kArgmaxChunks; }

extern "C" int bl_decode_advance(int* positions, int* ctx_lens, int* slots, const int* block_tables,
                                 int* ids, const int* sampled, int batch, int max_blocks,
                                 int block_size, void* stream, char* err, size_t errlen) {
  launch_k(k_decode_advance, dim3((batch + 127) / 128), dim3(128), 0,
           static_cast<cudaStream_t>(stream), positions, ctx_lens, slots, block_tables, ids, sampled,
           batch, max_blocks, block_size);
  OPS_LAUNCH_CHECK("decode_advance");
  return 0;
}

extern "C" int bl_argmax_merge(const void* pairs, int world, int rows, int* idx, void* stream,
                               char* err, size_t errlen) {
  launch_k(k_argmax_merge, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const float2*>(pairs), world, rows, idx, static_cast<float*>(nullptr));
  OPS_LAUNCH_CHECK("argmax_merge");
  return 0;
}

extern "C" int bl_paged_attn_decode(const void* q, int q_stride, const void* k_cache,
                                    const void* v_cache, const int* block_tables,
                                    const int* ctx_lens, void* out, int batch, int nq, int nkv,
                                    int hd, int block_size, int max_blocks, float scale, int splits,
                                    void* scratch, size_t scratch_bytes, void* stream, char* err,
                                    size_t errlen) {
  if (hd != kHd || block_size != kPageTokens) {
    set_err(err, errlen, "barlink: paged attention is built for head_dim %d and block size %d", kHd,
            kPageTokens);
    return -1;
  }
  if (nkv < 1 || nq % nkv || nq / nkv > 16) {
    set_err(err, errlen, "barlink: paged attention needs nq %% nkv == 0 and at most 16 query heads per KV head");
    return -1;
  }
  if (splits <= 0) {
    // enough CTAs to fill the GPU once; more splits only add merge traffic.  From 64 CTAs
    // on, splitting measured no faster than one CTA per (sequence, KV head) and costs the
    // merge kernel, so it is not done.
    const int want = batch * nkv >= 64 ? 1 : (sm_count() + batch * nkv - 1) / (batch * nkv);
    const int by_len = max_blocks / (2 * kAttnWarps) > 0 ? max_blocks / (2 * kAttnWarps) : 1;
    splits = want < by_len ? want : by_len;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  const size_t need = size_t(batch) * nq * splits * (kHd + 2) * sizeof(float);
  if (splits > 1 && (!scratch || scratch_bytes < need)) splits = 1;
  static bool attr = false;
  const int smem = kAttnWarps * kWarpSmem;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_paged_attn_decode,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: paged attention shared memory opt-in failed: %s",
              cudaGetErrorString(e));
      return -1;
    }
    attr = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_k(k_paged_attn_decode, dim3(nkv, batch, splits), dim3(kAttnWarps * 32), smem, st,
      static_cast<const __nv_bfloat16*>(q), q_stride, static_cast<const __nv_bfloat16*>(k_cache),
      static_cast<const __nv_bfloat16*>(v_cache), block_tables, ctx_lens,
      static_cast<__nv_bfloat16*>(out), static_cast<float*>(scratch), nq, nkv, max_blocks,
      scale_log2);
  OPS_LAUNCH_CHECK("paged_attn_decode");
  if (splits > 1) {
    launch_k(k_attn_merge, dim3(batch * nq), dim3(kHd), 0, st, static_cast<const float*>(scratch),
                                             static_cast<__nv_bfloat16*>(out), splits);
    OPS_LAUNCH_CHECK("attn_merge");
  }
  return 0;
}

// RoPE + KV write + paged attention in one launch.  qkv: bf16 rows of width
// (nq + 2 nkv) * hd with pitch q_stride, or null with `slabs` = nsplit_in fp32
// slabs [rows][width] `slab` floats apart (+ optional bias of `width`).
extern "C" int bl_rope_attn_decode(const void* qkv, int q_stride, const void* slabs, int nsplit_in,
                                   size_t slab, const void* bias, const int* positions, const int* slots,
                                   float theta, void* k_cache, void* v_cache, const int* block_tables,
                                   const int* ctx_lens, void* out, int batch, int nq, int nkv,
                                    int hd, int block_size, int max_blocks, float scale, int splits,
                                    void* scratch, size_t scratch_bytes, void* counters, void* stream,
                                    char* err, size_t errlen) {
  if (hd != kHd || block_size != kPageTokens) {
    set_err(err, errlen, "barlink: paged attention is built for head_dim %d and block size %d", kHd,
            kPageTokens);
    return -1;
  }
  if (nkv < 1 || nq % nkv || nq / nkv > 16) {
    set_err(err, errlen, "barlink: paged attention needs nq %% nkv == 0 and at most 16 query heads per KV head");
    return -1;
  }
  if (batch * nkv > 65536) counters = nullptr;
  if (splits <= 0 && counters) {
    // the merge is done inside the kernel, so a split costs no launch: fill the resident slots
    // (two CTAs of this kernel fit on an SM)
    static const int env_splits = [] {
      const char* v = getenv("BL_ATTN_SPLITS");
      return (v && *v) ? atoi(v) : 0;
    }();
    // from 64 (sequence, KV head) pairs on, splitting measured no faster even with the merge inside
    // the kernel (TP=8 shard, batch 64 x 1024 tokens: 2.32 ms per step unsplit, 2.52 / 2.39 with 2 / 4)
    const int want = env_splits > 0 ? env_splits
                     : batch * nkv >= 64 ? 1 : (sm_count() + batch * nkv - 1) / (batch * nkv);
    const int by_len = max_blocks / (2 * kAttnWarps) > 0 ? max_blocks / (2 * kAttnWarps) : 1;
    splits = want < by_len ? want : by_len;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  if (splits <= 0) {
    // enough CTAs to fill the GPU once; more splits only add merge traffic.  From 64 CTAs
    // on, splitting measured no faster than one CTA per (sequence, KV head) and costs the
    // merge kernel, so it is not done.
    const int want = batch * nkv >= 64 ? 1 : (sm_count() + batch * nkv - 1) / (batch * nkv);
    const int by_len = max_blocks / (2 * kAttnWarps) > 0 ? max_blocks / (2 * kAttnWarps) : 1;
    splits = want < by_len ? want : by_len;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  const size_t need = size_t(batch) * nq * splits * (kHd + 2) * sizeof(float);
  if (splits > 1 && (!scratch || scratch_bytes < need)) splits = 1;
  if ((!qkv && !slabs) || !positions || !slots || ((q_stride | (nq + 2 * nkv) * hd) & 1)) {
    set_err(err, errlen, "barlink: fused RoPE + attention needs the QKV projection, positions and slots");
    return -1;
  }
  QkvSrc src;
  src.qkv = static_cast<const __nv_bfloat16*>(qkv);
  src.q_stride = q_stride;
  src.slabs = static_cast<const float*>(slabs);
  src.nsplit = nsplit_in;
  src.slab = slab;
  src.bias = static_cast<const __nv_bfloat16*>(bias);
  src.width = (nq + 2 * nkv) * hd;
  static bool attr = false;
  const int smem = kAttnWarps * kWarpSmem;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_rope_attn_decode,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: paged attention shared memory opt-in failed: %s",
              cudaGetErrorString(e));
      return -1;
    }
    attr = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_k(k_rope_attn_decode, dim3(nkv, batch, splits), dim3(kAttnWarps * 32), smem, st, src, positions,
      slots, log2f(theta), static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
      block_tables, ctx_lens,
      static_cast<__nv_bfloat16*>(out), static_cast<float*>(scratch), nq, nkv, max_blocks,
      scale_log2, static_cast<uint32_t*>(counters));
  OPS_LAUNCH_CHECK("rope_attn_decode");
  if (splits > 1 && !counters) {
    launch_k(k_attn_merge, dim3(batch * nq), dim3(kHd), 0, st, static_cast<const float*>(scratch),
                                             static_cast<__nv_bfloat16*>(out), splits);
    OPS_LAUNCH_CHECK("attn_merge");
  }
  return 0;
}

// ---------------------------------------------------------------------------
// MMDiT (Flux-style) elementwise kernels
// ---------------------------------------------------------------------------
// Per-head RMSNorm of q and k (weights gq, gk over head_dim = 128) followed by
// RoPE with 1 or 2 position axes, on a fused qkv row [(3*heads) * 128].
// One warp per (token, head); lane l owns dims l, l+32, l+64, l+96, which are
// exactly the rotation partners for both axis layouts.
__global__ void __launch_bounds__(256) k_qknorm_rope(__nv_bfloat16* __restrict__ qkv,
                                                     const __nv_bfloat16* __restrict__ gq,
                                                     const __nv_bfloat16* __restrict__ gk,
                                                     const int* __restrict__ positions, int heads,
                                                     int row_stride, float eps, float log2_theta,
                                                     int axes) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31;
  for (int h = (threadIdx.x >> 5) + blockIdx.y * 8; h < 2 * heads; h += 8 * gridDim.y) {
    __nv_bfloat16* p = qkv + size_t(row) * row_stride + size_t(h) * 128;  // q heads then k heads
    const __nv_bfloat16* gm = h < heads ? gq : gk;
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __bfloat162float(p[lane + 32 * j]);
    if (gm) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / 128.f + eps);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        x[j] = __bfloat162float(__float2bfloat16(x[j] * rstd)) * __bfloat162float(gm[lane + 32 * j]);
    }
    if (axes == 2) {
      // dims [0,64): axis 0, pairs (l, l+32); dims [64,128): axis 1, pairs (l+64, l+96)
      const float inv = exp2f(-log2_theta * (2.f * float(lane) / 64.f));
#pragma unroll
      for (int ax = 0; ax < 2; ++ax) {
        float sn, cs;
        sincosf(float(positions[row * 2 + ax]) * inv, &sn, &cs);
        const float a = x[2 * ax], b = x[2 * ax + 1];
        x[2 * ax] = a * cs - b * sn;
        x[2 * ax + 1] = b * cs + a * sn;
      }
    } else {
      // pairs (l, l+64) and (l+32, l+96)
      const float pos = float(positions[row]);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float inv = exp2f(-log2_theta * (2.f * float(lane + 32 * j) / 128.f));
        float sn, cs;
        sincosf(pos * inv, &sn, &cs);
        const float a = x[j], b = x[j + 2];
        x[j] = a * cs - b * sn;
        x[j + 2] = b * cs + a * sn;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) p[lane + 32 * j] = __float2bfloat16(x[j]);
  }
}

// out = LayerNorm(x) * (1 + scale[b]) + shift[b]   (no affine weights; b = row / rows_per_batch)
__global__ void __launch_bounds__(512) k_layernorm_modulate(const uint4* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ shift,
                                                            const __nv_bfloat16* __restrict__ scale,
                                                            uint4* __restrict__ out, int vpr,
                                                            int rows_per_batch, int mod_stride,
                                                            float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_a[16], s_b[16];
  __shared__ float s_mean, s_rstd;
  const size_t row = blockIdx.x;
  const int b = int(row / rows_per_batch);
  float v[kNormMaxVpt][8];
  float sum = 0.f, sq = 0.f;
#pragma unroll
  for (int k = 0; k < kNormMaxVpt; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < vpr) {
      const uint4 a = x[row * vpr + i];
      const float2 p0 = unpack_bf16x2(a.x), p1 = unpack_bf16x2(a.y), p2 = unpack_bf16x2(a.z),
                   p3 = unpack_bf16x2(a.w);
      const float f[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = f[j];
        sum += f[j];
        sq += f[j] * f[j];
      }
    }
  }
  sum = warp_sum(sum);
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) {
    s_a[threadIdx.x >> 5] = sum;
    s_b[threadIdx.x >> 5] = sq;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float a = threadIdx.x < (blockDim.x >> 5) ? s_a[threadIdx.x] : 0.f;
    float c = threadIdx.x < (blockDim.x >> 5) ? s_b[threadIdx.x] : 0.f;
    a = warp_sum(a);
    c = warp_sum(c);
    if (threadIdx.x == 0) {
      const float n = float(vpr * 8);
      const float mean = a / n;
      s_mean = mean;
      s_rstd = rsqrtf(fmaxf(c / n - mean * mean, 0.f) + eps);
    }
  }
  __syncthreads();
  const float mean = s_mean, rstd = s_rstd;
#pragma unroll
  for (int k = 0; k < kNormMaxVpt; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < vpr) {
      const uint4 sh = *reinterpret_cast<const uint4*>(shift + size_t(b) * mod_stride + i * 8);
      const uint4 sc = *reinterpret_cast<const uint4*>(scale + size_t(b) * mod_stride + i * 8);
      const float2 h0 = unpack_bf16x2(sh.x), h1 = unpack_bf16x2(sh.y), h2 = unpack_bf16x2(sh.z),
                   h3 = unpack_bf16x2(sh.w);
      const float2 c0 = unpack_bf16x2(sc.x), c1 = unpack_bf16x2(sc.y), c2 = unpack_bf16x2(sc.z),
                   c3 = unpack_bf16x2(sc.w);
      const float hs[8] = {h0.x, h0.y, h1.x, h1.y, h2.x, h2.y, h3.x, h3.y};
      const float cs[8] = {c0.x, c0.y, c1.x, c1.y, c2.x, c2.y, c3.x, c3.y};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd * (1.f + cs[j]) + hs[j];
      out[row * vpr + i] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                      pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
  }
}

// x += gate[b] * y
__global__ void k_gate_residual(uint4* __restrict__ x, const uint4* __restrict__ y,
                                const __nv_bfloat16* __restrict__ gate, int vpr, int rows_per_batch,
                                int mod_stride, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += size_t(gridDim.x) * blockDim.x) {
    const size_t row = t / vpr;
    const int i = int(t % vpr);
    const int b = int(row / rows_per_batch);
    const uint4 a = x[t], c = y[t];
    const uint4 g = *reinterpret_cast<const uint4*>(gate + size_t(b) * mod_stride + i * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = unpack_bf16x2(aw[j]), fc = unpack_bf16x2(cw[j]), fg = unpack_bf16x2(gw[j]);
      o[j] = pack_bf16x2(fa.x + fg.x * fc.x, fa.y + fg.y * fc.y);
    }
    x[t] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------------------
// arg max for callers that may not allocate (see bl_noalloc.h)
// ---------------------------------------------------------------------------
#include "bl_noalloc.h"

namespace bl {
// Partial (value, index) pairs of k_argmax: [kArgmaxChunks][rows].  Part of
// the library image, so no call ever has to allocate it.  In host code this
// name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float2 g_argmax_scratch[BL_ARGMAX_NOALLOC_MAX_ROWS * kArgmaxChunks];

constexpr int kNoallocMaxDevices = 64;
static float2* g_argmax_scratch_addr[kNoallocMaxDevices];  // per device, filled on first use
static std::mutex g_argmax_scratch_mu;
}  // namespace bl

extern "C" int bl_argmax_noalloc(const void* logits, int rows, int n, int ld, int offset, int* idx,
                                 float* val, void* stream, char* err, size_t errlen) {
  if (!logits || !idx || rows < 1 || n < 1 || ld < n) {
    set_err(err, errlen, "barlink: argmax_noalloc needs logits, idx, rows >= 1, n >= 1 and ld >= n");
    return -1;
  }
  if (rows > BL_ARGMAX_NOALLOC_MAX_ROWS) {
    set_err(err, errlen,
            "barlink: argmax_noalloc handles at most %d rows per call (%d given); split the batch or "
            "use bl_argmax with a scratch buffer of your own",
            BL_ARGMAX_NOALLOC_MAX_ROWS, rows);
    return -1;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) {
    set_err(err, errlen, "barlink: argmax_noalloc cannot tell the current device: %s",
            e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range");
    return -1;
  }
  float2* scratch = nullptr;
  {
    // once per device, with that device current: the array's address there
    std::lock_guard<std::mutex> g(g_argmax_scratch_mu);
    if (!g_argmax_scratch_addr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_argmax_scratch);
      if (e != cudaSuccess || !p) {
        set_err(err, errlen, "barlink: argmax_noalloc could not resolve its scratch array on device %d: %s",
                dev, cudaGetErrorString(e));
        return -1;
      }
      g_argmax_scratch_addr[dev] = static_cast<float2*>(p);
    }
    scratch = g_argmax_scratch_addr[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // plain launches: this path must not depend on how the caller's other kernels were launched
  k_argmax<<<dim3(rows, kArgmaxChunks), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), n, ld,
                                                     offset, scratch, rows);
  OPS_LAUNCH_CHECK("argmax_noalloc");
  k_argmax_merge<<<(rows + 127) / 128, 128, 0, st>>>(scratch, kArgmaxChunks, rows, idx, val);
  OPS_LAUNCH_CHECK("argmax_noalloc merge");
  return 0;
}

extern "C" int bl_qknorm_rope(void* qkv, const void* gq, const void* gk, const int* positions, int rows,
                              int heads, int hd, int row_stride, float eps, float theta, int axes,
                              void* stream, char* err, size_t errlen) {
  if (hd != 128 || axes < 1 || axes > 2 || rows < 1) {
    set_err(err, errlen, "barlink: qknorm_rope is built for head_dim 128 and 1 or 2 position axes");
    return -1;
  }
  const int gy = (2 * heads + 7) / 8 < 8 ? (2 * heads + 7) / 8 : 8;
  launch_k(k_qknorm_rope, dim3(rows, gy), dim3(256), 0, static_cast<cudaStream_t>(stream),
           static_cast<__nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(gq),
           static_cast<const __nv_bfloat16*>(gk), positions, heads, row_stride, eps, log2f(theta), axes);
  OPS_LAUNCH_CHECK("qknorm_rope");
  return 0;
}

extern "C" int bl_layernorm_modulate(const void* x, const void* shift, const void* scale, void* out,
                                     int rows, int hidden, int rows_per_batch, int mod_stride, float eps,
                                     void* stream, char* err, size_t errlen) {
  if (rows < 1 || (hidden & 7) || hidden / 8 > 512 * kNormMaxVpt || rows_per_batch < 1 || (mod_stride & 7)) {
    set_err(err, errlen, "barlink: layernorm_modulate needs hidden %% 8 == 0 (<= %d) and a modulation pitch %% 8 == 0",
            512 * kNormMaxVpt * 8);
    return -1;
  }
  const int vpr = hidden / 8;
  int threads = (vpr + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  launch_k(k_layernorm_modulate, dim3(rows), dim3(threads), 0, static_cast<cudaStream_t>(stream),
           static_cast<const uint4*>(x), static_cast<const __nv_bfloat16*>(shift),
           static_cast<const __nv_bfloat16*>(scale), static_cast<uint4*>(out), vpr, rows_per_batch,
           mod_stride, eps);
  OPS_LAUNCH_CHECK("layernorm_modulate");
  return 0;
}

extern "C" int bl_gate_residual(void* x, const void* y, const void* gate, int rows, int hidden,
                                int rows_per_batch, int mod_stride, void* stream, char* err,
                                size_t errlen) {
  if (rows < 1 || (hidden & 7) || (mod_stride & 7) || rows_per_batch < 1) {
    set_err(err, errlen, "barlink: gate_residual needs hidden %% 8 == 0 and a gate pitch %% 8 == 0");
    return -1;
  }
  const size_t total = size_t(rows) * (hidden / 8);
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_k(k_gate_residual, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
           static_cast<uint4*>(x), static_cast<const uint4*>(y), static_cast<const __nv_bfloat16*>(gate),
           hidden / 8, rows_per_batch, mod_stride, total);
  OPS_LAUNCH_CHECK("gate_residual");
  return 0;
}
