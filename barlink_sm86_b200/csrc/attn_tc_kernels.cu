// SPDX-License-Identifier: MIT
//
// Dense attention on the 5th-generation tensor cores (head_dim 128, bf16):
// prefill (causal, GQA) and MMDiT joint attention over packed sequences.
// The reference calls a library kernel here (flash-attn / SDPA inside
// transformers and diffusers: demos/flux2_tp/worker.py:148-160,
// demos/qwen_tp/qwen38_int8/worker.py:515-537).
//
// One CTA owns 256 query rows of one head as two 128-row tiles and walks the
// keys in tiles of 64:
//
//   warp 0      TMA producer: Q once, then a 4-deep ring of (K tile, V^T tile)
//   warp 1      one thread issues tcgen05.mma: S_t = Q_t K^T into TMEM (128x64 fp32),
//               O_t += P_t V into TMEM (128x128 fp32), for tiles t = 0, 1 in turn
//   warps 2-5   softmax of tile 0: every thread owns one query row (TMEM lane),
//   warps 6-9   softmax of tile 1   reads its 64 scores with tcgen05.ld, keeps the
//               running max and sum in registers, writes P (bf16) into shared
//               memory in the swizzled K-major layout the tensor core reads
//
// While one tile's softmax runs, the tensor core works on the other tile
// (order PV0_j, S0_j+1, PV1_j, S1_j+1), so neither side waits for long.  The
// accumulator is rescaled only when the running max has grown by more than
// 2^8 since the last rescale (the stale max is exact after the final division
// by the row sum), which takes the TMEM read-modify-write out of the loop.
// V is consumed as V^T [head_dim][keys] so that both operands of P V are
// K-major; a small kernel transposes V into a scratch buffer first.
//
// Every wait is bounded; a wait that runs out sets the CTA's abort word, all
// roles leave their loops, TMEM is freed and the error flag is raised.
#include <cuda_bf16.h>
#include <stdint.h>

#include "bl_ops.h"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

constexpr int kTcBM = 128;       // query rows per tile
constexpr int kTcTiles = 2;      // tiles per CTA
constexpr int kTcBKV = 64;       // keys per step
constexpr int kTcHD = 128;
constexpr int kTcStages = 4;
constexpr int kTcThreads = 320;
constexpr uint32_t kTcQBytes = kTcBM * kTcHD * 2;          // 32 KiB per query tile
constexpr uint32_t kTcPBytes = kTcBM * kTcBKV * 2;         // 16 KiB per P tile
constexpr uint32_t kTcKBytes = kTcBKV * kTcHD * 2;         // 16 KiB
constexpr uint32_t kTcVBytes = kTcHD * kTcBKV * 2;         // 16 KiB
constexpr uint32_t kTcOffP = kTcTiles * kTcQBytes;
constexpr uint32_t kTcOffKV = kTcOffP + kTcTiles * kTcPBytes;
constexpr uint32_t kTcStageBytes = kTcKBytes + kTcVBytes;
constexpr uint32_t kTcOffBar = kTcOffKV + kTcStages * kTcStageBytes;
constexpr uint32_t kTcSmem = kTcOffBar + 256 + 1024;       // barriers + alignment slack
constexpr uint32_t kTcTmemCols = 512;                      // S0 0-63, S1 64-127, O0 128-255, O1 256-383
constexpr float kTcRescale = 8.f;                          // log2 units

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// V [tokens, nkv, 128] (token stride v_stride) -> vt [nkv*128][batch*lpad]:
// sequence b's keys sit at columns b*lpad .. b*lpad+len; the pad is zeroed.
__global__ void __launch_bounds__(256) k_transpose_v(const __nv_bfloat16* __restrict__ v,
                                                     __nv_bfloat16* __restrict__ vt,
                                                     const int* __restrict__ cu_k, int v_stride,
                                                     int lpad, size_t vt_pitch) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __nv_bfloat16 tile[64][kTcHD + 8];
  const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * 64;
  const int k0 = cu_k[b], len = cu_k[b + 1] - k0;
  // 64 tokens x 128 dims: 16 threads per token row, 8 elements each
  for (int i = threadIdx.x; i < 64 * 16; i += 256) {
    const int r = i >> 4, c = (i & 15) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t0 + r < len) val = *reinterpret_cast<const uint4*>(v + size_t(k0 + t0 + r) * v_stride + h * kTcHD + c);
    *reinterpret_cast<uint4*>(&tile[r][c]) = val;
  }
  __syncthreads();
  // 128 dims x 64 tokens out: 8 threads per dim row, 8 tokens each
  for (int i = threadIdx.x; i < kTcHD * 8; i += 256) {
    const int d = i >> 3, c = (i & 7) * 8;
    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = tile[c + j][d];
    *reinterpret_cast<uint4*>(vt + size_t(h * kTcHD + d) * vt_pitch + size_t(b) * lpad + t0 + c) =
        *reinterpret_cast<const uint4*>(o);
  }
}

__global__ void __launch_bounds__(kTcThreads, 1)
    k_attn_tc(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_vt, __nv_bfloat16* __restrict__ out,
              const int* __restrict__ cu_q, const int* __restrict__ cu_k, int nq, int nkv, int o_stride,
              int lpad, float scale_log2, int causal, uint32_t* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTcOffBar);
  uint64_t* q_full = bars;             // 1
  uint64_t* kv_full = bars + 1;        // kTcStages
  uint64_t* kv_empty = bars + 5;       // kTcStages
  uint64_t* s_ready = bars + 9;        // 2
  uint64_t* p_ready = bars + 11;       // 2
  uint64_t* o_final = bars + 13;       // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(bars + 17);

  // cu_q / cu_k may come from the kernel just before this one
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, head = blockIdx.y, kvh = head / (nq / nkv);
  const int q0 = cu_q[b], lq = cu_q[b + 1] - q0;
  const int k0 = cu_k[b], lk = cu_k[b + 1] - k0;
  const int row0 = blockIdx.x * (kTcTiles * kTcBM);   // first query row of this CTA in its sequence
  if (row0 >= lq) return;
  const int off = lk - lq;                             // causal: key j visible to query i iff j <= i + off
  int kv_end = lk;
  if (causal) {
    const int last = min(lq, row0 + kTcTiles * kTcBM) - 1;
    kv_end = max(0, min(lk, last + off + 1));
  }
  const int n_steps = (kv_end + kTcBKV - 1) / kTcBKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < kTcTiles; ++t) {
      mbar_init(&s_ready[t], 1);
      mbar_init(&p_ready[t], kTcBM);
      mbar_init(&o_final[t], 1);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_vt);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTcTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(q_full, kTcTiles * kTcQBytes);
      for (int t = 0; t < kTcTiles; ++t)
        for (int h = 0; h < 2; ++h)
          tma_load_2d_hint_s(base + t * kTcQBytes + h * (kTcQBytes / 2), &tmap_q, smem_u32(q_full),
                             head * kTcHD + h * 64, q0 + row0 + t * kTcBM, kHintEvictFirst);
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      for (int j = 0; j < n_steps; ++j) {
        if (!mbar_wait_bounded(&kv_empty[stage], phase ^ 1u, s_abort)) break;
        const uint32_t dst = base + kTcOffKV + stage * kTcStageBytes;
        mbar_expect_tx(&kv_full[stage], kTcStageBytes);
        for (int h = 0; h < 2; ++h)
          tma_load_2d_hint_s(dst + h * (kTcKBytes / 2), &tmap_k, smem_u32(&kv_full[stage]),
                             kvh * kTcHD + h * 64, k0 + j * kTcBKV, kHintEvictLast);
        tma_load_2d_hint_s(dst + kTcKBytes, &tmap_vt, smem_u32(&kv_full[stage]), b * lpad + j * kTcBKV,
                           kvh * kTcHD, kHintEvictLast);
        ++issued;
        if (++stage == kTcStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (*s_abort) {
        // leaving early: let the copies still in flight land before the CTA exits
        for (int j = max(0, issued - kTcStages); j < issued; ++j) {
          const int s = j % kTcStages;
          const uint32_t ph = uint32_t(j / kTcStages) & 1u;
          for (uint32_t p = 0; p < (1u << 20); ++p)
            if (mbar_try_wait(&kv_full[s], ph)) break;
        }
        for (uint32_t p = 0; p < (1u << 20); ++p)
          if (mbar_try_wait(q_full, 0)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_s = umma_idesc_f16(kTcBM, kTcBKV, 1);
      const uint32_t idesc_o = umma_idesc_f16(kTcBM, kTcHD, 1);
      auto issue_s = [&](int t, int stage) {
        const uint32_t kb = base + kTcOffKV + stage * kTcStageBytes;
#pragma unroll
        for (int ks = 0; ks < kTcHD / 16; ++ks) {
          const uint64_t da = umma_desc_k_sw128(base + t * kTcQBytes + (ks >> 2) * (kTcQBytes / 2)) + uint64_t(2 * (ks & 3));
          const uint64_t db = umma_desc_k_sw128(kb + (ks >> 2) * (kTcKBytes / 2)) + uint64_t(2 * (ks & 3));
          umma_f16_ss(tmem_base + uint32_t(t * kTcBKV), da, db, idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_ready[t]);
      };
      auto issue_pv = [&](int t, int stage, bool acc) {
        const uint32_t vb = base + kTcOffKV + stage * kTcStageBytes + kTcKBytes;
#pragma unroll
        for (int ks = 0; ks < kTcBKV / 16; ++ks) {
          const uint64_t da = umma_desc_k_sw128(base + kTcOffP + t * kTcPBytes) + uint64_t(2 * ks);
          const uint64_t db = umma_desc_k_sw128(vb) + uint64_t(2 * ks);
          umma_f16_ss(tmem_base + 128u + uint32_t(t * kTcHD), da, db, idesc_o, (acc || ks > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait_bounded(q_full, 0, s_abort);
      int stage = 0;
      uint32_t phase = 0;
      if (ok) ok = mbar_wait_bounded(&kv_full[0], 0, s_abort);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0, 0);
        issue_s(1, 0);
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        int nstage = stage + 1;
        uint32_t nphase = phase;
        if (nstage == kTcStages) {
          nstage = 0;
          nphase ^= 1u;
        }
        const bool more = j + 1 < n_steps;
        for (int t = 0; t < kTcTiles && ok; ++t) {
          if (!mbar_wait_bounded(&p_ready[t], uint32_t(j) & 1u, s_abort)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_pv(t, stage, j > 0);
          if (more) {
            if (t == 0 && !mbar_wait_bounded(&kv_full[nstage], nphase, s_abort)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_s(t, nstage);
          } else {
            umma_commit(&o_final[t]);
          }
        }
        if (ok) umma_commit(&kv_empty[stage]);
        stage = nstage;
        phase = nphase;
      }
    }
  } else {
    // ------------------------------ softmax -------------------------------
    const int t = (warp - 2) >> 2;                 // tile of this warp group
    const int quarter = warp & 3;                  // TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;           // row inside the tile
    const int qi = row0 + t * kTcBM + row;         // query index inside the sequence
    const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + uint32_t(t * kTcBKV);
    const uint32_t o_addr = lane_addr + 128u + uint32_t(t * kTcHD);
    const uint32_t p_row = base + kTcOffP + t * kTcPBytes + row * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_steps; ++j) {
      if (!mbar_wait_bounded(&s_ready[t], uint32_t(j) & 1u, s_abort)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float s[kTcBKV];
      {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(s_addr, r0);
        tmem_ld_32x32(s_addr + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          s[c] = __uint_as_float(r0[c]) * scale_log2;
          s[c + 32] = __uint_as_float(r1[c]) * scale_log2;
        }
      }
      const int kbase = j * kTcBKV;
      const int lim = causal ? min(lk, qi + off + 1) : lk;   // keys [0, lim) are visible to this row
      if (kbase + kTcBKV > lim) {
#pragma unroll
        for (int c = 0; c < kTcBKV; ++c)
          if (kbase + c >= lim) s[c] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int c = 1; c < kTcBKV; ++c) mx = fmaxf(mx, s[c]);
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + kTcRescale;          // also true on the first finite max
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = (m_new == -INFINITY) ? 1.f : ex2_approx(m_used - m_new);
        if (j > 0) {
          // PV of the previous step has completed: its MMAs were issued before the
          // S that s_ready just announced, and the tensor pipe runs in order
#pragma unroll 1
          for (int c0 = 0; c0 < kTcHD; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(o_addr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
            tmem_st_32x32(o_addr + c0, r);
          }
          tmem_st_wait();
        }
        l *= alpha;
        m_used = m_new;
      }
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
      uint32_t pk[kTcBKV / 2];
#pragma unroll
      for (int c = 0; c < kTcBKV; c += 2) {
        const float p0 = ex2_approx(s[c] - mref), p1 = ex2_approx(s[c + 1] - mref);
        sum += p0 + p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l += sum;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_row + ((c ^ (row & 7)) << 4)),
                     "r"(pk[4 * c]), "r"(pk[4 * c + 1]), "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                     : "memory");
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[t]);
    }
    // ------------------------------ output --------------------------------
    const bool valid = qi < lq;
    __nv_bfloat16* orow = out + size_t(q0 + qi) * o_stride + head * kTcHD;
    if (n_steps == 0) {
      if (valid)
        for (int c = 0; c < kTcHD; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
    } else if (ok && mbar_wait_bounded(&o_final[t], 0, s_abort)) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTcHD; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(o_addr + c0, r);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            *reinterpret_cast<uint4*>(orow + c0 + c) = make_uint4(
                pack_bf16x2(__uint_as_float(r[c]) * inv, __uint_as_float(r[c + 1]) * inv),
                pack_bf16x2(__uint_as_float(r[c + 2]) * inv, __uint_as_float(r[c + 3]) * inv),
                pack_bf16x2(__uint_as_float(r[c + 4]) * inv, __uint_as_float(r[c + 5]) * inv),
                pack_bf16x2(__uint_as_float(r[c + 6]) * inv, __uint_as_float(r[c + 7]) * inv));
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTcTmemCols);
  }
  if (threadIdx.x == 0 && *s_abort && err) *err = 1u;
}

}  // namespace bl

using namespace bl;

extern "C" size_t bl_attn_tc_scratch_bytes(int batch, int max_k, int nkv) {
  const size_t lpad = size_t((max_k + kTcBKV - 1) / kTcBKV) * kTcBKV;
  return size_t(nkv) * kTcHD * lpad * size_t(batch) * 2;
}

// Tensor-core dense attention.  `vt` is scratch of bl_attn_tc_scratch_bytes();
// `total_q` / `total_k` are the row counts of q and k (cu_q[batch], cu_k[batch]).
extern "C" int bl_attn_fwd_tc(const void* q, const void* k, const void* v, void* out, const int* cu_q,
                              const int* cu_k, int batch, int max_q, int max_k, int total_q, int total_k,
                              int nq, int nkv, int hd, int q_stride, int k_stride, int v_stride,
                              int o_stride, float scale, int causal, void* vt, void* err_flag, void* stream,
                              char* err, size_t errlen) {
  if (hd != kTcHD || nkv < 1 || nq % nkv) {
    set_err(err, errlen, "barlink: tensor-core attention is built for head_dim %d and nq %% nkv == 0", kTcHD);
    return -1;
  }
  if ((q_stride | k_stride | v_stride | o_stride) & 7) {
    set_err(err, errlen, "barlink: attention needs token strides that are multiples of 8 elements");
    return -1;
  }
  if (batch < 1 || max_q < 1 || max_k < 1) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int lpad = (max_k + kTcBKV - 1) / kTcBKV * kTcBKV;
  const size_t pitch = size_t(lpad) * batch;
  launch_k(k_transpose_v, dim3(lpad / 64, nkv, batch), dim3(256), 0, st,
           static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(vt), cu_k, v_stride, lpad, pitch);
  CUtensorMap tq, tk, tv;
  if (make_tmap_kmajor(q, uint64_t(total_q), uint64_t(nq) * kTcHD, uint64_t(q_stride), kTcBM, 2, &tq, err, errlen) ||
      make_tmap_kmajor(k, uint64_t(total_k), uint64_t(nkv) * kTcHD, uint64_t(k_stride), kTcBKV, 2, &tk, err, errlen) ||
      make_tmap_kmajor(vt, uint64_t(nkv) * kTcHD, pitch, pitch, kTcHD, 2, &tv, err, errlen))
    return -1;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_attn_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTcSmem));
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: tensor-core attention shared memory opt-in failed: %s", cudaGetErrorString(e));
      return -1;
    }
    attr = true;
  }
  dim3 grid((max_q + kTcTiles * kTcBM - 1) / (kTcTiles * kTcBM), nq, batch);
  cudaError_t e = launch_k(k_attn_tc, grid, dim3(kTcThreads), kTcSmem, st, tq, tk, tv,
                           static_cast<__nv_bfloat16*>(out), cu_q, cu_k, nq, nkv, o_stride, lpad,
                           scale * 1.4426950408889634f, causal, static_cast<uint32_t*>(err_flag));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: tensor-core attention launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
