// SPDX-License-Identifier: MIT
//
// Decode linears for tensor-parallel inference: one kernel per linear layer of
// the decode step, with the collective that surrounds it folded in.
//
//   y[tokens, n] = x[tokens, k] @ w[n, k]^T          tokens <= 64, bf16, fp32 accumulate
//
// Shape of the kernel.  A thread-block cluster of CL CTAs owns one 128-row
// tile of w; CTA q of the cluster multiplies its own share of the k-blocks
// (tcgen05.mma, 128 x BN accumulator in TMEM, operands staged by TMA through
// an mbarrier ring), so a skinny decode product still fills the SMs.  The CL
// partial accumulators are summed through distributed shared memory: every CTA
// stores its partial columns into the shared memory of the CTA that owns those
// columns, one cluster barrier, and each CTA finishes its own columns.  No
// partial sum ever goes to global memory and no second kernel reduces.
//
// Prologue (optional): the activation operand is RMSNorm(residual + sum over
// ranks of the previous row-parallel linear).  The per-rank partial rows sit in
// this GPU's one-shot inbox, where every rank's previous linear stored them
// (payload words are their own arrival flags).  The epilogue warps of the first
// CTAs -- idle until the first accumulator is ready -- gather, reduce, add the
// residual, normalise and publish the rows; the TMA producer of every CTA
// streams weight tiles meanwhile and requests activation tiles once the rows
// are published.  The all-reduce therefore costs no kernel of its own.
//
// Epilogue: store (+ bias); SiLU(gate) * up on interleaved rows; or round to
// bf16 and store the tile straight into the one-shot inbox of every rank over
// NVLink (16-byte peer stores), which is the first half of the all-reduce that
// the next linear's prologue completes.
//
// The reference reaches the same data flow with cuBLAS F.linear, an
// all_reduce hook per row-parallel module and framework RMSNorm kernels
// (demos/qwen_tp/qwen38_int8/worker.py:167-183, 224): four launches and two
// kernel boundaries around every collective.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bl_ops.h"
#include "comm_dev.cuh"
#include "gemm_core.cuh"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

constexpr int kDlinThreads = 192;
constexpr int kDlinMaxVpt = 8;  // 16-byte vectors per thread and row in the prologue: hidden <= 8192
constexpr int kDlinMaxCluster = 8;

struct DlinParams {
  int n, k, tokens, kblocks;
  int cpc;   // columns of the tile that each CTA of the cluster finishes (a multiple of 4)
  int cpcp;  // row pitch of the exchange buffer in floats (>= cpc, == 4 mod 8)
  int pro;  // 0: x is ready in memory; 1: gather + residual + RMSNorm fills x first
  int epi;  // 0: store (+bias); 1: SiLU(gate)*up; 2: push bf16 rows to every rank's inbox
  // prologue
  const uint4* res_in;
  uint4* res_out;
  const uint4* gamma;
  uint4* xnorm;   // the activation operand, [tokens][k] bf16, written here and read back by TMA
  float eps;
  uint32_t* sync; // [0] row segments published so far (all launches), [1] that count at launch, [2] exit ticket
  float* ss_part; // [tokens][nseg] sums of squares of the row segments (nseg = ceil(k / 1024))
  int pro_ctas;   // CTAs that share the gather: the first ones of the grid, all resident together
  // epilogue
  __nv_bfloat16* out;
  int ldo;
  const __nv_bfloat16* bias;
  int push_ld;    // row pitch (elements) of the inbox rows: the full hidden size
  uint32_t* err;  // set to 1 when a bounded wait inside the kernel ran out
  unsigned long long* trace;  // debug: 12 global-timer stamps per CTA, or null
  Comm c;         // the link (or its one-rank stand-in in local memory)
};

// CPS = CTAs per SM.  1: a deep operand ring and an exchange buffer of its own.  2: half the
// shared memory, so that the CTAs of the next linear are already resident (barriers, TMEM and the
// first weight tiles in place) while this one finishes; the exchange buffer then reuses the ring,
// which costs one more cluster barrier (nobody may write into a ring that is still being read).
template <int BN, int CPS>
struct DlinSmem {
  static constexpr int kStageA = kTileA * kTileK * 2;
  static constexpr int kStageB = BN * kTileK * 2;
  static constexpr int kStageBytes = kStageA + kStageB;
  static constexpr int kStages = CPS == 2 ? 4 : (BN >= 64 ? 7 : 8);
  static constexpr int kXbufBytes = BN >= 64 ? 52224 : 32768;  // checked against the cluster shape at launch
  static constexpr int kStageTileOff = CPS == 2 ? 65536 : 0;    // bf16 staging tile of the push epilogue
  static constexpr int kBarBytes = 1024;
  static constexpr int kBytes = kBarBytes + 1024 + kStages * kStageBytes + (CPS == 2 ? 0 : kXbufBytes);
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static_assert(CPS == 1 || kStages * kStageBytes >= kStageTileOff + BN * kTileA * 2, "staging tile must fit the ring");
};

__device__ __forceinline__ void bar_epi() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Reset the inbox buffer that the call before this one used (it is written again two calls
// from now); every CTA of the grid takes a share.
__device__ __forceinline__ void dlin_clear_prev(const Comm& c, uint32_t e, uint32_t prev_vecs, int et) {
  const size_t clr_off = c.lamport_off + size_t((e + 2u) % 3u) * (size_t(c.world) * c.lamport_slice);
  const uint4 unw = make_uint4(kUnwritten, kUnwritten, kUnwritten, kUnwritten);
  for (size_t i = size_t(blockIdx.x) * 128 + et; i < prev_vecs; i += size_t(gridDim.x) * 128)
    for (int r = 0; r < c.world; ++r) st_v4(c.base[c.rank] + clr_off + size_t(r) * c.lamport_slice + i * 16, unw);
}

// The in-kernel form of the same gather, spread over the whole grid: the unit of work is a
// segment of 128 consecutive 16-byte vectors of one row (one vector per epilogue thread), dealt
// out to the CTAs round robin, two segments in flight per thread so that all loads of a step go
// out before the first one is needed.  A segment's thread sums the ranks' vectors, adds the
// residual, stores the new residual, stores residual * gamma as the activation operand and the
// block leaves the segment's sum of squares in ss_part[row][seg].  1 / rms is applied to the
// product by the epilogue (it is a per-token scale), so no thread waits for a whole row here.
__device__ __forceinline__ bool dlin_gather_segments(const DlinParams& p, int et, size_t cur_off, float* s_part,
                                                     int* done_out) {
  using E = Elem<BL_DTYPE_BF16>;
  const Comm& c = p.c;
  const int vpr = p.k / 8;
  const int nseg = (vpr + 127) / 128;
  const int total = p.tokens * nseg;
  const char* inbox = c.base[c.rank] + cur_off;
  bool ok = true;
  int done = 0;
  const int nc = p.pro_ctas;  // only CTAs that are certainly resident together may be waited for
  for (int s0 = blockIdx.x; s0 < total && int(blockIdx.x) < nc; s0 += 2 * nc) {
    uint4 got[2][kMaxRanks];
    uint4 resv[2], gam[2];
    size_t g[2];
    bool act[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int sidx = s0 + u * nc;
      const int row = sidx / nseg, sg = sidx - row * nseg;
      const int i = sg * 128 + et;
      act[u] = sidx < total && i < vpr;
      g[u] = size_t(row) * vpr + i;
      if (act[u]) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < c.world) got[u][r] = ld_volatile_v4(inbox + size_t(r) * c.lamport_slice + g[u] * 16);
        if (p.res_in) resv[u] = __ldcg(p.res_in + g[u]);
        gam[u] = __ldg(p.gamma + i);
      }
    }
    float ss[2] = {0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (act[u]) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < c.world) {
            uint4 w = got[u][r];
            if (!landed(w) && !poll_vec(c, inbox + size_t(r) * c.lamport_slice + g[u] * 16, w, r)) ok = false;
            acc_add<BL_DTYPE_BF16>(acc, w);
          }
        uint4 packed = E::pack(acc);  // the all-reduce result in its storage type
        if (p.res_in) {
          E::unpack(packed, acc);
          acc_add<BL_DTYPE_BF16>(acc, resv[u]);
          packed = E::pack(acc);
        }
        p.res_out[g[u]] = packed;
        float x[8], gm[8];
        E::unpack(packed, x);
        E::unpack(gam[u], gm);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss[u] += x[j] * x[j];
          x[j] *= gm[j];
        }
        p.xnorm[g[u]] = E::pack(x);
      }
    }
    ss[0] = warp_sum(ss[0]);
    ss[1] = warp_sum(ss[1]);
    if ((et & 31) == 0) {
      s_part[et >> 5] = ss[0];
      s_part[4 + (et >> 5)] = ss[1];
    }
    bar_epi();
    if (et < 2) {
      const int sidx = s0 + et * nc;
      if (sidx < total) p.ss_part[sidx] = s_part[4 * et] + s_part[4 * et + 1] + s_part[4 * et + 2] + s_part[4 * et + 3];
    }
    bar_epi();  // s_part is reused by the next pair
    done += (s0 < total) + (s0 + nc < total);
  }
  *done_out = done;
  return ok;
}

template <int BN, int CPS>
__global__ void __launch_bounds__(kDlinThreads, CPS)
    k_dlin(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
           const __grid_constant__ DlinParams p) {
  using S = DlinSmem<BN, CPS>;
  extern __shared__ uint8_t smem_raw[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* empty_bar = full_bar + S::kStages;
  uint64_t* tfull_bar = empty_bar + S::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile uint32_t* s_abort = tmem_slot + 1;
  volatile uint32_t* s_late = tmem_slot + 2;  // a link wait ran out: results are not valid
  float* s_part = reinterpret_cast<float*>(tmem_slot + 4);
  const uint32_t ring = (smem_u32(smem_raw) + S::kBarBytes + 1023u) & ~1023u;
  const uint32_t xbuf = CPS == 2 ? ring : ring + S::kStages * S::kStageBytes;

  pdl_launch_dependents();
  unsigned long long* tr = p.trace ? p.trace + size_t(blockIdx.x) * 12 : nullptr;
  if (tr && threadIdx.x == 0) tr[0] = globaltimer_ns();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int CL = int(cluster_nctarank());
  const int q = int(cluster_ctarank());
  const int tile = blockIdx.x / CL;
  const int kb_per = (p.kblocks + CL - 1) / CL;
  const int kb0 = min(p.kblocks, q * kb_per);
  const int nkb = min(p.kblocks, kb0 + kb_per) - kb0;
  // columns (tokens) of the tile are dealt out to the CTAs of the cluster for the final sum
  const int ncol = p.tokens < BN ? p.tokens : BN;
  const int cpc = p.cpc, cpcp = p.cpcp;
  const int nseg_row = (p.k / 8 + 127) / 128;       // prologue: segments per row
  const int nseg_total = p.tokens * nseg_row;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *s_abort = 0;
    *s_late = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // every CTA of the cluster is running: its shared memory may be written
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (tr && threadIdx.x == 0) tr[1] = globaltimer_ns();

  if (warp == 0) {
    // ------------------------------ producer --------------------------------
    if (lane == 0) {
      // weights do not depend on earlier kernels: the first lap is requested at once
      const int pre = nkb < S::kStages ? nkb : S::kStages;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], S::kStageBytes);
        tma_load_2d_hint_s(ring + i * S::kStageBytes, &tmap_w, smem_u32(&full_bar[i]), (kb0 + i) * kTileK,
                           tile * kTileA, kHintEvictFirst);
      }
      pdl_wait();
      if (tr) tr[2] = globaltimer_ns();
      if (p.pro) {
        // rows of the activation operand are being written by the first CTAs of this grid
        const uint32_t want = *reinterpret_cast<volatile uint32_t*>(p.sync + 1) + uint32_t(nseg_total);
        const uint64_t t0 = globaltimer_ns();
        uint32_t polls = 0;
        while (int32_t(ld_acquire_gpu(p.sync) - want) < 0) {
          if ((++polls & 63u) == 0u && globaltimer_ns() - t0 > p.c.timeout_ns + 500000000ull) {
            *s_late = 1;  // give up waiting; the product is computed on whatever is there
            break;
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy writes, read next by TMA
      }
      if (tr) tr[3] = globaltimer_ns();
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i) {
        const uint32_t sa = ring + stage * S::kStageBytes;
        if (i >= pre) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, s_abort)) break;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          tma_load_2d_hint_s(sa, &tmap_w, smem_u32(&full_bar[stage]), (kb0 + i) * kTileK, tile * kTileA,
                             kHintEvictFirst);
        }
        tma_load_2d_hint_s(sa + S::kStageA, &tmap_x, smem_u32(&full_bar[stage]), (kb0 + i) * kTileK, 0,
                           kHintEvictLast);
        if (++stage == S::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && nkb > 0) {
      const uint32_t idesc = umma_idesc_f16(kTileA, BN, 1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, s_abort)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (tr && i == 0) tr[4] = globaltimer_ns();
        const uint32_t sa = ring + stage * S::kStageBytes;
        const uint64_t da = umma_desc_k_sw128(sa);
        const uint64_t db = umma_desc_k_sw128(sa + S::kStageA);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k)
          umma_f16_ss(tmem_base, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == S::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit(tfull_bar);
      if (tr) tr[5] = globaltimer_ns();
    }
  } else {
    // ---------------- prologue rows, then this CTA's partial tile -----------
    const int et = threadIdx.x - 64;
    const int q4 = warp & 3;  // TMEM lane quarter this warp may read
    const int row = q4 * 32 + lane;
    pdl_wait();
    if (p.pro) {
      const Comm& c = p.c;
      uint32_t* sg = sig_of(c, c.rank);
      const uint32_t e = ld_volatile_u32(&sg[sig_epoch(P_LAMPORT)]);
      const uint32_t prev_vecs = ld_volatile_u32(&sg[sig_aux(P_LAMPORT)]);
      const size_t cur_off = c.lamport_off + size_t(e % 3u) * (size_t(c.world) * c.lamport_slice);
      int done = 0;
      const bool ok = dlin_gather_segments(p, et, cur_off, s_part, &done);
      if (!ok) *s_late = 1;
      if (done > 0) {
        // the barrier orders the other threads' stores before thread 0's release (cumulativity)
        bar_epi();
        if (et == 0) red_release_gpu_add(p.sync, uint32_t(done));
      }
      dlin_clear_prev(c, e, prev_vecs, et);
      if (tr && et == 0) tr[6] = globaltimer_ns();
    }
    if (nkb > 0 && !mbar_wait_bounded(tfull_bar, 0, s_abort)) {
      // the accumulator never became ready: nothing valid to hand over
    }
    tc_fence_after_sync();
    if (tr && et == 0) tr[7] = globaltimer_ns();
  }

  if constexpr (CPS == 2) {
    // the exchange buffers live in the operand rings: every CTA of the cluster must be done
    // with its main loop before anyone stores into a ring
    __syncwarp();
    cluster_sync_all();
  }

  if (warp >= 2) {
    // partial accumulator -> the owners' exchange buffers: xbuf[src q][row][column], rows
    // `cpcp` floats apart (cpcp % 8 == 4: the 16-byte accesses below are conflict free).  Four
    // consecutive columns always belong to one owner (cpc is a multiple of 4).
    const int et = threadIdx.x - 64;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(q4 * 32) << 16);
    const bool have = nkb > 0 && !*s_abort;
    constexpr int kChunk = BN < 32 ? 16 : 32;
    const uint32_t my_row = uint32_t((q * kTileA + row) * cpcp * 4);
    int owner = 0, cc = 0;
    uint32_t obase = map_to_cta(xbuf, 0u) + my_row;
#pragma unroll 1
    for (int c0 = 0; c0 < ncol; c0 += kChunk) {
      uint32_t r[kChunk];
      if (have) {
        if constexpr (kChunk == 32) tmem_ld_32x32(taddr + c0, r);
        else tmem_ld_32x16(taddr + c0, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) r[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < kChunk; i += 4) {
        if (c0 + i < ncol) {
          st_cluster_v4(obase + uint32_t(cc * 4), r[i], r[i + 1], r[i + 2], r[i + 3]);
          cc += 4;
          if (cc == cpc) {
            cc = 0;
            ++owner;
            obase = map_to_cta(xbuf, uint32_t(owner < CL ? owner : 0)) + my_row;
          }
        }
      }
    }
    tc_fence_before_sync();
    if (tr && et == 0) tr[8] = globaltimer_ns();
  }

  // every partial of this cluster is in place (the roles above diverged inside their warps)
  __syncwarp();
  cluster_sync_all();
  if (tr && threadIdx.x == 64) tr[9] = globaltimer_ns();

  if (warp >= 2) {
    const int et = threadIdx.x - 64;
    const int col0 = q * cpc;
    const int mine = max(0, min(ncol, col0 + cpc) - col0);  // a multiple of 4 except at the end of the tile
    const int row = (warp & 3) * 32 + lane;  // same row as in the hand-over above
    const int feat = tile * kTileA + row;
    const bool nok = feat < p.n;
    const uint32_t xrow = xbuf + uint32_t(row * cpcp * 4);
    const uint32_t src_stride = uint32_t(kTileA * cpcp * 4);
    const float bv = (nok && p.bias && p.epi != 2) ? __bfloat162float(p.bias[feat]) : 0.f;
    // with the gather prologue the operand rows were residual * gamma: the missing 1 / rms of each
    // token scales that token's column of the product
    float* s_rstd = reinterpret_cast<float*>(smem_raw + 512);
    if (p.pro) {
      if (et < mine) {
        // the segment sums were stored before the segments were published: acquire that count
        const uint32_t want = *reinterpret_cast<volatile uint32_t*>(p.sync + 1) + uint32_t(nseg_total);
        for (uint32_t polls = 0; int32_t(ld_acquire_gpu(p.sync) - want) < 0 && polls < (1u << 22); ++polls) {
        }
        float sum = 0.f;
        for (int sg = 0; sg < nseg_row; ++sg) sum += __ldcg(p.ss_part + size_t(col0 + et) * nseg_row + sg);
        s_rstd[et] = rsqrtf(sum / float(p.k) + p.eps);
      }
      bar_epi();
    }
    // epi 2: the reduced tile goes through shared memory once more ([column][row] bf16, in the
    // operand ring, which nothing reads any more) so that it leaves as 16-byte vectors
    const uint32_t stg = ring + S::kStageTileOff;
    for (int cc = 0; cc < mine; cc += 4) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < CL; ++s) {
        float4 t;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w)
                     : "r"(xrow + uint32_t(s) * src_stride + uint32_t(cc * 4)));
        v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = v[j] * ((p.pro && cc + j < mine) ? s_rstd[cc + j] : 1.f) + bv;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = col0 + cc + j;
        if (p.epi == 1) {
          // even row = gate, odd row = up of output column feat / 2
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          if (cc + j < mine && nok && !(row & 1))
            p.out[size_t(m) * p.ldo + (feat >> 1)] = __float2bfloat16(v[j] / (1.f + __expf(-v[j])) * other);
        } else if (p.epi == 0) {
          if (cc + j < mine && nok) p.out[size_t(m) * p.ldo + feat] = __float2bfloat16(v[j]);
        } else {
          const __nv_bfloat16 h = __float2bfloat16(v[j]);
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(stg + uint32_t((cc + j) * (kTileA * 2) + row * 2)),
                       "h"(*reinterpret_cast<const unsigned short*>(&h))
                       : "memory");
        }
      }
    }
    if (p.epi == 2) {
      bar_epi();
      // 8 consecutive features of one token per item: one 16-byte store per rank
      const Comm& c = p.c;
      const uint32_t e = ld_volatile_u32(&sig_of(c, c.rank)[sig_epoch(P_LAMPORT)]);
      const size_t dst_off = c.lamport_off + size_t(e % 3u) * (size_t(c.world) * c.lamport_slice) +
                             size_t(c.rank) * c.lamport_slice;
      for (int item = et; item < mine * (kTileA / 8); item += 128) {
        const int cc = item / (kTileA / 8), f8 = item - cc * (kTileA / 8);
        const int f0 = tile * kTileA + f8 * 8;
        if (f0 + 8 <= p.n) {
          uint4 v;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(stg + uint32_t(cc * (kTileA * 2) + f8 * 16)));
          v = scrub(v);
          const size_t off = dst_off + (size_t(col0 + cc) * p.push_ld + f0) * 2;
#pragma unroll 1
          for (int k = 0; k < c.world; ++k) {
            int r = c.rank + k;
            if (r >= c.world) r -= c.world;
            st_v4(c.base[r] + off, v);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tr && threadIdx.x == 0) tr[10] = globaltimer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
  if (threadIdx.x == 0) {
    if ((*s_abort || *s_late) && p.err) *p.err = 1u;
    if (p.pro) {
      // the last CTA to leave records how many rows have been published in total
      __threadfence();
      const uint32_t t = atomicAdd(p.sync + 2, 1u);
      if (t == gridDim.x - 1) {
        p.sync[2] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.sync + 1) = p.sync[1] + uint32_t(nseg_total);
      }
    }
  }
  if (p.pro) {
    const uint32_t e = ld_volatile_u32(&sig_of(p.c, p.c.rank)[sig_epoch(P_LAMPORT)]);
    finish_epoch(p.c, P_LAMPORT, e, uint32_t(p.tokens) * uint32_t(p.k / 8), true);
  }
}

// The gather as a kernel of its own: all-reduce (second half) + residual + RMSNorm, one token row
// per block of 256 threads.  Small (no dynamic shared memory, few registers), so it becomes
// resident while the linear before it is still running and finishes shortly after the last
// partial row has landed.  Every load of a batch goes out before the first one is used.
constexpr int kGatherThreads = 256;
__global__ void __launch_bounds__(kGatherThreads, 2) k_gather_norm(const __grid_constant__ DlinParams p) {
  using E = Elem<BL_DTYPE_BF16>;
  __shared__ float s_part[kGatherThreads / 32];
  pdl_launch_dependents();
  const Comm& c = p.c;
  const int vpr = p.k / 8;
  const int t = threadIdx.x;
  pdl_wait();
  uint32_t* sg = sig_of(c, c.rank);
  const uint32_t e = ld_volatile_u32(&sg[sig_epoch(P_LAMPORT)]);
  const uint32_t prev_vecs = ld_volatile_u32(&sg[sig_aux(P_LAMPORT)]);
  const char* inbox = c.base[c.rank] + c.lamport_off + size_t(e % 3u) * (size_t(c.world) * c.lamport_slice);
  bool ok = true;
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x) {
    float ss = 0.f;
#pragma unroll
    for (int v0 = 0; v0 < 4; v0 += 2) {
      uint4 got[2][kMaxRanks], resv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = t + (v0 + u) * kGatherThreads;
        if (i < vpr) {
          const size_t g = size_t(row) * vpr + i;
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < c.world) got[u][r] = ld_volatile_v4(inbox + size_t(r) * c.lamport_slice + g * 16);
          if (p.res_in) resv[u] = __ldcg(p.res_in + g);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = t + (v0 + u) * kGatherThreads;
        if (i < vpr) {
          const size_t g = size_t(row) * vpr + i;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < c.world) {
              uint4 w = got[u][r];
              if (!landed(w) && !poll_vec(c, inbox + size_t(r) * c.lamport_slice + g * 16, w, r)) ok = false;
              acc_add<BL_DTYPE_BF16>(acc, w);
            }
          uint4 packed = E::pack(acc);  // the all-reduce result in its storage type
          if (p.res_in) {
            E::unpack(packed, acc);
            acc_add<BL_DTYPE_BF16>(acc, resv[u]);
            packed = E::pack(acc);
          }
          p.res_out[g] = packed;
          float x[8];
          E::unpack(packed, x);  // the norm sees the rounded residual
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
        }
      }
    }
    ss = warp_sum(ss);
    if ((t & 31) == 0) s_part[t >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kGatherThreads / 32; ++w) tot += s_part[w];
    const float rstd = rsqrtf(tot / float(p.k) + p.eps);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int i = t + v * kGatherThreads;
      if (i < vpr) {
        // this thread's own store of a moment ago (kept out of registers: the kernel stays small
        // enough to share an SM with the linears around it)
        float gm[8], o[8], x[8];
        E::unpack(__ldcg(p.res_out + size_t(row) * vpr + i), x);
        E::unpack(__ldg(p.gamma + i), gm);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = x[j] * rstd;
        // x * rstd is rounded to bf16 before the weight multiply, as a framework RMSNorm module does
        uint4 tt = E::pack(o);
        E::unpack(tt, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= gm[j];
        p.xnorm[size_t(row) * vpr + i] = E::pack(o);
      }
    }
    __syncthreads();  // s_part is reused by the next row
  }
  if (!ok && p.err && t == 0) *p.err = 1u;
  // reset the inbox buffer of the call before this one (written again two calls from now)
  {
    const size_t clr_off = c.lamport_off + size_t((e + 2u) % 3u) * (size_t(c.world) * c.lamport_slice);
    const uint4 unw = make_uint4(kUnwritten, kUnwritten, kUnwritten, kUnwritten);
    for (size_t i = size_t(blockIdx.x) * kGatherThreads + t; i < prev_vecs; i += size_t(gridDim.x) * kGatherThreads)
      for (int r = 0; r < c.world; ++r) st_v4(c.base[c.rank] + clr_off + size_t(r) * c.lamport_slice + i * 16, unw);
  }
  finish_epoch(c, P_LAMPORT, e, uint32_t(p.tokens) * uint32_t(p.k / 8), true);
}

// One-rank stand-in for the link in ordinary device memory: three inbox buffers of one
// slice each, then a small signal pad.  Lets a single GPU run the same kernels.
static Comm local_comm(void* buf, size_t slice) {
  Comm c;
  memset(&c, 0, sizeof(c));
  c.rank = 0;
  c.world = 1;
  c.base[0] = static_cast<char*>(buf);
  c.lamport_off = 0;
  c.lamport_slice = slice;
  c.sig_off = 3 * slice;
  c.timeout_ns = 2000000000ull;
  c.status = nullptr;
  return c;
}

__global__ void k_dlin_fill(uint32_t* p, size_t n_unwritten, size_t n_zero) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_unwritten + n_zero;
       i += size_t(gridDim.x) * blockDim.x)
    p[i] = i < n_unwritten ? kUnwritten : 0u;
}

// How many clusters of `cl` CTAs of k_dlin<BN> the GPU holds at once (one CTA per SM; a cluster
// must fit inside one GPC, so this is less than SMs / cl for some sizes).  Asked once per shape.
template <int BN, int CPS>
static int max_active_clusters(int cl) {
  static int cache[kDlinMaxCluster + 1] = {0};
  if (cl < 1 || cl > kDlinMaxCluster) return 1;
  if (cache[cl] > 0) return cache[cl];
  using S = DlinSmem<BN, CPS>;
  int n = 0;
  cudaFuncSetAttribute(k_dlin<BN, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(cl * sm_count()));
  cfg.blockDim = dim3(kDlinThreads);
  cfg.dynamicSmemBytes = S::kBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(cl);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaOccupancyMaxActiveClusters(&n, k_dlin<BN, CPS>, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = CPS * sm_count() / cl;
  }
  cache[cl] = n > 0 ? n : 1;
  return cache[cl];
}
// One CTA per SM with the deep ring is the default: on a TP=8 shard of the 7B shape it measured
// 2.12 ms per decode step against 2.39 with two CTAs per SM (BL_DLIN_CPS=2).
static int dlin_cps() {
  static const int v = [] {
    const char* e = getenv("BL_DLIN_CPS");
    return (e && e[0] == '2') ? 2 : 1;
  }();
  return v;
}
static int max_active_clusters_bn(int bn, int cl) {
  if (dlin_cps() == 2)
    return bn <= 16 ? max_active_clusters<16, 2>(cl) : bn <= 32 ? max_active_clusters<32, 2>(cl)
                                                                 : max_active_clusters<64, 2>(cl);
  return bn <= 16 ? max_active_clusters<16, 1>(cl) : bn <= 32 ? max_active_clusters<32, 1>(cl)
                                                               : max_active_clusters<64, 1>(cl);
}

// columns per CTA (a multiple of 4) and the row pitch of the exchange buffer (== 4 mod 8 floats)
static void cluster_columns(int ncol, int cl, int* cpc, int* cpcp) {
  int c = (ncol + cl - 1) / cl;
  c = (c + 3) / 4 * 4;
  int pp = c;
  while (pp % 8 != 4) ++pp;
  *cpc = c;
  *cpcp = pp;
}
static bool cluster_fits(int bn, int ncol, int cl) {
  int cpc, cpcp;
  cluster_columns(ncol, cl, &cpc, &cpcp);
  const int xbuf = bn >= 64 ? DlinSmem<64, 1>::kXbufBytes : DlinSmem<32, 1>::kXbufBytes;
  return cl * kTileA * cpcp * 4 <= xbuf;
}

// Cluster size for `tiles` weight tiles of `kblocks` k-blocks: the one with the shortest estimated
// time, waves x (fixed cost + k-blocks per CTA x cost per k-block) + a term for the exchange; the
// constants are the measured ones of this kernel on a B200 (5.5 us, 0.27 us, 0.15 us per CTA).
static int pick_cluster(int tiles, int kblocks, int want, int bn, int ncol) {
  static const int cap = [] {
    const char* v = getenv("BL_DLIN_CL");  // tuning: upper bound of the automatic choice
    return (v && *v) ? atoi(v) : 0;
  }();
  int hi = kDlinMaxCluster;
  if (hi > kblocks) hi = kblocks;
  if (hi < 1) hi = 1;
  if (want > 0) {
    int cl = want < hi ? want : hi;
    while (cl > 1 && !cluster_fits(bn, ncol, cl)) --cl;
    return cl;
  }
  if (cap > 0 && hi > cap) hi = cap;
  int best = 1;
  float best_t = 1e30f;
  for (int cl = 1; cl <= hi; ++cl) {
    if (!cluster_fits(bn, ncol, cl)) continue;
    if (cl > 1 && kblocks / cl < 2) continue;  // at least two k-blocks per CTA
    const int act = max_active_clusters_bn(bn, cl);
    const int waves = (tiles + act - 1) / act;
    // CTAs that share an SM share its load bandwidth; a larger cluster has more partials to sum
    const int ctas = tiles * cl < act * cl ? tiles * cl : act * cl;
    const float share = ctas > sm_count() ? float(ctas) / float(sm_count()) : 1.f;
    const float t = float(waves) * (5.5f + 0.27f * share * float((kblocks + cl - 1) / cl)) + 0.15f * float(cl);
    if (t < best_t - 1e-3f) {
      best_t = t;
      best = cl;
    }
  }
  return best;
}

template <int BN, int CPS>
static int launch_dlin(const CUtensorMap& tw, const CUtensorMap& tx, const DlinParams& p, int tiles, int cl,
                       cudaStream_t st, char* err, size_t errlen) {
  using S = DlinSmem<BN, CPS>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(k_dlin<BN, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes, cudaGetErrorString(e));
      return -1;
    }
    attr_set = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(tiles * cl));
  cfg.blockDim = dim3(kDlinThreads);
  cfg.dynamicSmemBytes = S::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(cl);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k_dlin<BN, CPS>, tw, tx, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: decode linear launch failed (grid %d, cluster %d): %s", tiles * cl, cl,
            cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace bl

using namespace bl;

extern "C" size_t bl_dlin_local_link_bytes(int tokens, int hidden) {
  const size_t slice = ((size_t(tokens) * hidden * 2 + 4095) / 4096) * 4096;
  return 3 * slice + 4096;
}

extern "C" int bl_dlin_local_link_init(void* buf, int tokens, int hidden, void* stream, char* err, size_t errlen) {
  if (!buf || (reinterpret_cast<uintptr_t>(buf) & 15u)) {
    set_err(err, errlen, "barlink: the local link buffer must be 16-byte aligned");
    return -1;
  }
  const size_t slice = (bl_dlin_local_link_bytes(tokens, hidden) - 4096) / 3;
  k_dlin_fill<<<256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(buf), 3 * slice / 4, 1024);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: local link init failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

static int dlin_comm(blCtx* ctx, const blDlinArgs* a, Comm* out, char* err, size_t errlen) {
  const size_t need = size_t(a->tokens) * size_t(a->hidden) * 2;
  if (a->local_link) {
    const size_t slice = (bl_dlin_local_link_bytes(a->tokens, a->hidden) - 4096) / 3;
    *out = local_comm(a->local_link, slice);
    return 0;
  }
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: a decode linear with a collective needs the link (init_peer) or a local link buffer");
    return -1;
  }
  if (need > ctx->layout.lamport_slice) {
    set_err(err, errlen, "barlink: %d tokens x %d features exceed the %zu B one-shot inbox slice", a->tokens, a->hidden,
            ctx->layout.lamport_slice);
    return -1;
  }
  *out = ctx->comm_for(ctx->rank);
  return 0;
}

static int dlin_fill_pro(const blDlinArgs* a, DlinParams* p, char* err, size_t errlen) {
  if (!a->residual_out || !a->gamma || !a->x || a->hidden < 8 || (a->hidden & 7) ||
      a->hidden / 8 > 128 * kDlinMaxVpt) {
    set_err(err, errlen, "barlink: the fused all-reduce + norm needs residual_out, gamma, x and hidden %% 8 == 0, hidden <= %d",
            128 * kDlinMaxVpt * 8);
    return -1;
  }
  p->res_in = static_cast<const uint4*>(a->residual_in);
  p->res_out = static_cast<uint4*>(a->residual_out);
  p->gamma = static_cast<const uint4*>(a->gamma);
  p->xnorm = static_cast<uint4*>(const_cast<void*>(a->x));
  p->eps = a->eps;
  return 0;
}

extern "C" int bl_gather_norm(blCtx* ctx, const blDlinArgs* a, void* stream, char* err, size_t errlen) {
  if (!a || a->tokens < 1) {
    set_err(err, errlen, "barlink: gather_norm needs at least one token");
    return -1;
  }
  DlinParams p;
  memset(&p, 0, sizeof(p));
  p.k = a->hidden;
  p.tokens = a->tokens;
  p.err = static_cast<uint32_t*>(a->err_flag);
  if (dlin_fill_pro(a, &p, err, errlen) != 0) return -1;
  if (dlin_comm(ctx, a, &p.c, err, errlen) != 0) return -1;
  const int grid = a->tokens < 2 * sm_count() ? a->tokens : 2 * sm_count();
  cudaError_t e = launch_k(k_gather_norm, dim3(grid), dim3(kGatherThreads), 0, static_cast<cudaStream_t>(stream), p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: gather_norm launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

extern "C" int bl_dlin_cluster(int n, int k, int tokens, int want) {
  const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64;
  return pick_cluster((n + kTileA - 1) / kTileA, (k + kTileK - 1) / kTileK, want, bn, tokens < bn ? tokens : bn);
}

extern "C" int bl_dlin(blCtx* ctx, const blDlinArgs* a, void* stream, char* err, size_t errlen) {
  if (!a || !a->w || !a->x || a->n < 1 || a->k < 8 || (a->k & 7) || a->tokens < 1 || a->tokens > 64) {
    set_err(err, errlen, "barlink: decode linear needs w, x, K a multiple of 8 and 1..64 tokens");
    return -1;
  }
  if (a->pro < 0 || a->pro > 1 || a->epi < 0 || a->epi > 2 || (a->pro == 1 && a->epi == 2)) {
    set_err(err, errlen, "barlink: decode linear: prologue %d / epilogue %d is not a supported pair", a->pro, a->epi);
    return -1;
  }
  DlinParams p;
  memset(&p, 0, sizeof(p));
  p.n = a->n;
  p.k = a->k;
  p.tokens = a->tokens;
  p.kblocks = (a->k + kTileK - 1) / kTileK;
  p.pro = a->pro;
  p.epi = a->epi;
  p.err = static_cast<uint32_t*>(a->err_flag);
  p.trace = static_cast<unsigned long long*>(a->trace);
  if (a->pro == 1) {
    if (a->hidden != a->k || !a->sync) {
      set_err(err, errlen, "barlink: with the fused all-reduce + norm, K must be the hidden size and sync must be set");
      return -1;
    }
    if (dlin_fill_pro(a, &p, err, errlen) != 0) return -1;
    p.sync = static_cast<uint32_t*>(a->sync);
    // the segment sums live behind the three counters: 64 tokens x at most 8 segments
    p.ss_part = reinterpret_cast<float*>(static_cast<uint32_t*>(a->sync) + 16);
  }
  if (a->epi == 2) {
    if (a->hidden < a->n || (a->hidden & 7) || (a->n & 7)) {
      set_err(err, errlen, "barlink: the pushed rows need n <= hidden and both multiples of 8");
      return -1;
    }
    p.push_ld = a->hidden;
  } else {
    if (!a->out || (a->epi == 1 && (a->n & 1))) {
      set_err(err, errlen, "barlink: decode linear needs an output (and an even n for SiLU*mul)");
      return -1;
    }
    p.out = static_cast<__nv_bfloat16*>(a->out);
    p.ldo = a->ldo;
    p.bias = static_cast<const __nv_bfloat16*>(a->bias);
  }
  if ((a->pro == 1 || a->epi == 2) && dlin_comm(ctx, a, &p.c, err, errlen) != 0) return -1;
  const int bn = a->tokens <= 16 ? 16 : a->tokens <= 32 ? 32 : 64;
  const int tiles = (a->n + kTileA - 1) / kTileA;
  const int cl = pick_cluster(tiles, p.kblocks, a->cluster, bn, a->tokens < bn ? a->tokens : bn);
  cluster_columns(a->tokens < bn ? a->tokens : bn, cl, &p.cpc, &p.cpcp);
  {
    const int resident = max_active_clusters_bn(bn, cl) * cl;
    p.pro_ctas = tiles * cl < resident ? tiles * cl : resident;
  }
  CUtensorMap tw, tx;
  if (make_tmap_kmajor(a->w, a->n, a->k, a->ldw, kTileA, 2, &tw, err, errlen) != 0) return -1;
  if (make_tmap_kmajor(a->x, a->tokens, a->k, a->ldx, bn, 2, &tx, err, errlen) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dlin_cps() == 2) {
    switch (bn) {
      case 16: return launch_dlin<16, 2>(tw, tx, p, tiles, cl, st, err, errlen);
      case 32: return launch_dlin<32, 2>(tw, tx, p, tiles, cl, st, err, errlen);
      default: return launch_dlin<64, 2>(tw, tx, p, tiles, cl, st, err, errlen);
    }
  }
  switch (bn) {
    case 16: return launch_dlin<16, 1>(tw, tx, p, tiles, cl, st, err, errlen);
    case 32: return launch_dlin<32, 1>(tw, tx, p, tiles, cl, st, err, errlen);
    default: return launch_dlin<64, 1>(tw, tx, p, tiles, cl, st, err, errlen);
  }
}
