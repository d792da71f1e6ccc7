// SPDX-License-Identifier: MIT
//
// tcgen05 GEMM core for sm_100a:  D[i, j] = sum_k A[i, k] * B[j, k]
// with A [ra x K] and B [rb x K] both K-major bf16/fp16 in global memory.
//
//   warp 0      TMA producer: 128x64 tile of A and BNx64 tile of B per stage
//               (128-byte swizzle), ring of kStages shared-memory stages
//   warp 1      allocates TMEM, one elected lane issues tcgen05.mma
//               (M=128, N=BN, K=16, fp32 accumulate in TMEM), commits stage
//               release and accumulator-ready barriers
//   warps 2..5  epilogue: tcgen05.ld the accumulator (lane = row of A),
//               hand 32-column chunks to a Sink
// Two accumulators (2*BN TMEM columns) let the epilogue of one tile overlap
// the main loop of the next; the kernel is persistent over work units
// (tile_a, tile_b, k-split).  With k-splits, partial tiles go through an fp32
// workspace and the CTA that arrives last for a tile reduces them in split
// order (deterministic) and runs the Sink.
//
// The same core serves decode ("swap" orientation: A = weight rows, B = the
// few tokens, BN = 16..64) and prefill (A = tokens, B = weight rows, BN = 256)
// and the fused GEMM+collective kernels, which differ only in their Sink.
//
// The reference has no tensor-core GEMM of its own: its linears are cuBLAS
// F.linear / torch._int_mm calls (demos/qwen_tp/qwen38_int8/worker.py:84-93,
// 224); this file is what replaces those library calls on the hot path.
#pragma once

#include <cuda.h>

#include "ptx.cuh"

namespace bl {

constexpr int kGemmThreads = 192;
constexpr int kTileA = 128;
constexpr int kTileK = 64;

struct GemmShape {
  int ra, rb, k;            // rows of A, rows of B, reduction length
  int tiles_a, tiles_b;     // ceil(ra/128), ceil(rb/BN)
  int kblocks;              // ceil(k/64)
  int splits;               // k-splits per tile
  int ab_fmt;               // 1 = bf16, 0 = fp16
  int i8;                   // 1: both operands are signed 8-bit, a k-block is 128 elements, int32 accumulators;
                            // 2: the same with one weight scale per (A row, k-group): every k-block is multiplied
                            //    into an accumulator of its own (the two TMEM buffers alternate) and the epilogue
                            //    warps add acc * scale into fp32 registers, k-block by k-block (BN <= 64, no k-split)
  const __nv_bfloat16* gscale_bf;  // i8 == 2: [ra][gs_groups], gs_kblocks k-blocks of 128 per group
  int direct;               // 1: every k-split hands its raw partial tile to the Sink (no in-kernel reduce)
  int weights_in_a;         // operand that no earlier kernel writes: 1 = A, 0 = B, 2 = neither
  float* ws;                // [tiles*splits][BN][128] fp32 partials (splits > 1)
  uint32_t* counters;       // [tiles] arrival counters, zero between launches
  uint32_t* err;            // set to 1 when a wait inside the kernel ran out
  unsigned long long* trace; // debug: 8 global-timer stamps per CTA, or nullptr
  // Pre-tiled weights: the weight matrix is stored as [row block of 128][k block of 64]
  // tiles of 16 KiB, each already in the swizzled shared-memory image, so a tile is
  // ONE bulk copy instead of 128 row requests.  0 = none, 1 = operand A, 2 = operand B.
  int tiled;
  const uint8_t* tiled_base;
  int tiled_kblocks;        // k blocks per row block in the tiled matrix
  // All-gather fused in front of the GEMM: the activation operand lives in this
  // rank's arena and peers store their rows into it.  Before the first
  // activation tile is requested, each of gate_n flag words must have reached
  // *gate_cum + gate_add (peers add 1 per finished row block with a release at
  // system scope); the last CTA to finish moves *gate_cum forward.
  // W8 only: per-(row, k-group) scales relative to the row's largest one, fp16 [ra][gs_groups],
  // applied while widening (the row's largest scale is applied by the epilogue); null = none
  const __half* gscale;
  int gs_groups;
  int gs_kblocks;           // k-blocks of 64 per scale group (group size / 64)
  const uint32_t* gate_flags;
  uint32_t* gate_cum;
  uint32_t* gate_ticket;
  uint32_t gate_add;
  int gate_n;
  unsigned long long gate_timeout_ns;
  // paired-CTA kernel: walk order of the output tiles (see pair_tile_of)
  int band, band_m;
};

// W8: the A operand (weight rows) is int8 in global memory; its 128x64-byte raw
// tile lands in a third region of the stage and eight extra warps (two groups that
// take alternate k-blocks) widen it to bf16 into a swizzled A tile before the MMA
// warp may use it.
template <int BN, int CPS = 1, bool W8 = false>
struct GemmSmem {
  static constexpr int kStageA = kTileA * kTileK * 2;
  static constexpr int kStageB = BN * kTileK * 2;  // one k-block of the B operand
  // W8, narrow tiles: a stage holds TWO k-blocks.  The raw int8 A tile is then 128 rows of 128
  // bytes (one request per row and per 128-byte line instead of two of 64 bytes): the number of
  // row requests per k-block, which bounds these weight-streaming shapes, drops by a third to a
  // half.
  static constexpr int kKS = (W8 && BN <= 64) ? 2 : 1;
  static constexpr int kStageRaw = W8 ? kTileA * kTileK * kKS : 0;
  // bf16: a stage is [A 16 KiB][B]; W8: a stage is [B of each k-block][raw int8 A] and the
  // widened A tiles live in a short ring of their own behind the stages, so
  // that many raw stages (= bytes in flight from HBM) fit
  static constexpr int kStageBytes = W8 ? kKS * kStageB + kStageRaw : kStageA + kStageB;
  static constexpr int kOffB = W8 ? 0 : kStageA;
  static constexpr int kOffRaw = kKS * kStageB;
  static constexpr int kA16Stages = W8 ? (BN <= 64 ? 4 : 3) : 0;
  static constexpr int kTxBytes = kStageBytes;  // bytes TMA delivers per full stage
  static constexpr int kConvThreads = W8 ? 256 : 0;
  static constexpr int kThreads = kGemmThreads + kConvThreads;
  // narrow tiles (decode): 4 stages so that two CTAs share an SM -- the same
  // bytes in flight per SM, but a CTA of the next kernel can move in and
  // prefetch weights while one of this kernel is still in its epilogue
  static constexpr int kStages = W8 ? (BN <= 16 ? 8 : BN <= 32 ? 6 : BN <= 64 ? 5 : BN <= 128 ? 7 : 4)
                                    : (CPS == 2) ? 4 : (BN <= 64 ? 8 : (BN <= 128 ? 6 : 4));
  static constexpr int kCtasPerSm = CPS;
  static constexpr int kBarBytes = 1024;
  // + 1024 so that the tile ring can be aligned to the swizzle atom
  static constexpr int kBytes = kStages * kStageBytes + kA16Stages * kStageA + kBarBytes + 1024;
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static_assert(kBytes <= 232448, "stage ring does not fit the shared memory of one CTA");
  static_assert(kStageBytes % 1024 == 0 && kOffRaw % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

// Sink concept:
//   __device__ void operator()(int tile_a, int tile_b, int split, int row_in_tile, int col0,
//                              const float (&v)[32], int ncols) const;
// called by each of the 128 epilogue threads (row_in_tile = TMEM lane) once per
// 32-column chunk of a finished tile; all 32 threads of a warp call it together.

// four int8 in one word -> two bf16x2 words, exactly (|v| <= 128 fits bf16's 8 bits)
__device__ __forceinline__ void s8x4_to_bf16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;  // biased to 0..255
  const float bias = 8388608.f + 128.f;
  const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - bias;
  const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - bias;
  const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - bias;
  const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - bias;
  lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
  hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

// four int8 in one word times a scale -> two bf16x2 words (round to nearest).  The scale rides
// on the subtraction that removes the conversion bias, so it costs no instruction: with
// scale = 1 the result is the exact integer.
__device__ __forceinline__ void s8x4_to_bf16x4_scaled(uint32_t w, float sc, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;  // biased to 0..255
  const float nb = -(8388608.f + 128.f) * sc;
  const float f0 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)), sc, nb);
  const float f1 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)), sc, nb);
  const float f2 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)), sc, nb);
  const float f3 = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)), sc, nb);
  lo = pack_bf16x2(f0, f1);
  hi = pack_bf16x2(f2, f3);
}

// an accumulator word as fp32: the bits of a float, or (int8 products) an int32 to convert
__device__ __forceinline__ float acc_f32(uint32_t bits, bool i8) {
  return i8 ? float(int32_t(bits)) : __uint_as_float(bits);
}

// MODE = GemmShape::i8 (0 bf16/fp16 operands, 1 int8 operands, 2 int8 with per-group weight scales) is a
// compile-time switch: with the int8 branches taken at run time the bf16 decode GEMMs measured 20-45 % slower
// (gate/up at 64 tokens 64-73 us instead of 51-53), so each mode is a kernel of its own.
template <int BN, int CPS, bool W8, int MODE = 0, class Sink>
__device__ __forceinline__ void gemm_body(const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                                          const GemmShape& g, const Sink& sink, uint64_t hint_a,
                                          uint64_t hint_b) {
  using S = GemmSmem<BN, CPS, W8>;
  extern __shared__ uint8_t smem_raw[];
  // barriers first, then the 1024-aligned stage ring
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* empty_bar = full_bar + S::kStages;
  uint64_t* tfull_bar = empty_bar + S::kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* ready_bar = tempty_bar + 2;  // W8: a widened A tile is ready / free again
  uint64_t* afree_bar = ready_bar + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(afree_bar + 4);
  volatile uint32_t* s_abort = tmem_slot + 1;
  uint32_t* s_last = tmem_slot + 2;
  const uint32_t ring = (smem_u32(smem_raw) + S::kBarBytes + 1023u) & ~1023u;

  // the next kernel of the stream may start its own preamble from here on
  pdl_launch_dependents();
  unsigned long long* tr = g.trace ? g.trace + size_t(blockIdx.x) * 8 : nullptr;
  if (tr && threadIdx.x == 0) tr[0] = globaltimer_ns();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles = g.tiles_a * g.tiles_b;
  const int units = tiles * g.splits;
  const int kb_per = (g.kblocks + g.splits - 1) / g.splits;

  // operand loads of one stage: 2-D tensor copies, or bulk copies of pre-tiled weights
  auto load_a = [&](uint32_t dst, uint32_t bar, int kb, int ta) {
    if (!W8 && g.tiled == 1)
      bulk_load_s(dst, g.tiled_base + (size_t(ta) * g.tiled_kblocks + kb) * S::kStageA, S::kStageA, bar,
                  hint_a);
    else
      tma_load_2d_hint_s(dst, tmap_a, bar, kb * (MODE ? 2 * kTileK : kTileK), ta * kTileA, hint_a);
  };
  auto load_b = [&](uint32_t dst, uint32_t bar, int kb, int tb) {
    if (!W8 && g.tiled == 2) {
      if constexpr (BN <= kTileA) {
        const int r0 = tb * BN;
        bulk_load_s(dst,
                    g.tiled_base + (size_t(r0 / kTileA) * g.tiled_kblocks + kb) * S::kStageA +
                        size_t(r0 % kTileA) * 128,
                    BN * 128, bar, hint_b);
      } else {
#pragma unroll
        for (int h = 0; h < BN / kTileA; ++h)
          bulk_load_s(dst + h * S::kStageA,
                      g.tiled_base + (size_t(tb * (BN / kTileA) + h) * g.tiled_kblocks + kb) * S::kStageA,
                      S::kStageA, bar, hint_b);
      }
    } else {
      tma_load_2d_hint_s(dst, tmap_b, bar, kb * (MODE ? 2 * kTileK : kTileK), tb * BN, hint_b);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&ready_bar[s], S::kConvThreads > 0 ? S::kConvThreads / 64 : 1);  // one lane of each warp of a widening group  // one group of widening threads per k-block
      mbar_init(&afree_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 128);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(tmap_a);
    tma_prefetch_desc(tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (tr && threadIdx.x == 0) tr[1] = globaltimer_ns();

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      // Weights do not depend on the kernels before this one: the first lap
      // of weight tiles is requested before waiting for them, so HBM keeps
      // streaming across the kernel boundary.  Activation tiles follow once
      // the predecessors have completed.
      int pre = 0;
      for (int u = blockIdx.x; g.weights_in_a != 2 && u < units && pre < S::kStages; u += gridDim.x) {
        const int tile = u / g.splits, sp = u - tile * g.splits;
        const int ta = tile / g.tiles_b, tb = tile - ta * g.tiles_b;
        const int kb0 = sp * kb_per;
        const int kb1 = min(g.kblocks, kb0 + kb_per);
        for (int kb = kb0; kb < kb1 && pre < S::kStages; kb += S::kKS, ++pre) {
          const int nsub = S::kKS == 1 ? 1 : min(S::kKS, kb1 - kb);  // k-blocks in this stage
          mbar_expect_tx(&full_bar[pre], S::kTxBytes - (S::kKS - nsub) * S::kStageB);
          const uint32_t sa = ring + pre * S::kStageBytes;
          if (g.weights_in_a)
            load_a(sa + (W8 ? S::kOffRaw : 0), smem_u32(&full_bar[pre]), kb, ta);
          else
            load_b(sa + S::kOffB, smem_u32(&full_bar[pre]), kb, tb);
        }
      }
      pdl_wait();
      if (tr) tr[2] = globaltimer_ns();
      if (g.gate_flags) {
        const uint32_t want = *reinterpret_cast<volatile uint32_t*>(g.gate_cum) + g.gate_add;
        const uint64_t t0 = globaltimer_ns();
        for (int f = 0; f < g.gate_n; ++f) {
          uint32_t polls = 0;
          while (int32_t(ld_acquire_sys(g.gate_flags + f) - want) < 0) {
            if ((++polls & 63u) == 0u && globaltimer_ns() - t0 > g.gate_timeout_ns) {
              *s_abort = 1;  // peers never delivered their rows: give up, nothing was requested yet
              break;
            }
          }
          if (*s_abort) break;
        }
        // the rows were written by other GPUs and are read next by the TMA unit
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      int stage = 0;
      uint32_t phase = 0;
      int armed = 0;
      bool ok = !*s_abort;
      if (!ok && pre > 0) {
        // weight tiles of the first lap are in flight with half of their bytes
        // expected: complete the stages with the activation tiles anyway so
        // that the copies land before the CTA leaves
        ok = true;
      }
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int tile = u / g.splits, sp = u - tile * g.splits;
        const int ta = tile / g.tiles_b, tb = tile - ta * g.tiles_b;
        const int kb0 = sp * kb_per;
        const int kb1 = min(g.kblocks, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; kb += S::kKS) {
          if (*s_abort && armed >= pre) {
            ok = false;
            break;
          }
          const int nsub = S::kKS == 1 ? 1 : min(S::kKS, kb1 - kb);
          const uint32_t sa = ring + stage * S::kStageBytes;
          const bool early = armed < pre;  // weight tile of this stage is already on its way
          if (!early) {
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, s_abort)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&full_bar[stage], S::kTxBytes - (S::kKS - nsub) * S::kStageB);
          }
          if (!early || !g.weights_in_a)
            load_a(sa + (W8 ? S::kOffRaw : 0), smem_u32(&full_bar[stage]), kb, ta);
          if (!early || g.weights_in_a) {
#pragma unroll
            for (int sb = 0; sb < S::kKS; ++sb)
              if (sb < nsub) load_b(sa + S::kOffB + sb * S::kStageB, smem_u32(&full_bar[stage]), kb + sb, tb);
          }
          ++armed;
          if (++stage == S::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Let copies that are still in flight land before the CTA goes away:
        // the stages armed in the last lap complete their full barriers.
        int n = armed < S::kStages ? armed : S::kStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < n; ++i) {
          if (--s < 0) {
            s = S::kStages - 1;
            ph ^= 1u;
          }
          for (uint32_t p = 0; p < (1u << 20); ++p)
            if (mbar_try_wait(&full_bar[s], ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------
    if (lane == 0) {
      const uint32_t idesc = MODE ? umma_idesc_i8(kTileA, BN) : umma_idesc_f16(kTileA, BN, g.ab_fmt);
      int stage = 0, astage = 0;
      uint32_t phase = 0, aphase = 0;
      uint32_t tphase[2] = {0, 0};
      int it = 0;
      int gcount = 0;  // grouped int8: k-blocks issued so far (selects the accumulator buffer)
      constexpr bool grouped = MODE == 2;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++it) {
        const int tile = u / g.splits, sp = u - tile * g.splits;
        const int kb0 = sp * kb_per;
        const int kb1 = min(g.kblocks, kb0 + kb_per);
        int acc = it & 1;
        if (!grouped) {
          if (!mbar_wait_bounded(&tempty_bar[acc], tphase[acc] ^ 1u, s_abort)) break;
          tphase[acc] ^= 1u;
          tc_fence_after_sync();
        }
        uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = kb0; kb < kb1 && ok; kb += S::kKS) {
          const int nsub = S::kKS == 1 ? 1 : min(S::kKS, kb1 - kb);
          const uint32_t sa = ring + stage * S::kStageBytes;
          if (!W8 && !mbar_wait_bounded(&full_bar[stage], phase, s_abort)) {
            ok = false;
            break;
          }
          if (grouped) {
            // an accumulator per k-block: wait until the epilogue warps have drained this buffer
            acc = gcount & 1;
            if (!mbar_wait_bounded(&tempty_bar[acc], tphase[acc] ^ 1u, s_abort)) {
              ok = false;
              break;
            }
            tphase[acc] ^= 1u;
            tc_fence_after_sync();
            d_tmem = tmem_base + uint32_t(acc * BN);
          }
#pragma unroll
          for (int sb = 0; sb < S::kKS; ++sb) {
            if (sb >= nsub) break;
            // W8: the widening threads have waited for the stage; the widened tile is what counts
            if (W8 && !mbar_wait_bounded(&ready_bar[astage], aphase, s_abort)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (tr && kb == kb0 && sb == 0 && it == 0) tr[3] = globaltimer_ns();
            const uint64_t da =
                umma_desc_k_sw128(W8 ? ring + S::kStages * S::kStageBytes + astage * S::kStageA : sa);
            const uint64_t db = umma_desc_k_sw128(sa + S::kOffB + sb * S::kStageB);
#pragma unroll
            for (int k = 0; k < kTileK / 16; ++k) {
              // +32 bytes along K inside the swizzle atom = +2 in the address field
              if constexpr (MODE != 0)
                umma_i8_ss(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc,
                           ((!grouped && kb + sb > kb0) || k > 0) ? 1u : 0u);
              else
                umma_f16_ss(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc,
                            (kb + sb > kb0 || k > 0) ? 1u : 0u);
            }
            if (W8) {
              umma_commit(&afree_bar[astage]);
              if (++astage == S::kA16Stages) {
                astage = 0;
                aphase ^= 1u;
              }
            }
          }
          if (!ok) break;
          umma_commit(&empty_bar[stage]);
          if (grouped) {
            umma_commit(&tfull_bar[acc]);
            ++gcount;
          }
          if (++stage == S::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && !grouped) umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (W8 && warp >= 6) {
    // ------------------------ int8 -> bf16 widening -----------------------
    // Two groups of 128 threads take alternate stages, so that the load -> convert -> store ->
    // proxy fence chain of one stage overlaps the next one's.  A thread widens one whole tile
    // row per k-block: 64 int8 in (four 16-byte loads issued together), eight swizzled 16-byte
    // chunks of bf16 out; one warp lane per warp then reports the tile.  Bank conflicts: with two
    // k-blocks per stage the raw tile has 128-byte rows in the 128-byte swizzle, so the eight
    // rows of a quarter warp find the same logical chunk in eight different banks groups.  With
    // one k-block per stage the raw rows are 64 plain bytes and thread t reads its chunks in the
    // order sig(t) ^ c, sig a permutation of 0..3 over (t / 2) & 3 for which sig ^ ((t / 2) & 3)
    // is a permutation too: again 32 different banks per quarter warp, loads and stores.
    const int ct = threadIdx.x - kGemmThreads;
    const int grp = ct >> 7, row = ct & 127;
    const int sig = S::kKS == 1 ? (0x2130 >> (4 * ((row >> 1) & 3))) & 3 : 0;
    constexpr int kA16 = S::kA16Stages > 0 ? S::kA16Stages : 1;
    int nst = 0;  // stages of this CTA so far, over all its units
    int nkb = 0;  // k-blocks so far
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int tile = u / g.splits, sp = u - tile * g.splits;
      const int kb0 = sp * kb_per;
      const int kb1 = min(g.kblocks, kb0 + kb_per);
      const int grow = (tile / g.tiles_b) * kTileA + row;
      const __half* gs = (g.gscale && grow < g.ra) ? g.gscale + size_t(grow) * g.gs_groups : nullptr;
      for (int kb = kb0; kb < kb1 && ok; kb += S::kKS, ++nst) {
        const int nsub = S::kKS == 1 ? 1 : min(S::kKS, kb1 - kb);
        if ((nst & 1) != grp) {
          nkb += nsub;
          continue;
        }
        const int stage = nst % S::kStages;
        if (!mbar_wait_bounded(&full_bar[stage], uint32_t(nst / S::kStages) & 1u, s_abort)) {
          ok = false;
          break;
        }
        const uint32_t raw = ring + stage * S::kStageBytes + S::kOffRaw + row * (kTileK * S::kKS);
#pragma unroll
        for (int sb = 0; sb < S::kKS; ++sb, ++nkb) {
          if (sb >= nsub) break;
          const int astage = nkb % kA16;
          const float sc = gs ? __half2float(gs[(kb + sb) / g.gs_kblocks]) : 1.f;
          if (!mbar_wait_bounded(&afree_bar[astage], (uint32_t(nkb / kA16) & 1u) ^ 1u, s_abort)) {
            ok = false;
            break;
          }
          const uint32_t dst = ring + S::kStages * S::kStageBytes + astage * S::kStageA + row * 128;
          uint32_t w[4][4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int ch = S::kKS == 1 ? (sig ^ c) : ((sb * 4 + c) ^ (row & 7));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w[c][0]), "=r"(w[c][1]), "=r"(w[c][2]), "=r"(w[c][3])
                         : "r"(raw + (ch << 4)));
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o0, o1, o2, o3, o4, o5, o6, o7;
            if (g.gscale) {
              s8x4_to_bf16x4_scaled(w[c][0], sc, o0, o1);
              s8x4_to_bf16x4_scaled(w[c][1], sc, o2, o3);
              s8x4_to_bf16x4_scaled(w[c][2], sc, o4, o5);
              s8x4_to_bf16x4_scaled(w[c][3], sc, o6, o7);
            } else {
              s8x4_to_bf16x4(w[c][0], o0, o1);
              s8x4_to_bf16x4(w[c][1], o2, o3);
              s8x4_to_bf16x4(w[c][2], o4, o5);
              s8x4_to_bf16x4(w[c][3], o6, o7);
            }
            const int c0 = (S::kKS == 1 ? (sig ^ c) : c) * 2, c1 = c0 + 1;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (((c0 ^ (row & 7))) << 4)),
                         "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                         : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (((c1 ^ (row & 7))) << 4)),
                         "r"(o4), "r"(o5), "r"(o6), "r"(o7)
                         : "memory");
          }
          fence_proxy_async_smem();  // the tensor core reads what these threads just wrote
          __syncwarp();
          if (lane == 0) mbar_arrive(&ready_bar[astage]);
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;
    const int et = threadIdx.x - 64;  // 0..127
    constexpr bool i8 = MODE != 0;
    uint32_t tphase[2] = {0, 0};
    int it = 0;
    [[maybe_unused]] int gcount = 0;  // grouped int8: k-blocks drained so far
    pdl_wait();  // outputs, residuals and the split-K scratch belong to earlier kernels until now
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++it) {
      const int tile = u / g.splits, sp = u - tile * g.splits;
      const int ta = tile / g.tiles_b, tb = tile - ta * g.tiles_b;
      if constexpr (MODE == 2) {
        {
          // one accumulator per k-block: acc * scale[row][group] summed in registers
          const int kb0 = sp * kb_per, kb1 = min(g.kblocks, kb0 + kb_per);
          const int grow = ta * kTileA + row;
          const __nv_bfloat16* gs = grow < g.ra ? g.gscale_bf + size_t(grow) * g.gs_groups : nullptr;
          float accf[BN];
#pragma unroll
          for (int i = 0; i < BN; ++i) accf[i] = 0.f;
          bool ok = true;
          for (int kb = kb0; kb < kb1; ++kb, ++gcount) {
            const int gb = gcount & 1;
            const float sc = gs ? __bfloat162float(gs[kb / g.gs_kblocks]) : 0.f;
            if (!mbar_wait_bounded(&tfull_bar[gb], tphase[gb], s_abort)) {
              ok = false;
              break;
            }
            tphase[gb] ^= 1u;
            tc_fence_after_sync();
            const uint32_t ta2 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(gb * BN);
            if constexpr (BN >= 32) {
#pragma unroll
              for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(ta2 + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) accf[c0 + i] = fmaf(float(int32_t(r[i])), sc, accf[c0 + i]);
              }
            } else {
              uint32_t r[16];
              tmem_ld_32x16(ta2, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) accf[i] = fmaf(float(int32_t(r[i])), sc, accf[i]);
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[gb]);
          }
          if (!ok) break;
#pragma unroll
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = (c0 + i < BN) ? accf[(c0 + i) < BN ? (c0 + i) : 0] : 0.f;
            sink(ta, tb, sp, row, c0, v, BN < 32 ? BN : 32);
          }
          sink.unit_done(et);
          continue;
        }
      }
      const int acc = it & 1;
      if (!mbar_wait_bounded(&tfull_bar[acc], tphase[acc], s_abort)) break;
      tphase[acc] ^= 1u;
      tc_fence_after_sync();
      if (tr && et == 0 && it == 0) tr[4] = globaltimer_ns();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN);
      if (g.splits == 1 || g.direct) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          if constexpr (BN >= 32) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = acc_f32(r[i], i8);
          } else {
            uint32_t r[16];
            tmem_ld_32x16(taddr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = acc_f32(r[i], i8);
#pragma unroll
            for (int i = 16; i < 32; ++i) v[i] = 0.f;
          }
          sink(ta, tb, sp, row, c0, v, BN < 32 ? BN : 32);
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
        sink.unit_done(et);
      } else {
        // partial tile -> workspace [unit][row][col] (each thread owns a row)
        float4* wp = reinterpret_cast<float4*>(g.ws + (size_t(u) * kTileA + row) * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if constexpr (BN >= 32) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              __stcg(wp + (c0 + i) / 4,
                     make_float4(acc_f32(r[i], i8), acc_f32(r[i + 1], i8), acc_f32(r[i + 2], i8), acc_f32(r[i + 3], i8)));
          } else {
            uint32_t r[16];
            tmem_ld_32x16(taddr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              __stcg(wp + (c0 + i) / 4,
                     make_float4(acc_f32(r[i], i8), acc_f32(r[i + 1], i8), acc_f32(r[i + 2], i8), acc_f32(r[i + 3], i8)));
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          const uint32_t old = atomicAdd(&g.counters[tile], 1u);
          *s_last = (old == uint32_t(g.splits - 1)) ? 1u : 0u;
          if (old == uint32_t(g.splits - 1)) g.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tr && et == 0 && it == 0) tr[5] = globaltimer_ns();
        if (*s_last) {
          __threadfence();
          const float* base = g.ws + (size_t(tile) * g.splits * kTileA + row) * BN;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            constexpr int kW = BN < 32 ? BN : 32;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
            // splits are summed in order: the result does not depend on arrival order
            for (int s2 = 0; s2 < g.splits; ++s2) {
              const float4* p =
                  reinterpret_cast<const float4*>(base + size_t(s2) * (BN * kTileA) + c0);
#pragma unroll
              for (int i = 0; i < kW / 4; ++i) {
                const float4 f = __ldcg(p + i);
                v[4 * i] += f.x;
                v[4 * i + 1] += f.y;
                v[4 * i + 2] += f.z;
                v[4 * i + 3] += f.w;
              }
            }
            sink(ta, tb, 0, row, c0, v, kW);
          }
          if (tr && et == 0 && it == 0) tr[7] = globaltimer_ns();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tr && threadIdx.x == 0) tr[6] = globaltimer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
  if (threadIdx.x == 0 && *s_abort && g.err) *g.err = 1u;
  if (threadIdx.x == 0 && g.gate_flags) {
    __threadfence();
    const uint32_t t = atomicAdd(g.gate_ticket, 1u);
    if (t == gridDim.x - 1) {
      *g.gate_ticket = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(g.gate_cum) = *g.gate_cum + g.gate_add;
    }
  }
}

}  // namespace bl
