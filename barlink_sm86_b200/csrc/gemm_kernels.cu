// SPDX-License-Identifier: MIT
//
// bf16 linear layers on the tcgen05 core: kernel instantiations, the local
// epilogue (bias / residual / SiLU*mul on interleaved gate-up rows), tensor
// map cache and launch heuristics.  These are the kernels behind every
// nn.Linear of the tensor-parallel models; the reference runs the same
// layers through cuBLAS (demos/qwen_tp/qwen38_int8/worker.py:224) or its
// dp4a kernel (torch_ext/barlink_sm86/w8a16.cu:94-153).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "bl_ops.h"
#include "gemm_core.cuh"
#include "heap.h"
#include "launch.h"

namespace bl {

// Epilogue that stores to local memory.
//   swap = 0: A rows are tokens (m), B rows are output features (n)
//   swap = 1: A rows are output features (n), B rows are tokens (m)
// out is [tokens, ldo] bf16.  epi bits: 1 bias[n], 2 residual[m, n] added,
// 4 SiLU(gate)*up where gate/up rows are interleaved (even n = gate, odd n =
// up) and the result lands in column n/2.
// tanh on the special-function unit (one instruction; relative error about 2^-11, below bf16's)
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int BN>
struct LocalSink {
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ldo, ra, rb, swap, epi;
  const __nv_bfloat16* scale;  // per output feature (W8A16), or null
  const float* xscale;         // per token (int8 activations), or null
  // Row push (token-major only, pworld > 0): row m belongs to rank (prow0 + m) / ptpr and is stored
  // into that rank's staging inbox slot for this rank -- the scatter half of a two-shot all-reduce
  // done by the GEMM epilogue over NVLink, tile by tile, while the other tiles are still in the
  // tensor cores.
  char* parena[kMaxRanks];
  uint32_t* pflag[kMaxRanks];
  const uint32_t* pseq;
  size_t pstage_off, pstage_slice;
  int pworld, prank, ptpr, prow0;

  // every epilogue thread of the CTA calls this after a tile (nthr of them: 128 or 256)
  template <int NTHR>
  __device__ __forceinline__ void tile_done(int et) const {
    if (pworld > 0) {
      __threadfence_system();
      if (NTHR == 128) asm volatile("bar.sync 1, 128;" ::: "memory");
      else asm volatile("bar.sync 1, 256;" ::: "memory");
      if (et < pworld) red_release_sys_add(pflag[et], 1u);
    }
  }
  __device__ __forceinline__ void unit_done(int et) const { tile_done<128>(et); }
  __device__ __forceinline__ void operator()(int ta, int tb, int /*split*/, int row, int c0,
                                             const float (&vin)[32], int ncols) const {
    const int i = ta * kTileA + row;
    const int j0 = tb * BN + c0;
    float v[32];
    if (scale) {
      if (swap) {
        const float sc = i < ra ? __bfloat162float(scale[i]) : 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = vin[c] * sc;
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          v[c] = (c < ncols && j0 + c < rb) ? vin[c] * __bfloat162float(scale[j0 + c]) : 0.f;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = vin[c];
    }
    if (xscale) {
      if (swap) {
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] *= (c < ncols && j0 + c < rb) ? xscale[j0 + c] : 0.f;
      } else {
        const float sc = i < ra ? xscale[i] : 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] *= sc;
      }
    }
    if (!swap) {
      const int m = i;
      if (m >= ra) return;
      if (epi & 4) {
        // pairs (gate, up) sit in adjacent columns of this thread
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const int n = j0 + c;
          if (c < ncols && n + 1 < rb) {
            float gte = v[c], up = v[c + 1];
            if (epi & 1) {
              gte += __bfloat162float(bias[n]);
              up += __bfloat162float(bias[n + 1]);
            }
            const float r = gte / (1.f + __expf(-gte)) * up;
            out[size_t(m) * ldo + (n >> 1)] = __float2bfloat16(r);
          }
        }
        return;
      }
      __nv_bfloat16* orow = out + size_t(m) * ldo;
      if (pworld > 0) {
        const int gm = prow0 + m;
        const int owner = gm / ptpr;
        const size_t buf = pstage_off + size_t(*pseq & 1u) * (2 * size_t(pworld) * pstage_slice);
        orow = reinterpret_cast<__nv_bfloat16*>(parena[owner] + buf + size_t(prank) * pstage_slice) +
               size_t(gm - owner * ptpr) * ldo;
      }
      const __nv_bfloat16* rrow = residual ? residual + size_t(m) * ldo : nullptr;
      if (ncols == 32 && j0 + 32 <= rb && (ldo & 7) == 0) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          float x[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) x[t] = v[c + t];
          if (epi & 1) {
            const uint4 b = *reinterpret_cast<const uint4*>(bias + j0 + c);
            const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
                         b3 = unpack_bf16x2(b.w);
            x[0] += b0.x; x[1] += b0.y; x[2] += b1.x; x[3] += b1.y;
            x[4] += b2.x; x[5] += b2.y; x[6] += b3.x; x[7] += b3.y;
          }
          if (epi & 8) {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const float u = x[t];
              x[t] = 0.5f * u * (1.f + tanh_fast(0.7978845608f * (u + 0.044715f * u * u * u)));
            }
          }
          if (epi & 2) {
            const uint4 b = *reinterpret_cast<const uint4*>(rrow + j0 + c);
            const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
                         b3 = unpack_bf16x2(b.w);
            x[0] += b0.x; x[1] += b0.y; x[2] += b1.x; x[3] += b1.y;
            x[4] += b2.x; x[5] += b2.y; x[6] += b3.x; x[7] += b3.y;
          }
          *reinterpret_cast<uint4*>(orow + j0 + c) =
              make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                         pack_bf16x2(x[6], x[7]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int n = j0 + c;
          if (c < ncols && n < rb) {
            float x = v[c];
            if (epi & 1) x += __bfloat162float(bias[n]);
            if (epi & 8) x = 0.5f * x * (1.f + tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x)));
            if (epi & 2) x += __bfloat162float(rrow[n]);
            orow[n] = __float2bfloat16(x);
          }
        }
      }
    } else {
      const int n = i;
      const bool nok = n < ra;
      const float bv = (nok && (epi & 1)) ? __bfloat162float(bias[n]) : 0.f;
      if (epi & 4) {
        // even lane holds the gate row, odd lane the matching up row
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float mine = v[c] + bv;
          const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
          const int m = j0 + c;
          if (c < ncols && m < rb && nok && !(row & 1)) {
            const float r = mine / (1.f + __expf(-mine)) * other;
            out[size_t(m) * ldo + (n >> 1)] = __float2bfloat16(r);
          }
        }
        return;
      }
      if (!nok) return;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int m = j0 + c;
        if (c < ncols && m < rb) {
          float x = v[c] + bv;
          if (epi & 8) x = 0.5f * x * (1.f + tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x)));
          if (epi & 2) x += __bfloat162float(residual[size_t(m) * ldo + n]);
          out[size_t(m) * ldo + n] = __float2bfloat16(x);
        }
      }
    }
  }
};

template <int BN, int CPS>
__global__ void __launch_bounds__(kGemmThreads, CPS)
    k_gemm(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
           GemmShape g, LocalSink<BN> sink, uint64_t hint_a, uint64_t hint_b) {
  gemm_body<BN, CPS, false>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}

// int8 operands (GemmShape::i8 = MODE: 1 plain, 2 per-group weight scales with one accumulator per k-block)
template <int BN, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
    k_gemm_i8(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              GemmShape g, LocalSink<BN> sink, uint64_t hint_a, uint64_t hint_b) {
  static_assert(MODE == 1 || (MODE == 2 && BN <= 64), "the per-group accumulators live in registers");
  gemm_body<BN, 1, false, MODE>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}

// Epilogue of the split-K decode path: every k-split stores its raw fp32
// partial tile to slab[split][token][feature]; the kernel that consumes the
// linear's output (add+RMSNorm, RoPE+KV write, the fused all-reduce) sums the
// slabs while it reads them, so the GEMM has no reduction tail at all.
template <int BN>
struct PartialSink {
  float* out;          // [splits][tokens][n]
  size_t slab;         // elements per split
  int ldo, ra, rb, swap;
  const __nv_bfloat16* scale;  // per output feature (W8A16), or null

  __device__ __forceinline__ void unit_done(int) const {}
  __device__ __forceinline__ void operator()(int ta, int tb, int split, int row, int c0,
                                             const float (&vin)[32], int ncols) const {
    const int i = ta * kTileA + row;
    const int j0 = tb * BN + c0;
    float* base = out + size_t(split) * slab;
    float v[32];
    if (scale) {
      if (swap) {
        const float sc = i < ra ? __bfloat162float(scale[i]) : 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = vin[c] * sc;
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          v[c] = (c < ncols && j0 + c < rb) ? vin[c] * __bfloat162float(scale[j0 + c]) : 0.f;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = vin[c];
    }
    if (swap) {
      if (i >= ra) return;  // i = feature, j = token: a warp stores 32 consecutive features
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < ncols && j0 + c < rb) __stcg(base + size_t(j0 + c) * ldo + i, v[c]);
    } else {
      if (i >= ra) return;  // i = token, j = feature
      float* orow = base + size_t(i) * ldo;
      if (ncols == 32 && j0 + 32 <= rb && (ldo & 3) == 0) {
#pragma unroll
        for (int c = 0; c < 32; c += 4)
          __stcg(reinterpret_cast<float4*>(orow + j0 + c), make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]));
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c < ncols && j0 + c < rb) __stcg(orow + j0 + c, v[c]);
      }
    }
  }
};

// Epilogue of the row-parallel linear fused with the reduce-scatter: token m
// belongs to rank m / tpr; every k-split stores its fp32 partial row straight
// into that rank's inbox [src rank][split][local token][feature] over NVLink
// and, once a tile is out, bumps the owners' arrival counters with a release at
// system scope.  No collective library call, no local staging.
template <int BN>
struct PeerSlabSink {
  float* inbox[kMaxRanks];      // each owner's inbox as mapped here
  uint32_t* flag[kMaxRanks];    // each owner's arrival word for this source rank
  int world, rank, tpr, n, splits, tokens;

  __device__ __forceinline__ void operator()(int ta, int tb, int split, int row, int c0,
                                             const float (&v)[32], int ncols) const {
    const int i = ta * kTileA + row;  // feature
    const int j0 = tb * BN + c0;      // first token of this chunk
    if (i >= n) return;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const int m = j0 + c;
      if (c < ncols && m < tokens) {
        const int owner = m / tpr, lm = m - owner * tpr;
        float* dst = inbox[owner] + ((size_t(rank) * splits + split) * tpr + lm) * n + i;
        asm volatile("st.global.f32 [%0], %1;" ::"l"(dst), "f"(v[c]) : "memory");
      }
    }
  }
  __device__ __forceinline__ void unit_done(int et) const {
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et < world) red_release_sys_add(flag[et], 1u);
  }
};

template <int BN, int CPS>
__global__ void __launch_bounds__(kGemmThreads, CPS)
    k_gemm_peer(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                GemmShape g, PeerSlabSink<BN> sink, uint64_t hint_a, uint64_t hint_b) {
  gemm_body<BN, CPS, false>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}

template <int BN, int CPS>
__global__ void __launch_bounds__(kGemmThreads, CPS)
    k_gemm_partial(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, GemmShape g, PartialSink<BN> sink,
                   uint64_t hint_a, uint64_t hint_b) {
  gemm_body<BN, CPS, false>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}

// Re-layout of a weight matrix [n x k] (row pitch ld) into 16 KiB tiles
// [ceil(n/128)][ceil(k/64)][128 rows x 128 bytes], each tile in the 128-byte
// swizzled shared-memory image (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
// Rows and columns beyond the matrix are zero.
__global__ void k_tile_weight(const __nv_bfloat16* __restrict__ src, uint4* __restrict__ dst, int n, int k,
                              int ld, int tkb, size_t total_chunks) {
  for (size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total_chunks;
       t += size_t(gridDim.x) * blockDim.x) {
    const size_t tile = t >> 10;           // 1024 chunks per tile
    const int in_tile = int(t & 1023);
    const int r = in_tile >> 3, cpos = in_tile & 7;
    const int c = cpos ^ (r & 7);          // logical chunk stored at this position
    const int rb = int(tile / tkb), kb = int(tile % tkb);
    const int row = rb * 128 + r, col = kb * 64 + c * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n && col < k) {
      if (col + 8 <= k && ((size_t(row) * ld + col) & 7) == 0) {
        v = *reinterpret_cast<const uint4*>(src + size_t(row) * ld + col);
      } else {
        __nv_bfloat16 tmp[8];
        for (int j = 0; j < 8; ++j) tmp[j] = col + j < k ? src[size_t(row) * ld + col + j] : __float2bfloat16(0.f);
        v = *reinterpret_cast<uint4*>(tmp);
      }
    }
    dst[t] = v;
  }
}

// ---------------------------------------------------------------------------
// tensor map cache
// ---------------------------------------------------------------------------
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, esize, box_cols;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && esize == o.esize && box_cols == o.box_cols;
  }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    return (h * 31u + k.esize) * 31u + k.box_cols;
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapHash> g_tmaps;
static std::mutex g_tmap_mu;

// K-major matrix [rows x cols] of 1- or 2-byte elements, row pitch ld elements, box = box_rows x
// box_cols elements: 128 bytes per box row in the 128-byte swizzle (64 bf16, or 128 int8 = two
// k-blocks), or 64 plain bytes of int8.
int make_tmap_kmajor(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t esize, CUtensorMap* out, char* err, size_t errlen, uint32_t box_cols) {
  TmapKey key{ptr, rows, cols, ld, box_rows, esize, box_cols};
  if (box_cols * esize != 128 && !(esize == 1 && box_cols == 64)) {
    set_err(err, errlen, "barlink: unsupported tensor-map box of %u elements of %u bytes", box_cols, esize);
    return -1;
  }
  {
    std::lock_guard<std::mutex> g(g_tmap_mu);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return 0;
    }
  }
  const DriverApi* d = driver(err, errlen);
  if (!d) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || ((ld * esize) & 15u)) {
    set_err(err, errlen,
            "barlink: GEMM operand must be 16-byte aligned with a row pitch that is a multiple of 16 bytes (ptr %p, pitch %llu B)",
            ptr, (unsigned long long)(ld * esize));
    return -1;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = d->cuTensorMapEncodeTiled(
      &m, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      box_cols * esize == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    const char* s = nullptr;
    d->cuGetErrorString(r, &s);
    set_err(err, errlen, "barlink: cuTensorMapEncodeTiled(rows %llu, cols %llu, box %u) failed: %s",
            (unsigned long long)rows, (unsigned long long)cols, box_rows, s ? s : "?");
    return -1;
  }
  {
    std::lock_guard<std::mutex> g(g_tmap_mu);
    if (g_tmaps.size() > 65536) g_tmaps.clear();
    g_tmaps[key] = m;
  }
  *out = m;
  return 0;
}

static int g_sm_count = 0;
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

// splits such that tiles*splits fills the SMs once and every split is non-empty
int pick_splits(int tiles, int kblocks, int sms, int want) {
  int s = want;
  if (s <= 0) {
    s = 1;
    if (tiles * 2 <= sms) {
      s = sms / tiles;
      const int max_by_k = kblocks / 4 > 0 ? kblocks / 4 : 1;  // >= 4 k-blocks per split
      if (s > max_by_k) s = max_by_k;
    }
  }
  if (s > kblocks) s = kblocks;
  if (s < 1) s = 1;
  const int per = (kblocks + s - 1) / s;
  return (kblocks + per - 1) / per;
}

static int env_int_or(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

template <class SinkT>
static void fill_push(SinkT& sink, const blRowPush* p) {
  sink.pworld = 0;
  sink.pseq = nullptr;
  sink.pstage_off = sink.pstage_slice = 0;
  sink.prank = sink.ptpr = sink.prow0 = 0;
  for (int r = 0; r < kMaxRanks; ++r) {
    sink.parena[r] = nullptr;
    sink.pflag[r] = nullptr;
  }
  if (!p) return;
  sink.pworld = p->world;
  sink.prank = p->rank;
  sink.ptpr = p->rows_per_rank;
  sink.prow0 = p->row0;
  sink.pseq = static_cast<const uint32_t*>(p->seq_word);
  sink.pstage_off = p->stage_off;
  sink.pstage_slice = p->stage_slice;
  for (int r = 0; r < p->world; ++r) {
    sink.parena[r] = static_cast<char*>(p->arena[r]);
    sink.pflag[r] = static_cast<uint32_t*>(p->flag[r]);
  }
}

template <int BN, int CPS>
static int launch_gemm(const blGemmArgs& a, int splits_want, cudaStream_t st, char* err,
                       size_t errlen) {
  using S = GemmSmem<BN, CPS>;
  CUtensorMap ta, tb;
  // a pre-tiled weight operand needs no tensor map (the other operand's map stands in)
  const bool a_tiled = a.weight_tiled && a.swap, b_tiled = a.weight_tiled && !a.swap;
  const uint32_t esize = a.i8 ? 1 : 2, box_cols = a.i8 ? 2 * kTileK : kTileK;  // 128 bytes per box row either way
  if (!b_tiled && make_tmap_kmajor(a.b, a.rb, a.k, a.ldb, BN, esize, &tb, err, errlen, box_cols) != 0) return -1;
  if (!a_tiled && make_tmap_kmajor(a.a, a.ra, a.k, a.lda, kTileA, esize, &ta, err, errlen, box_cols) != 0) return -1;
  if (a_tiled) ta = tb;
  if (b_tiled) tb = ta;
  GemmShape g;
  g.ra = a.ra;
  g.rb = a.rb;
  g.k = a.k;
  g.tiles_a = (a.ra + kTileA - 1) / kTileA;
  g.tiles_b = (a.rb + BN - 1) / BN;
  g.kblocks = (a.k + int(box_cols) - 1) / int(box_cols);
  g.i8 = a.i8 ? 1 : 0;
  g.gscale_bf = nullptr;
  if (a.i8 && a.group_scale) {
    g.i8 = 2;
    g.gscale_bf = static_cast<const __nv_bfloat16*>(a.group_scale);
    g.gs_groups = (a.k + a.group_k - 1) / a.group_k;
    g.gs_kblocks = a.group_k / int(box_cols);
  }
  const int tiles = g.tiles_a * g.tiles_b;
  const int sms = sm_count();
  // CTAs launched at most (BL_GEMM_WAVE: percent of the resident slots)
  static const int wave = env_int_or("BL_GEMM_WAVE", 100);
  int slots = sms * S::kCtasPerSm * wave / 100;
  if (slots < 1) slots = 1;
  g.splits = g.i8 == 2 ? 1 : pick_splits(tiles, g.kblocks, slots, splits_want);
  const bool partial = a.partial_out != nullptr || a.peer != nullptr;
  if (partial) {
    if (a.partial_splits < 1 || g.splits > a.partial_splits) g.splits = a.partial_splits;
    // the caller sized the slabs for exactly partial_splits; fewer is not allowed
    const int per = (g.kblocks + a.partial_splits - 1) / a.partial_splits;
    if ((g.kblocks + per - 1) / per != a.partial_splits) {
      set_err(err, errlen, "barlink: %d k-splits do not divide %d k-blocks into non-empty parts",
              a.partial_splits, g.kblocks);
      return -1;
    }
    g.splits = a.partial_splits;
  } else if (g.splits > 1) {
    const size_t need = size_t(tiles) * g.splits * BN * kTileA * sizeof(float);
    if (!a.ws || a.ws_bytes < need || !a.counters || a.n_counters < tiles) g.splits = 1;
  }
  if (a.push) g.splits = 1;  // a tile is pushed once, whole
  g.direct = 0;
  g.tiled = a_tiled ? 1 : b_tiled ? 2 : 0;
  g.tiled_base = static_cast<const uint8_t*>(a_tiled ? a.a : a.b);
  g.tiled_kblocks = (a.k + kTileK - 1) / kTileK;
  g.gate_flags = static_cast<const uint32_t*>(a.gate_flags);
  g.gate_cum = static_cast<uint32_t*>(a.gate_cum);
  g.gate_ticket = static_cast<uint32_t*>(a.gate_ticket);
  g.gate_add = a.gate_add;
  g.gate_n = a.gate_n;
  g.gate_timeout_ns = a.gate_timeout_ns ? a.gate_timeout_ns : 2000000000ull;
  g.ab_fmt = 1;
  g.gscale = nullptr;
  if (g.i8 != 2) {
    g.gs_groups = 0;
    g.gs_kblocks = 1;
  }
  g.weights_in_a = a.dynamic_weights ? 2 : (a.swap ? 1 : 0);
  g.ws = static_cast<float*>(a.ws);
  g.counters = static_cast<uint32_t*>(a.counters);
  g.err = static_cast<uint32_t*>(a.err_flag);
  g.trace = static_cast<unsigned long long*>(a.trace);
  const int units = tiles * g.splits;
  const int grid = units < slots ? units : slots;
  // weights stream through L2 once, activations are re-read by every CTA
  const uint64_t hint_w = kHintEvictFirst, hint_x = kHintEvictLast;
  cudaError_t e;
  if (a.peer) {
    g.direct = 1;
    const blPeerSink& ps_in = *a.peer;
    PeerSlabSink<BN> ps;
    for (int r = 0; r < kMaxRanks; ++r) {
      ps.inbox[r] = static_cast<float*>(ps_in.inbox[r]);
      ps.flag[r] = static_cast<uint32_t*>(ps_in.flag[r]);
    }
    ps.world = ps_in.world;
    ps.rank = ps_in.rank;
    ps.tpr = ps_in.tokens_per_rank;
    ps.n = a.ra;
    ps.splits = g.splits;
    ps.tokens = a.rb;
    static bool attr_q = false;
    if (!attr_q) {
      e = cudaFuncSetAttribute(k_gemm_peer<BN, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               S::kBytes);
      if (e != cudaSuccess) {
        set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes,
                cudaGetErrorString(e));
        return -1;
      }
      attr_q = true;
    }
    e = launch_k(k_gemm_peer<BN, CPS>, dim3(grid), dim3(kGemmThreads), size_t(S::kBytes), st, ta, tb,
                 g, ps, hint_w, hint_x);
  } else if (partial) {
    g.direct = 1;
    PartialSink<BN> ps;
    ps.out = static_cast<float*>(a.partial_out);
    ps.slab = a.partial_stride;
    ps.ldo = a.ldo;
    ps.ra = a.ra;
    ps.rb = a.rb;
    ps.swap = a.swap;
    ps.scale = nullptr;
    static bool attr_p = false;
    if (!attr_p) {
      e = cudaFuncSetAttribute(k_gemm_partial<BN, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               S::kBytes);
      if (e != cudaSuccess) {
        set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes,
                cudaGetErrorString(e));
        return -1;
      }
      attr_p = true;
    }
    e = launch_k(k_gemm_partial<BN, CPS>, dim3(grid), dim3(kGemmThreads), size_t(S::kBytes), st, ta,
                 tb, g, ps, a.swap ? hint_w : hint_x, a.swap ? hint_x : hint_w);
  } else {
    LocalSink<BN> sink;
    sink.out = static_cast<__nv_bfloat16*>(a.out);
    sink.bias = static_cast<const __nv_bfloat16*>(a.bias);
    sink.residual = static_cast<const __nv_bfloat16*>(a.residual);
    sink.ldo = a.ldo;
    sink.ra = a.ra;
    sink.rb = a.rb;
    sink.swap = a.swap;
    sink.epi = (a.bias ? 1 : 0) | (a.residual ? 2 : 0) | (a.silu_mul ? 4 : 0) | (a.gelu ? 8 : 0);
    sink.scale = static_cast<const __nv_bfloat16*>(a.feat_scale);
    sink.xscale = static_cast<const float*>(a.tok_scale);
    fill_push(sink, a.push);
    static bool attr_set = false;
    if (!attr_set) {
      e = cudaFuncSetAttribute(k_gemm<BN, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               S::kBytes);
      if (e != cudaSuccess) {
        set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes,
                cudaGetErrorString(e));
        return -1;
      }
      attr_set = true;
    }
    bool done = false;
    if (g.i8) {
      using S1 = GemmSmem<BN, 1>;
      auto go = [&](auto kern) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S1::kBytes);
        if (e == cudaSuccess)
          e = launch_k(kern, dim3(grid), dim3(kGemmThreads), size_t(S1::kBytes), st, ta, tb, g, sink,
                       a.swap ? hint_w : hint_x, a.swap ? hint_x : hint_w);
      };
      if (g.i8 == 1) {
        go(k_gemm_i8<BN, 1>);
        done = true;
      } else if constexpr (BN <= 64) {
        go(k_gemm_i8<BN, 2>);
        done = true;
      }
      if (!done) {
        set_err(err, errlen, "barlink: per-group int8 scales need a tile of at most 64 tokens");
        return -1;
      }
    }
    if (!done)
      e = launch_k(k_gemm<BN, CPS>, dim3(grid), dim3(kGemmThreads), size_t(S::kBytes), st, ta, tb, g,
                   sink, a.swap ? hint_w : hint_x, a.swap ? hint_x : hint_w);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: GEMM launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

// ---------------------------------------------------------------------------
// W8A16: int8 per-channel weights widened to bf16 inside the main loop
// ---------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(GemmSmem<BN, 1, true>::kThreads, 1)
    k_gemm_w8(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              GemmShape g, LocalSink<BN> sink, uint64_t hint_a, uint64_t hint_b) {
  gemm_body<BN, 1, true>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}
template <int BN>
__global__ void __launch_bounds__(GemmSmem<BN, 1, true>::kThreads, 1)
    k_gemm_w8_partial(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b, GemmShape g, PartialSink<BN> sink,
                      uint64_t hint_a, uint64_t hint_b) {
  gemm_body<BN, 1, true>(&tmap_a, &tmap_b, g, sink, hint_a, hint_b);
}

__global__ void k_w8_dequant(const int8_t* __restrict__ wq, const __nv_bfloat16* __restrict__ scale,
                             __nv_bfloat16* __restrict__ out, int n, int k) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = size_t(n) * k / 8;
  for (size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += size_t(gridDim.x) * blockDim.x) {
    const size_t e = t * 8;
    const int row = int(e / k);
    const float sc = __bfloat162float(scale[row]);
    const uint2 w = *reinterpret_cast<const uint2*>(wq + e);
    uint32_t a, b, c, d;
    s8x4_to_bf16x4(w.x, a, b);
    s8x4_to_bf16x4(w.y, c, d);
    const float2 f0 = unpack_bf16x2(a), f1 = unpack_bf16x2(b), f2 = unpack_bf16x2(c),
                 f3 = unpack_bf16x2(d);
    *reinterpret_cast<uint4*>(out + e) =
        make_uint4(pack_bf16x2(f0.x * sc, f0.y * sc), pack_bf16x2(f1.x * sc, f1.y * sc),
                   pack_bf16x2(f2.x * sc, f2.y * sc), pack_bf16x2(f3.x * sc, f3.y * sc));
  }
}

template <int BN>
static int launch_w8(const blW8A16Args& a, cudaStream_t st, char* err, size_t errlen) {
  using S = GemmSmem<BN, 1, true>;
  CUtensorMap ta, tb;
  if (make_tmap_kmajor(a.wq, a.n, a.k, a.k, kTileA, 1, &ta, err, errlen, 64 * S::kKS) != 0) return -1;
  if (make_tmap_kmajor(a.x, a.m, a.k, a.ldx, BN, 2, &tb, err, errlen) != 0) return -1;
  GemmShape g;
  memset(&g, 0, sizeof(g));
  g.ra = a.n;
  g.rb = a.m;
  g.k = a.k;
  g.tiles_a = (a.n + kTileA - 1) / kTileA;
  g.tiles_b = (a.m + BN - 1) / BN;
  g.kblocks = (a.k + kTileK - 1) / kTileK;
  const int tiles = g.tiles_a * g.tiles_b;
  const int sms = sm_count();
  const bool partial = a.partial_out != nullptr;
  g.splits = partial ? a.partial_splits : pick_splits(tiles, g.kblocks, sms, a.splits);
  if (!partial && g.splits > 1) {
    const size_t need = size_t(tiles) * g.splits * BN * kTileA * sizeof(float);
    if (!a.ws || a.ws_bytes < need || !a.counters || a.n_counters < tiles) g.splits = 1;
  }
  if (partial) {
    const int per = (g.kblocks + g.splits - 1) / g.splits;
    if (g.splits < 1 || (g.kblocks + per - 1) / per != g.splits) {
      set_err(err, errlen, "barlink: %d k-splits do not divide %d k-blocks into non-empty parts", g.splits,
              g.kblocks);
      return -1;
    }
  }
  g.ab_fmt = 1;
  if (a.group_rel) {
    g.gscale = static_cast<const __half*>(a.group_rel);
    g.gs_kblocks = a.group_k / kTileK;
    g.gs_groups = (a.k + a.group_k - 1) / a.group_k;
  }
  g.direct = partial ? 1 : 0;
  g.weights_in_a = 1;
  g.ws = static_cast<float*>(a.ws);
  g.counters = static_cast<uint32_t*>(a.counters);
  g.err = static_cast<uint32_t*>(a.err_flag);
  g.gate_timeout_ns = 2000000000ull;
  const int units = tiles * g.splits;
  const int grid = units < sms ? units : sms;
  cudaError_t e;
  if (partial) {
    PartialSink<BN> ps;
    ps.out = static_cast<float*>(a.partial_out);
    ps.slab = a.partial_stride;
    ps.ldo = a.ldo;
    ps.ra = a.n;
    ps.rb = a.m;
    ps.swap = 1;
    ps.scale = static_cast<const __nv_bfloat16*>(a.scale);
    static bool attr = false;
    if (!attr) {
      e = cudaFuncSetAttribute(k_gemm_w8_partial<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
      if (e != cudaSuccess) {
        set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes, cudaGetErrorString(e));
        return -1;
      }
      attr = true;
    }
    e = launch_k(k_gemm_w8_partial<BN>, dim3(grid), dim3(S::kThreads), size_t(S::kBytes), st, ta, tb, g, ps,
                 kHintEvictFirst, kHintEvictLast);
  } else {
    LocalSink<BN> sink;
    sink.out = static_cast<__nv_bfloat16*>(a.out);
    sink.bias = static_cast<const __nv_bfloat16*>(a.bias);
    sink.residual = nullptr;
    sink.ldo = a.ldo;
    sink.ra = a.n;
    sink.rb = a.m;
    sink.swap = 1;
    sink.epi = (a.bias ? 1 : 0) | (a.silu_mul ? 4 : 0);
    sink.scale = static_cast<const __nv_bfloat16*>(a.scale);
    sink.xscale = nullptr;
    fill_push(sink, nullptr);
    static bool attr = false;
    if (!attr) {
      e = cudaFuncSetAttribute(k_gemm_w8<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
      if (e != cudaSuccess) {
        set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", S::kBytes, cudaGetErrorString(e));
        return -1;
      }
      attr = true;
    }
    e = launch_k(k_gemm_w8<BN>, dim3(grid), dim3(S::kThreads), size_t(S::kBytes), st, ta, tb, g, sink,
                 kHintEvictFirst, kHintEvictLast);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: W8A16 launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

// ---------------------------------------------------------------------------
// Paired-CTA GEMM (token-major products of 512 tokens or more): two CTAs of a cluster work on one
// 256 x 256 output tile.  Each CTA loads 128 rows of A and 128 rows of B per
// k-block (32 KiB instead of the 48 KiB a lone CTA needs for 128 x 256), the
// leader CTA issues tcgen05.mma.cta_group::2 (M = 256 over the pair, N = 256),
// and each CTA's epilogue drains its own 128 accumulator rows.  The single-CTA
// kernel at these sizes is bound by tile delivery from L2; the pair moves a
// third less per SM.  Barrier protocol:
//   full[s]   leader only: its producer arms it for both CTAs' bytes; both
//             CTAs' TMA loads complete on the leader's barrier
//   empty[s]  one per CTA: the leader's MMA thread commits to its own and to
//             the peer's (two commits, the peer's through its cluster address)
//   tfull[a]  one per CTA, committed the same way when a tile's MMAs are done
//   tempty[a] leader only, 256 arrivals: every epilogue thread of both CTAs
// Large, unsplit, token-major ("no swap") products only.
// ---------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kTileA * kTileK * 2;  // A 16 KiB + B 16 KiB per CTA
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 + 1024;
constexpr int kPairBN = 256;
// warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue: two warps per TMEM lane quarter, each
// draining half of the 256 accumulator columns, so that the epilogue of a tile (bias, GELU,
// residual, stores) stays shorter than the main loop of the next one
constexpr int kPairThreads = 320;

__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t leader_bar,
                                                 int x, int y, uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
      "l"(tmap), "r"(leader_bar), "r"(x), "r"(y), "l"(hint)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once every MMA issued so far is done) on a barrier given by its cluster address
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar_addr)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}

// Order in which the pairs walk the output tiles.  The tiles of one dimension are cut into bands
// of `band` tiles; inside a band the other dimension is the slow index.  The operand slab of a band
// (band x 256 rows x K) stays in L2 while the other operand streams past it once per band, so each
// operand is fetched from DRAM a few times at most instead of once per wave of pairs.
__device__ __forceinline__ void pair_tile_of(int u, int tiles_m, int tiles_n, int band, int along_m, int& tm,
                                             int& tn) {
  const int nf = along_m ? tiles_m : tiles_n;  // banded dimension
  const int ns = along_m ? tiles_n : tiles_m;  // swept dimension
  const int per = band * ns;
  const int b = u / per, r = u - b * per;
  const int f0 = b * band;
  const int w = min(band, nf - f0);
  const int sl = r / w, f = f0 + r - sl * w;
  tm = along_m ? f : sl;
  tn = along_m ? sl : f;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    k_gemm_pair(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                GemmShape g, LocalSink<kPairBN> sink, uint64_t hint_a, uint64_t hint_b) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (ring - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kPairStages * kPairStageBytes);
  uint64_t* full_bar = bars;                       // kPairStages
  uint64_t* empty_bar = bars + kPairStages;        // kPairStages
  uint64_t* tfull_bar = bars + 2 * kPairStages;    // 2
  uint64_t* tempty_bar = tfull_bar + 2;            // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(tempty_bar + 3);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();           // 0 = leader
  const uint32_t peer = cr ^ 1u;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (g.ra + 255) / 256, tiles_n = (g.rb + 255) / 256;
  const int units = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * (kPairThreads - 64));
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    // both CTAs of the pair allocate together (same warp index, same slot address)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ producer (both CTAs) ------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += n_pairs) {
        int tm, tn;
        pair_tile_of(u, tiles_m, tiles_n, g.band, g.band_m, tm, tn);
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, s_abort)) {
            ok = false;
            break;
          }
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cr == 0) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          const uint32_t dst = ring + stage * kPairStageBytes;
          tma_load_2d_pair(dst, &tmap_a, leader_full, kb * kTileK, tm * 256 + int(cr) * 128, hint_a);
          tma_load_2d_pair(dst + kTileA * kTileK * 2, &tmap_b, leader_full, kb * kTileK, tn * 256 + int(cr) * 128,
                           hint_b);
          ++issued;
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      (void)issued;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) --------------
    if (lane == 0 && cr == 0) {
      const uint32_t idesc = umma_idesc_f16(256, kPairBN, g.ab_fmt);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tphase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += n_pairs, ++it) {
        const int acc = it & 1;
        if (!mbar_wait_bounded(&tempty_bar[acc], tphase[acc] ^ 1u, s_abort)) break;
        tphase[acc] ^= 1u;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * kPairBN);
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, s_abort)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = ring + stage * kPairStageBytes;
          const uint64_t da = umma_desc_k_sw128(sa);
          const uint64_t db = umma_desc_k_sw128(sa + kTileA * kTileK * 2);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k)
            umma_f16_ss_pair(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 1));
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int chalf = (warp - 2) >> 2;  // which half of the columns this warp drains
    uint32_t tphase[2] = {0, 0};
    int it = 0;
    for (int u = pair; u < units; u += n_pairs, ++it) {
      int tm, tn;
      pair_tile_of(u, tiles_m, tiles_n, g.band, g.band_m, tm, tn);
      const int acc = it & 1;
      if (!mbar_wait_bounded(&tfull_bar[acc], tphase[acc], s_abort)) break;
      tphase[acc] ^= 1u;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * kPairBN);
#pragma unroll 1
      for (int c0 = chalf * (kPairBN / 2); c0 < (chalf + 1) * (kPairBN / 2); c0 += 32) {
        float v[32];
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        // this CTA holds rows [tm*256 + cr*128, +128): the Sink's tile index is in units of 128 rows
        sink(tm * 2 + int(cr), tn, 0, row, c0, v, 32);
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      sink.template tile_done<256>(int(threadIdx.x) - 64);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the other may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort && g.err) *g.err = 1u;
}

// on by default: measured 1.22-1.54 PFLOP/s on the 4608-token MMDiT linears against 1.01-1.24 for
// the single-CTA kernel; BL_GEMM_PAIR=0 keeps the single-CTA kernel
static bool gemm_pair_enabled() {
  static const int v = env_int_or("BL_GEMM_PAIR", 1);
  return v == 1;
}

// token-major product with at least 512 tokens, no k-split, no fused collective
static bool gemm_pair_ok(const blGemmArgs& a) {
  return gemm_pair_enabled() && !a.i8 && !a.swap && a.ra >= 512 && a.rb >= 256 && !a.partial_out && !a.peer &&
         !a.gate_flags && !a.weight_tiled && !a.silu_mul && a.splits <= 1;
}

static int launch_gemm_pair(const blGemmArgs& a, cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap ta, tb;
  if (make_tmap_kmajor(a.a, a.ra, a.k, a.lda, kTileA, 2, &ta, err, errlen) != 0) return -1;
  if (make_tmap_kmajor(a.b, a.rb, a.k, a.ldb, kTileA, 2, &tb, err, errlen) != 0) return -1;
  GemmShape g{};
  g.ra = a.ra;
  g.rb = a.rb;
  g.k = a.k;
  g.kblocks = (a.k + kTileK - 1) / kTileK;
  g.splits = 1;
  g.ab_fmt = 1;
  g.err = static_cast<uint32_t*>(a.err_flag);
  LocalSink<kPairBN> sink;
  sink.out = static_cast<__nv_bfloat16*>(a.out);
  sink.bias = static_cast<const __nv_bfloat16*>(a.bias);
  sink.residual = static_cast<const __nv_bfloat16*>(a.residual);
  sink.ldo = a.ldo;
  sink.ra = a.ra;
  sink.rb = a.rb;
  sink.swap = 0;
  sink.epi = (a.bias ? 1 : 0) | (a.residual ? 2 : 0) | (a.gelu ? 8 : 0);
  sink.scale = nullptr;
  sink.xscale = nullptr;
  fill_push(sink, a.push);
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: cannot raise shared memory to %d B: %s", kPairSmem, cudaGetErrorString(e));
      return -1;
    }
    attr = true;
  }
  const int tiles_m = (a.ra + 255) / 256, tiles_n = (a.rb + 255) / 256;
  const int units = tiles_m * tiles_n;
  // band width: the slab that has to stay in L2 is at most 32 MB; bands of equal width; the
  // orientation that fetches fewer bytes from DRAM (slab operand once, the other once per band)
  const double tile_bytes = 256.0 * a.k * 2;
  int cap_tiles = int(32e6 / tile_bytes);
  if (cap_tiles < 1) cap_tiles = 1;
  auto even_band = [](int n, int wmax) {
    const int nb = (n + wmax - 1) / wmax;
    return (n + nb - 1) / nb;
  };
  const int wn = even_band(tiles_n, cap_tiles), wm = even_band(tiles_m, cap_tiles);
  const double dram_n = tile_bytes * (tiles_n + double(tiles_m) * ((tiles_n + wn - 1) / wn));
  const double dram_m = tile_bytes * (tiles_m + double(tiles_n) * ((tiles_m + wm - 1) / wm));
  static const int band_env = env_int_or("BL_GEMM_BAND", 0);  // debug: 0 = choose, n > 0 = bands of n along n, n < 0 along m
  g.band_m = band_env ? (band_env < 0) : (dram_m < dram_n);
  g.band = band_env ? (band_env < 0 ? -band_env : band_env) : (g.band_m ? wm : wn);
  if (g.band > (g.band_m ? tiles_m : tiles_n)) g.band = g.band_m ? tiles_m : tiles_n;
  int pairs = sm_count() / 2;
  if (pairs > units) pairs = units;
  if (pairs < 1) pairs = 1;
  // the cluster shape is compiled into the kernel (__cluster_dims__); the grid is a whole number of pairs
  // the slab operand is the one to keep in L2
  cudaError_t e = launch_k(k_gemm_pair, dim3(2 * pairs), dim3(kPairThreads), size_t(kPairSmem), st, ta, tb, g, sink,
                           g.band_m ? kHintEvictLast : kHintEvictFirst, g.band_m ? kHintEvictFirst : kHintEvictLast);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: paired GEMM launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace bl

using namespace bl;

extern "C" int bl_w8a16_linear(const blW8A16Args* a, void* stream, char* err, size_t errlen) {
  if (!a || (!a->x && !a->xq) || !a->wq || (!a->scale && !a->group_scale) || (!a->out && !a->partial_out) || a->m < 1 || a->n < 1 ||
      a->k < 16 || (a->k & 15)) {
    set_err(err, errlen, "barlink: w8a16_linear needs x, wq, scale, an output, and K a multiple of 16");
    return -1;
  }
  if (a->group_rel && (a->group_k < kTileK || a->group_k % kTileK)) {
    set_err(err, errlen, "barlink: in-kernel group scales need a group size that is a multiple of %d (got %d)", kTileK,
            a->group_k);
    return -1;
  }
  if (a->m > 256) {
    set_err(err, errlen, "barlink: the in-mainloop W8A16 kernel takes at most 256 tokens; dequantise (bl_w8_dequant) and use the bf16 GEMM for prefill");
    return -2;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int bn = a->m <= 16 ? 16 : a->m <= 32 ? 32 : a->m <= 64 ? 64 : a->m <= 128 ? 128 : 256;
  if (a->xq) {
    // int8 activations: the weights go from HBM to the tensor cores as they are
    if (!a->xs || a->group_rel || a->partial_out) {
      set_err(err, errlen, "barlink: int8 activations need their per-token scales and a plain output (group scales: group_scale)");
      return -1;
    }
    blGemmArgs g;
    memset(&g, 0, sizeof(g));
    g.a = a->wq; g.ra = a->n; g.lda = a->k;
    g.b = a->xq; g.rb = a->m; g.ldb = a->k;
    g.k = a->k;
    g.out = a->out; g.ldo = a->ldo;
    g.swap = 1;
    g.bias = a->bias;
    g.silu_mul = a->silu_mul;
    g.bn = bn;
    g.splits = a->splits;
    g.ws = a->ws; g.ws_bytes = a->ws_bytes;
    g.counters = a->counters; g.n_counters = a->n_counters;
    g.err_flag = a->err_flag;
    g.i8 = 1;
    if (a->group_scale) {
      g.group_scale = a->group_scale;
      g.group_k = a->group_k;
    } else {
      g.feat_scale = a->scale;
    }
    g.tok_scale = a->xs;
    return bl_gemm_bf16(&g, stream, err, errlen);
  }
  switch (bn) {
    case 16: return launch_w8<16>(*a, st, err, errlen);
    case 32: return launch_w8<32>(*a, st, err, errlen);
    case 64: return launch_w8<64>(*a, st, err, errlen);
    case 128: return launch_w8<128>(*a, st, err, errlen);
    default: return launch_w8<256>(*a, st, err, errlen);
  }
}

extern "C" int bl_w8_dequant(const void* wq, const void* scale, void* out, int n, int k, void* stream,
                             char* err, size_t errlen) {
  if (!wq || !scale || !out || n < 1 || k < 8 || (k & 7)) {
    set_err(err, errlen, "barlink: w8_dequant needs K a multiple of 8");
    return -1;
  }
  const size_t total = size_t(n) * k / 8;
  int grid = int((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  cudaError_t e = launch_k(k_w8_dequant, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const int8_t*>(wq), static_cast<const __nv_bfloat16*>(scale),
                           static_cast<__nv_bfloat16*>(out), n, k);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w8_dequant launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

__global__ void k_w8_group_scales(const __nv_bfloat16* __restrict__ sc, int n, int groups,
                                  __nv_bfloat16* __restrict__ row_max, __half* __restrict__ rel) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  float mx = 0.f;
  for (int g = 0; g < groups; ++g) mx = fmaxf(mx, fabsf(__bfloat162float(sc[size_t(row) * groups + g])));
  // the row factor goes through bf16 (the epilogue reads it in that type): divide by the rounded value
  const __nv_bfloat16 mb = __float2bfloat16(mx > 0.f ? mx : 1.f);
  const float m = __bfloat162float(mb);
  row_max[row] = mb;
  for (int g = 0; g < groups; ++g)
    rel[size_t(row) * groups + g] = __float2half(__bfloat162float(sc[size_t(row) * groups + g]) / m);
}

extern "C" int bl_w8_group_scales(const void* scales, int n, int groups, void* row_max, void* rel, void* stream,
                                  char* err, size_t errlen) {
  if (!scales || !row_max || !rel || n < 1 || groups < 1) {
    set_err(err, errlen, "barlink: w8_group_scales needs scales [n][groups] and two outputs");
    return -1;
  }
  k_w8_group_scales<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(scales), n, groups, static_cast<__nv_bfloat16*>(row_max),
      static_cast<__half*>(rel));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: w8_group_scales launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

extern "C" size_t bl_tiled_weight_bytes(int n, int k) {
  return size_t((n + kTileA - 1) / kTileA) * size_t((k + kTileK - 1) / kTileK) * (kTileA * kTileK * 2);
}

extern "C" int bl_tile_weight(const void* src, int n, int k, int ld, void* dst, void* stream, char* err,
                              size_t errlen) {
  if (!src || !dst || n < 1 || k < 1 || (reinterpret_cast<uintptr_t>(dst) & 15u)) {
    set_err(err, errlen, "barlink: tile_weight needs a source, and a destination aligned to 16 bytes");
    return -1;
  }
  const int tkb = (k + kTileK - 1) / kTileK;
  const size_t chunks = bl_tiled_weight_bytes(n, k) / 16;
  size_t blocks = (chunks + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  k_tile_weight<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<uint4*>(dst), n, k, ld, tkb, chunks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: tile_weight launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

extern "C" int bl_gemm_splits(int n, int k, int tokens) {
  if (tokens > 128) return 1;
  const int tiles = (n + kTileA - 1) / kTileA;
  const int kblocks = (k + kTileK - 1) / kTileK;
  return pick_splits(tiles, kblocks, sm_count(), 0);
}

// arrival counts (per owner) of a pushed linear: one per 128-row x 256-column tile of a CTA, in the
// paired kernel as in the single-CTA one (both are only taken with 256-column tiles)
extern "C" int bl_gemm_push_units(int rows, int n) {
  const int col_tiles = (n + 255) / 256;
  if (gemm_pair_enabled() && rows >= 512) return ((rows + 255) / 256) * 2 * col_tiles;  // two CTAs per 256-row unit
  return ((rows + kTileA - 1) / kTileA) * col_tiles;
}

extern "C" int bl_gemm_bf16(const blGemmArgs* a, void* stream, char* err, size_t errlen) {
  if (a && a->push) {
    if (a->swap || a->partial_out || a->peer || a->silu_mul || a->ldo != a->rb || (a->rb & 7) || a->rb < 256) {
      set_err(err, errlen, "barlink: a pushed linear is token-major, dense (ldo == n), n >= 256 and a multiple of 8");
      return -1;
    }
  }
  if (!a || !a->a || !a->b || (!a->out && !a->partial_out && !a->peer && !a->push) || a->ra < 1 || a->rb < 1 || a->k < 8 || (a->k & 7)) {
    set_err(err, errlen, "barlink: gemm needs non-null operands and K a multiple of 8");
    return -1;
  }
  if (a->i8 && ((a->k & 15) || a->weight_tiled || a->peer || a->push || a->gate_flags || a->partial_out)) {
    set_err(err, errlen, "barlink: the int8 product needs K a multiple of 16 and plain operands and output");
    return -1;
  }
  if (a->group_scale && (!a->i8 || !a->swap || a->rb > 64 || a->group_k < 128 || (a->group_k & 127) || a->feat_scale ||
                         (a->bn > 64))) {
    set_err(err, errlen, "barlink: per-group scales go with the int8 product, weights first, at most 64 tokens, groups of a multiple of 128");
    return -1;
  }
  if (!a->i8 && (a->feat_scale || a->tok_scale)) {
    set_err(err, errlen, "barlink: feat_scale / tok_scale belong to the int8 product");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->bn <= 0 && gemm_pair_ok(*a)) return launch_gemm_pair(*a, st, err, errlen);
  int bn = a->bn;
  if (bn <= 0) {
    if (a->swap) bn = a->rb <= 16 ? 16 : a->rb <= 32 ? 32 : a->rb <= 64 ? 64 : a->rb <= 128 ? 128 : 256;
    else bn = a->rb >= 256 ? 256 : a->rb > 64 ? 128 : 64;
  }
  static const int cps = env_int_or("BL_GEMM_CPS", 1);
  switch (bn) {
    case 16: return cps == 2 ? launch_gemm<16, 2>(*a, a->splits, st, err, errlen)
                             : launch_gemm<16, 1>(*a, a->splits, st, err, errlen);
    case 32: return cps == 2 ? launch_gemm<32, 2>(*a, a->splits, st, err, errlen)
                             : launch_gemm<32, 1>(*a, a->splits, st, err, errlen);
    case 64: return cps == 2 ? launch_gemm<64, 2>(*a, a->splits, st, err, errlen)
                             : launch_gemm<64, 1>(*a, a->splits, st, err, errlen);
    case 128: return launch_gemm<128, 1>(*a, a->splits, st, err, errlen);
    case 256: return launch_gemm<256, 1>(*a, a->splits, st, err, errlen);
    default:
      set_err(err, errlen, "barlink: gemm tile width %d not in {16,32,64,128,256}", bn);
      return -1;
  }
}
