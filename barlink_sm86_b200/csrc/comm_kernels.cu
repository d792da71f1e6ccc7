// SPDX-License-Identifier: MIT
//
// Collective kernels over peer memory (NVLink 5 / NVSwitch) and their
// launchers.  Every collective is ONE kernel: it stores into peers' arenas,
// signals with release stores at system scope, waits with bounded acquire
// loads, and reduces in fp32.  Expectations are device counters advanced by
// the kernel itself, so a captured CUDA graph can be replayed.
//
// Counterparts in the reference (torch_ext/barlink_sm86/core.cu): six-kernel
// arm-handshake allreduce :2957-3016 -> k_twoshot; fused <=64 KiB allreduce
// :2915-2955 -> k_lamport (one hop, data words are their own flags);
// p2p send/recv :3108-3209 -> k_p2p_send/k_p2p_recv; verify/readback
// :400-484 -> k_verify_*; new here: NVLS multimem allreduce, all-gather,
// reduce-scatter, broadcast, barrier, allreduce+residual+RMSNorm.
#include <cooperative_groups.h>
#include <cuda_fp8.h>
#include <stdio.h>
#include <string.h>

#include <type_traits>

#include "bl_ops.h"
#include "comm_dev.cuh"
#include "heap.h"
#include "launch.h"
#include "ptx.cuh"

namespace bl {

constexpr int kThreads = 512;
bool env_flag_set(const char* name);

struct CollArgs {
  CommPack pack;
  const void* in[kMaxRanks];
  void* out[kMaxRanks];
  const void* aux_in[kMaxRanks];
  void* aux_out[kMaxRanks];
  const void* gamma[kMaxRanks];
  size_t nvec;      // 16-byte vectors in the message (all-gather/reduce-scatter: per rank)
  size_t slice_stride;  // vectors between rank slices of the big operand (0: dense)
  int rows;         // fused norm: tokens
  int vec_per_row;  // fused norm: vectors per token
  float eps;
  int root;
  int peer;
  int mode;
  unsigned long long* bad;
  unsigned seed;
  int iters;
  int nsplit;    // fused norm: `in` is nsplit fp32 slabs (slab elements apart) to be summed first
  size_t slab;
};

// ---------------------------------------------------------------------------
// barrier
// ---------------------------------------------------------------------------
__global__ void k_barrier(CollArgs a) {
  const Comm& c = comm_of(a.pack);
  uint32_t* s = sig_of(c, c.rank);
  const uint32_t e = ld_volatile_u32(&s[sig_epoch(P_BARRIER)]);
  block_sync_peers(c, P_BARRIER, 0, e + 1);
  finish_epoch(c, P_BARRIER, e, 0, false);
}

// ---------------------------------------------------------------------------
// one-shot all-reduce, data words are their own arrival flags.
// Three inbox buffers rotate by epoch: peers write buffer e%3 during call e,
// buffer (e+2)%3 (used by call e-1, fully consumed when call e starts) is
// reset to "unwritten" for call e+2.  No flag round trip: one NVLink hop.
// kNorm: the reduced row gets the residual added, is written out, and its
// RMSNorm (weight gamma) is written to a second output.
// ---------------------------------------------------------------------------
template <int DT, bool kNorm>
__global__ void __launch_bounds__(kThreads) k_lamport(CollArgs a) {
  using E = Elem<DT>;
  // Launched as a programmatic dependent in peer mode: the kernel after this
  // one (a GEMM) may become resident now and stream its first weight tiles
  // while this kernel waits for the peers; this kernel itself reads nothing
  // before its predecessors have completed.
  pdl_launch_dependents();
  pdl_wait();
  const Comm& c = comm_of(a.pack);
  const int y = a.pack.emu ? blockIdx.y : 0;
  const int rank = c.rank, world = c.world;
  uint32_t* s = sig_of(c, rank);
  const uint32_t e = ld_volatile_u32(&s[sig_epoch(P_LAMPORT)]);
  const uint32_t prev_vecs = ld_volatile_u32(&s[sig_aux(P_LAMPORT)]);
  const size_t buf_bytes = size_t(world) * c.lamport_slice;
  const size_t cur_off = c.lamport_off + size_t(e % 3u) * buf_bytes;
  const size_t clr_off = c.lamport_off + size_t((e + 2u) % 3u) * buf_bytes;
  const uint4* in = static_cast<const uint4*>(a.in[y]);
  uint4* out = static_cast<uint4*>(a.out[y]);
  const size_t nvec = a.nvec;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  bool ok = true;

  if constexpr (!kNorm) {
    // push my vectors into every peer's inbox slot [rank]
    for (size_t i = first; i < nvec; i += stride) {
      uint4 v = scrub(in[i]);
#pragma unroll 1
      for (int k = 1; k < world; ++k) {
        int p = rank + k;
        if (p >= world) p -= world;
        st_v4(c.base[p] + cur_off + size_t(rank) * c.lamport_slice + i * 16, v);
      }
    }
    // reset the buffer that call e-1 used
    const uint4 unw = make_uint4(kUnwritten, kUnwritten, kUnwritten, kUnwritten);
    for (size_t i = first; i < prev_vecs; i += stride)
      for (int r = 0; r < world; ++r)
        if (r != rank) st_v4(c.base[rank] + clr_off + size_t(r) * c.lamport_slice + i * 16, unw);
    // gather + reduce in rank order (same order on every rank: same bits)
    for (size_t i = first; i < nvec && ok; i += stride) {
      typename E::acc_t acc[E::N];
#pragma unroll
      for (int j = 0; j < E::N; ++j) acc[j] = 0;
      // all ranks' vectors are requested before the first one is looked at: one round trip to L2
      // instead of one per rank; whatever has not landed yet is polled afterwards
      uint4 got[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world)
          got[r] = r == rank ? scrub(in[i])
                             : ld_volatile_v4(c.base[rank] + cur_off + size_t(r) * c.lamport_slice + i * 16);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world && ok) {
          uint4 v = got[r];
          if (r != rank && !landed(v) &&
              !poll_vec(c, c.base[rank] + cur_off + size_t(r) * c.lamport_slice + i * 16, v, r))
            ok = false;
          acc_add<DT>(acc, v);
        }
      if (ok) out[i] = E::pack(acc);
    }
  } else {
    constexpr int kMaxVpt = 4;
    __shared__ float s_part[kThreads / 32];
    __shared__ float s_rstd;
    const int vpr = a.vec_per_row;
    // the row-parallel linear before this kernel may have left k-split slabs:
    // their sum, rounded to the storage type, is this rank's contribution
    const float* slabs = a.nsplit > 0 ? static_cast<const float*>(a.in[y]) : nullptr;
    auto load_in = [&](size_t g) -> uint4 {
      if (!slabs) return scrub(in[g]);
      float acc[E::N];
#pragma unroll
      for (int j = 0; j < E::N; ++j) acc[j] = 0.f;
      if constexpr (E::N == 8) {
        float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        sum_slabs8(slabs + g * 8, a.slab, a.nsplit, a8);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = a8[j];
      }
      return scrub(E::pack(acc));
    };
    const uint4* res_in = static_cast<const uint4*>(a.aux_in[y]);
    uint4* res_out = static_cast<uint4*>(a.aux_out[y]);
    const uint4* gamma = static_cast<const uint4*>(a.gamma[y]);
    // push all my rows first so that every peer's gather overlaps
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x)
      for (int i = threadIdx.x; i < vpr; i += blockDim.x) {
        const size_t g = size_t(row) * vpr + i;
        uint4 v = load_in(g);
        if (slabs) st_v4(c.base[rank] + cur_off + size_t(rank) * c.lamport_slice + g * 16, v);
#pragma unroll 1
        for (int k = 1; k < world; ++k) {
          int p = rank + k;
          if (p >= world) p -= world;
          st_v4(c.base[p] + cur_off + size_t(rank) * c.lamport_slice + g * 16, v);
        }
      }
    const uint4 unw = make_uint4(kUnwritten, kUnwritten, kUnwritten, kUnwritten);
    for (size_t i = first; i < prev_vecs; i += stride)
      for (int r = 0; r < world; ++r)
        if (r != rank) st_v4(c.base[rank] + clr_off + size_t(r) * c.lamport_slice + i * 16, unw);

    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
      float x[kMaxVpt][E::N];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < kMaxVpt; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < vpr && ok) {
          const size_t g = size_t(row) * vpr + i;
          float acc[E::N];
#pragma unroll
          for (int j = 0; j < E::N; ++j) acc[j] = 0.f;
          // all ranks' vectors (and the residual) are requested before the first one is looked
          // at; whatever has not landed yet is polled afterwards
          uint4 got[kMaxRanks];
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < world) {
              // with slabs, my own contribution was parked in my inbox slot by this same thread
              got[r] = (r == rank && !slabs)
                           ? scrub(in[g])
                           : ld_volatile_v4(c.base[rank] + cur_off + size_t(r) * c.lamport_slice + g * 16);
            }
          uint4 resv = make_uint4(0, 0, 0, 0);
          if (res_in) resv = res_in[g];
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < world && ok) {
              uint4 v = got[r];
              if (r != rank && !landed(v) &&
                  !poll_vec(c, c.base[rank] + cur_off + size_t(r) * c.lamport_slice + g * 16, v, r))
                ok = false;
              acc_add<DT>(acc, v);
            }
          if (res_in) {
            // the all-reduce result is rounded to the storage type first,
            // exactly as an unfused all_reduce followed by an add would
            uint4 rv = E::pack(acc);
            E::unpack(rv, acc);
            acc_add<DT>(acc, resv);
          }
          uint4 packed = E::pack(acc);
          if (ok) res_out[g] = packed;
          E::unpack(packed, x[k]);  // the norm sees the rounded residual
#pragma unroll
          for (int j = 0; j < E::N; ++j) ss += x[k][j] * x[k][j];
        }
      }
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) s_rstd = rsqrtf(t / float(vpr * E::N) + a.eps);
      }
      __syncthreads();
      const float rstd = s_rstd;
#pragma unroll
      for (int k = 0; k < kMaxVpt; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < vpr && ok) {
          float gmm[E::N];
          E::unpack(gamma[i], gmm);
          float o[E::N];
#pragma unroll
          for (int j = 0; j < E::N; ++j) {
            // x*rstd is rounded to the storage type before the weight multiply,
            // the order a framework's RMSNorm module uses
            o[j] = x[k][j] * rstd;
          }
          uint4 t = E::pack(o);
          E::unpack(t, o);
#pragma unroll
          for (int j = 0; j < E::N; ++j) o[j] *= gmm[j];
          out[size_t(row) * vpr + i] = E::pack(o);
        }
      }
      __syncthreads();
    }
  }
  finish_epoch(c, P_LAMPORT, e, uint32_t(nvec), true);
}

// ---------------------------------------------------------------------------
// flag-based push collectives through the staging zone.
//   mode 0 all-reduce (two-shot: reduce-scatter then all-gather)
//   mode 1 reduce-scatter     (in: world slices of nvec, out: nvec)
//   mode 2 all-gather         (in: nvec, out: world slices of nvec)
//   mode 3 broadcast from root (in == out, nvec)
//   mode 4 all-reduce whose scatter was done by the GEMM that produced the data (its epilogue
//          stored every tile into the owners' inboxes and bumped their arrival counters): wait
//          for a.iters arrivals from every rank, then reduce + all-gather as in mode 0
// Block b owns, inside every slice, the vector indices (b + k*grid)*T + t.
// A block only ever consumes what block b of a peer produced, so blocks
// synchronise with their namesakes only (slot = blockIdx.x).
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kThreads) k_staged(CollArgs a) {
  using E = Elem<DT>;
  const Comm& c = comm_of(a.pack);
  const int y = a.pack.emu ? blockIdx.y : 0;
  const int rank = c.rank, world = c.world;
  const int mode = a.mode;
  const int proto = mode == 0 ? P_TWOSHOT : mode == 1 ? P_REDSCAT : mode == 2 ? P_ALLGATHER
                    : mode == 3 ? P_BCAST : P_ROWPUSH;
  uint32_t* s = sig_of(c, rank);
  const uint32_t e = ld_volatile_u32(&s[sig_epoch(proto)]);
  const uint4* in = static_cast<const uint4*>(a.in[y]);
  uint4* out = static_cast<uint4*>(a.out[y]);
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // slice geometry
  size_t sv;  // vectors per slice
  size_t total;
  if (mode == 0 || mode == 4) {
    total = a.nvec;
    sv = (a.nvec + world - 1) / world;
  } else {
    sv = a.nvec;
    total = a.nvec * world;
  }
  const size_t bs = (mode == 0 || mode == 4 || a.slice_stride == 0) ? sv : a.slice_stride;  // big-operand pitch
  auto slice_len = [&](int r) -> size_t {
    size_t b = size_t(r) * sv;
    return b >= total ? 0 : (total - b < sv ? total - b : sv);
  };
  const size_t sbuf = stage_buf_off(c);
  char* my_stage = c.base[rank] + sbuf;
  const size_t half = size_t(world) * c.stage_slice;  // inbox half, then outbox half
  bool ok = true;

  uint32_t push_cum = 0;
  if (mode == 4) {
    // the producers' tiles: every rank's arrival word must reach the running total
    __shared__ int s_ok4;
    push_cum = ld_volatile_u32(&s[sig_aux(P_ROWPUSH)]);
    if (threadIdx.x == 0) s_ok4 = 1;
    __syncthreads();
    if (threadIdx.x < world &&
        !wait_flag(c, s + sig_flag(P_ROWPUSH, kMaxSlots - 1, threadIdx.x), push_cum + uint32_t(a.iters), P_ROWPUSH, threadIdx.x))
      s_ok4 = 0;
    __syncthreads();
    ok = s_ok4 != 0;
    if (ok) {
      const size_t len = slice_len(rank);
      for (size_t j = first; j < len; j += stride) {
        typename E::acc_t acc[E::N];
#pragma unroll
        for (int q = 0; q < E::N; ++q) acc[q] = 0;
        for (int r = 0; r < world; ++r) acc_add<DT>(acc, ld_volatile_v4(my_stage + size_t(r) * c.stage_slice + j * 16));
        const uint4 res = E::pack(acc);
        out[size_t(rank) * sv + j] = res;
        for (int k = 1; k < world; ++k) {
          int p = rank + k;
          if (p >= world) p -= world;
          st_v4(c.base[p] + sbuf + half + size_t(rank) * c.stage_slice + j * 16, res);
        }
      }
    }
  } else if (mode == 0 || mode == 1) {
    // scatter: slice p of my input goes to rank p's inbox [rank]
    for (int k = 1; k < world; ++k) {
      int p = rank + k;
      if (p >= world) p -= world;
      const size_t len = slice_len(p);
      char* dst = c.base[p] + sbuf + size_t(rank) * c.stage_slice;
      for (size_t j = first; j < len; j += stride) st_v4(dst + j * 16, in[size_t(p) * bs + j]);
    }
    ok = block_sync_peers(c, proto, blockIdx.x, e * 4 + 1);
    if (ok) {
      const size_t len = slice_len(rank);
      for (size_t j = first; j < len; j += stride) {
        typename E::acc_t acc[E::N];
#pragma unroll
        for (int q = 0; q < E::N; ++q) acc[q] = 0;
        for (int r = 0; r < world; ++r) {
          uint4 v = r == rank ? in[size_t(rank) * bs + j]
                              : ld_volatile_v4(my_stage + size_t(r) * c.stage_slice + j * 16);
          acc_add<DT>(acc, v);
        }
        const uint4 res = E::pack(acc);
        if (mode == 1) {
          out[j] = res;
        } else {
          out[size_t(rank) * sv + j] = res;
          for (int k = 1; k < world; ++k) {
            int p = rank + k;
            if (p >= world) p -= world;
            st_v4(c.base[p] + sbuf + half + size_t(rank) * c.stage_slice + j * 16, res);
          }
        }
      }
    }
  } else if (mode == 2) {
    for (size_t j = first; j < sv; j += stride) {
      const uint4 v = in[j];
      out[size_t(rank) * bs + j] = v;
      for (int k = 1; k < world; ++k) {
        int p = rank + k;
        if (p >= world) p -= world;
        st_v4(c.base[p] + sbuf + half + size_t(rank) * c.stage_slice + j * 16, v);
      }
    }
  } else {
    if (rank == a.root)
      for (size_t j = first; j < sv; j += stride) {
        const uint4 v = in[j];
        for (int k = 1; k < world; ++k) {
          int p = rank + k;
          if (p >= world) p -= world;
          st_v4(c.base[p] + sbuf + half + size_t(rank) * c.stage_slice + j * 16, v);
        }
      }
  }
  if (mode != 1) {
    if (ok) ok = block_sync_peers(c, proto, blockIdx.x, e * 4 + 2);
    if (ok) {
      if (mode == 3) {
        if (rank != a.root)
          for (size_t j = first; j < sv; j += stride)
            out[j] = ld_volatile_v4(my_stage + half + size_t(a.root) * c.stage_slice + j * 16);
      } else {
        for (int r = 0; r < world; ++r) {
          if (r == rank) continue;
          const size_t len = (mode == 0 || mode == 4) ? slice_len(r) : sv;
          const char* src = my_stage + half + size_t(r) * c.stage_slice;
          for (size_t j = first; j < len; j += stride)
            out[size_t(r) * bs + j] = ld_volatile_v4(src + j * 16);
        }
      }
    }
  }
  finish_epoch(c, proto, e, push_cum + uint32_t(a.iters), mode == 4, true);
}

// ---------------------------------------------------------------------------
// NVLS all-reduce: stage into the multicast-bound arena, let the switch
// reduce my slice (multimem.ld_reduce) and replicate it (multimem.st).
// ---------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ uint4 mm_ld_reduce(const void* p) {
  if constexpr (DT == BL_DTYPE_BF16) return multimem_ld_reduce_bf16x8(p);
  else if constexpr (DT == BL_DTYPE_FP16) return multimem_ld_reduce_f16x8(p);
  else return multimem_ld_reduce_f32x4(p);
}

template <int DT>
__global__ void __launch_bounds__(kThreads) k_nvls(CollArgs a) {
  const Comm& c = comm_of(a.pack);
  const int rank = c.rank, world = c.world;
  uint32_t* s = sig_of(c, rank);
  const uint32_t e = ld_volatile_u32(&s[sig_epoch(P_NVLS)]);
  const uint4* in = static_cast<const uint4*>(a.in[0]);
  uint4* out = static_cast<uint4*>(a.out[0]);
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = a.nvec;
  const size_t sv = (total + world - 1) / world;
  auto slice_len = [&](int r) -> size_t {
    size_t b = size_t(r) * sv;
    return b >= total ? 0 : (total - b < sv ? total - b : sv);
  };
  const size_t sbuf = stage_buf_off(c);
  char* stage = c.base[rank] + sbuf;
  char* mstage = c.mc + sbuf;
  for (int r = 0; r < world; ++r) {
    const size_t len = slice_len(r);
    for (size_t j = first; j < len; j += stride)
      st_v4(stage + (size_t(r) * sv + j) * 16, in[size_t(r) * sv + j]);
  }
  __threadfence_system();
  bool ok = block_sync_peers(c, P_NVLS, blockIdx.x, e * 4 + 1);
  if (ok) {
    const size_t len = slice_len(rank);
    for (size_t j = first; j < len; j += stride) {
      const size_t o = (size_t(rank) * sv + j) * 16;
      const uint4 v = mm_ld_reduce<DT>(mstage + o);
      multimem_st_v4(mstage + o, v);
    }
    __threadfence_system();
    ok = block_sync_peers(c, P_NVLS, blockIdx.x, e * 4 + 2);
  }
  if (ok)
    for (int r = 0; r < world; ++r) {
      const size_t len = slice_len(r);
      for (size_t j = first; j < len; j += stride)
        out[size_t(r) * sv + j] = ld_volatile_v4(stage + (size_t(r) * sv + j) * 16);
    }
  finish_epoch(c, P_NVLS, e, 0, false, true);
}

// ---------------------------------------------------------------------------
// point to point: per-pair inbox, data flag at the receiver, consumed
// receipt at the sender (posted after the receiver finished reading).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) k_p2p_send(CollArgs a) {
  const Comm& c = comm_of(a.pack);
  const int y = a.pack.emu ? blockIdx.y : 0;
  const int rank = c.rank, peer = a.peer;
  uint32_t* s = sig_of(c, rank);
  const uint32_t ord = ld_volatile_u32(&s[sig_p2p_send(peer)]) + 1;
  __shared__ int s_ok;
  if (threadIdx.x == 0)
    s_ok = wait_flag(c, s + sig_flag(P_P2P_RCPT, 0, peer), ord - 1, P_P2P_RCPT, peer) ? 1 : 0;
  __syncthreads();
  if (s_ok) {
    const uint4* in = static_cast<const uint4*>(a.in[y]);
    char* dst = c.base[peer] + c.p2p_off + size_t(rank) * c.p2p_slice;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < a.nvec;
         i += size_t(gridDim.x) * blockDim.x)
      st_v4(dst + i * 16, in[i]);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t t = atomicAdd(&s[sig_ticket(P_P2P_DATA)], 1u);
    if (t == gridDim.x - 1) {
      s[sig_ticket(P_P2P_DATA)] = 0;
      __threadfence_system();
      if (s_ok) st_release_sys(sig_of(c, peer) + sig_flag(P_P2P_DATA, 0, rank), ord);
      *reinterpret_cast<volatile uint32_t*>(&s[sig_p2p_send(peer)]) = ord;
    }
  }
}

__global__ void __launch_bounds__(kThreads) k_p2p_recv(CollArgs a) {
  const Comm& c = comm_of(a.pack);
  const int y = a.pack.emu ? blockIdx.y : 0;
  const int rank = c.rank, peer = a.peer;
  uint32_t* s = sig_of(c, rank);
  const uint32_t ord = ld_volatile_u32(&s[sig_p2p_recv(peer)]) + 1;
  __shared__ int s_ok;
  if (threadIdx.x == 0)
    s_ok = wait_flag(c, s + sig_flag(P_P2P_DATA, 0, peer), ord, P_P2P_DATA, peer) ? 1 : 0;
  __syncthreads();
  if (s_ok) {
    uint4* out = static_cast<uint4*>(a.out[y]);
    const char* src = c.base[rank] + c.p2p_off + size_t(peer) * c.p2p_slice;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < a.nvec;
         i += size_t(gridDim.x) * blockDim.x)
      out[i] = ld_volatile_v4(src + i * 16);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t t = atomicAdd(&s[sig_ticket(P_P2P_RCPT)], 1u);
    if (t == gridDim.x - 1) {
      s[sig_ticket(P_P2P_RCPT)] = 0;
      __threadfence_system();
      if (s_ok) st_release_sys(sig_of(c, peer) + sig_flag(P_P2P_RCPT, 0, rank), ord);
      *reinterpret_cast<volatile uint32_t*>(&s[sig_p2p_recv(peer)]) = ord;
    }
  }
}

// ---------------------------------------------------------------------------
// byte proof of every path: pattern through each peer mapping (and through
// the multicast mapping), verified by the owner from its own memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pat_word(uint32_t src, uint32_t dst, uint64_t word, uint32_t seed) {
  uint64_t x = word * 0x9E3779B97F4A7C15ull + (uint64_t(src) << 40) + (uint64_t(dst) << 48) + seed;
  x ^= x >> 29;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 32;
  return uint32_t(x);
}
__device__ __forceinline__ uint4 pat_vec(uint32_t src, uint32_t dst, size_t i, uint32_t seed) {
  return make_uint4(pat_word(src, dst, i * 4, seed), pat_word(src, dst, i * 4 + 1, seed),
                    pat_word(src, dst, i * 4 + 2, seed), pat_word(src, dst, i * 4 + 3, seed));
}
__device__ __forceinline__ uint32_t bad_bytes(uint4 a, uint4 b) {
  uint32_t n = 0;
  const uint32_t x[4] = {a.x ^ b.x, a.y ^ b.y, a.z ^ b.z, a.w ^ b.w};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) n += ((x[i] >> (8 * j)) & 0xffu) ? 1u : 0u;
  return n;
}

__global__ void __launch_bounds__(kThreads) k_verify(CollArgs a) {
  const Comm& c = comm_of(a.pack);
  const int rank = c.rank, world = c.world;
  uint32_t* s = sig_of(c, rank);
  const uint32_t e = ld_volatile_u32(&s[sig_epoch(P_VERIFY)]);
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t half = size_t(world) * c.stage_slice;
  const size_t sbuf = stage_buf_off(c);
  for (int p = 0; p < world; ++p) {
    char* dst = c.base[p] + sbuf + size_t(rank) * c.stage_slice;
    for (size_t i = first; i < a.nvec; i += stride) st_v4(dst + i * 16, pat_vec(rank, p, i, a.seed));
  }
  if (c.mc) {
    char* dst = c.mc + sbuf + half + size_t(rank) * c.stage_slice;
    for (size_t i = first; i < a.nvec; i += stride)
      multimem_st_v4(dst + i * 16, pat_vec(rank, 255, i, a.seed));
    __threadfence_system();
  }
  bool ok = block_sync_peers(c, P_VERIFY, blockIdx.x, e * 4 + 1);
  unsigned long long bad = 0;
  if (ok) {
    for (int r = 0; r < world; ++r) {
      const char* src = c.base[rank] + sbuf + size_t(r) * c.stage_slice;
      for (size_t i = first; i < a.nvec; i += stride)
        bad += bad_bytes(ld_volatile_v4(src + i * 16), pat_vec(r, rank, i, a.seed));
      if (c.mc) {
        const char* m = c.base[rank] + sbuf + half + size_t(r) * c.stage_slice;
        for (size_t i = first; i < a.nvec; i += stride)
          bad += bad_bytes(ld_volatile_v4(m + i * 16), pat_vec(r, 255, i, a.seed));
      }
    }
  } else {
    bad = (threadIdx.x == 0) ? a.nvec * 16 : 0;
  }
  if (bad) atomicAdd_system(a.bad, bad);
  // nobody may start the next pattern before everyone has checked this one
  if (ok) block_sync_peers(c, P_VERIFY, blockIdx.x, e * 4 + 2);
  finish_epoch(c, P_VERIFY, e, 0, false, true);
}

__global__ void k_probe(CollArgs a, unsigned long long* res) {
  const Comm& c = comm_of(a.pack);
  const int rank = c.rank;
  if (c.world < 2 || rank > 1 || threadIdx.x != 0) return;
  uint32_t* s = sig_of(c, rank);
  const uint32_t e0 = ld_volatile_u32(&s[sig_epoch(P_PROBE)]);
  const int peer = 1 - rank;
  uint32_t* mine = s + sig_flag(P_PROBE, 0, peer);
  uint32_t* theirs = sig_of(c, peer) + sig_flag(P_PROBE, 0, rank);
  bool ok = true;
  uint64_t t0 = globaltimer_ns();
  for (int i = 1; i <= a.iters && ok; ++i) {
    const uint32_t v = e0 + uint32_t(i);
    if (rank == 0) {
      st_release_sys(theirs, v);
      ok = wait_flag(c, mine, v, P_PROBE, peer);
    } else {
      ok = wait_flag(c, mine, v, P_PROBE, peer);
      st_release_sys(theirs, v);
    }
  }
  uint64_t t1 = globaltimer_ns();
  res[0] = ok ? (t1 - t0) / uint64_t(a.iters > 0 ? a.iters : 1) : ~0ull;
  *reinterpret_cast<volatile uint32_t*>(&s[sig_epoch(P_PROBE)]) = e0 + uint32_t(a.iters);
}

__global__ void k_empty() {}

__global__ void k_fill_u32(uint32_t* p, size_t n, uint32_t v) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    p[i] = v;
}

__global__ void k_copy_vec(const uint4* src, uint4* dst, size_t nvec) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += size_t(gridDim.x) * blockDim.x)
    dst[i] = ld_volatile_v4(src + i);
}

// ---------------------------------------------------------------------------
// second half of the fused row-parallel linear: reduce my tokens' partial rows
// that every rank's GEMM epilogue stored into my inbox, add the residual,
// RMS-normalise and all-gather the result by storing it into every rank's
// gather buffer.  One block per local token.
// ---------------------------------------------------------------------------
struct RsFinishArgs {
  Comm c;
  size_t inbox_off, gather_off;
  int tpr, n, splits, units;
  const uint4* residual_in;
  uint4* residual_out;
  const uint4* gamma;
  float eps;
};

__global__ void __launch_bounds__(kThreads) k_rs_finish(RsFinishArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const Comm& c = a.c;
  const int rank = c.rank, world = c.world;
  __shared__ int s_ok;
  __shared__ float s_part[kThreads / 32];
  __shared__ float s_rstd;
  uint32_t* s = sig_of(c, rank);
  const uint32_t cum = ld_volatile_u32(&s[sig_aux(P_GEMM_RS)]);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world)
    if (!wait_flag(c, s + sig_flag(P_GEMM_RS, 0, threadIdx.x), cum + uint32_t(a.units), P_GEMM_RS,
                   threadIdx.x))
      s_ok = 0;
  __syncthreads();
  const int lm = blockIdx.x;
  const int vpr = a.n / 8;
  constexpr int kMaxVpt = 4;
  float x[kMaxVpt][8];
  float ss = 0.f;
  const float* inbox = reinterpret_cast<const float*>(c.base[rank] + a.inbox_off);
  if (s_ok) {
#pragma unroll
    for (int k = 0; k < kMaxVpt; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < vpr) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // world x splits partial rows, summed in (rank, split) order
        sum_slabs8(inbox + size_t(lm) * a.n + i * 8, size_t(a.tpr) * a.n, world * a.splits, acc);
        using E = Elem<BL_DTYPE_BF16>;
        uint4 packed = E::pack(acc);  // the linear's output, rounded as an unfused linear would
        if (a.residual_in) {
          E::unpack(packed, acc);
          acc_add<BL_DTYPE_BF16>(acc, a.residual_in[size_t(lm) * vpr + i]);
          packed = E::pack(acc);
        }
        a.residual_out[size_t(lm) * vpr + i] = packed;
        E::unpack(packed, x[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[k][j] * x[k][j];
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_rstd = rsqrtf(t / float(a.n) + a.eps);
  }
  __syncthreads();
  const float rstd = s_rstd;
  const int token = rank * a.tpr + lm;
  if (s_ok) {
#pragma unroll
    for (int k = 0; k < kMaxVpt; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < vpr) {
        using E = Elem<BL_DTYPE_BF16>;
        float gmm[8], o[8];
        E::unpack(a.gamma[i], gmm);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = x[k][j] * rstd;
        uint4 t = E::pack(o);
        E::unpack(t, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= gmm[j];
        const uint4 res = E::pack(o);
        const size_t off = a.gather_off + (size_t(token) * vpr + i) * 16;
        for (int kk = 0; kk < world; ++kk) {
          int p = rank + kk;
          if (p >= world) p -= world;
          st_v4(c.base[p] + off, res);
        }
      }
    }
  }
  // my row is in every rank's gather buffer: tell them
  __syncthreads();
  if (threadIdx.x < world && s_ok) {
    __threadfence_system();
    red_release_sys_add(sig_of(c, threadIdx.x) + sig_flag(P_AG_GEMM, 0, rank), 1u);
  }
  // the last block moves the arrival expectation forward
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&s[sig_ticket(P_GEMM_RS)], 1u);
    if (t == gridDim.x - 1) {
      s[sig_ticket(P_GEMM_RS)] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&s[sig_aux(P_GEMM_RS)]) = cum + uint32_t(a.units);
    }
  }
}

// ---------------------------------------------------------------------------
// host: device state
// ---------------------------------------------------------------------------
#define RT_TRY(call, what)                                                       \
  do {                                                                           \
    cudaError_t _e = (call);                                                     \
    if (_e != cudaSuccess) {                                                     \
      set_err(err, errlen, "barlink: %s failed: %s", what, cudaGetErrorString(_e)); \
      return -1;                                                                 \
    }                                                                            \
  } while (0)

static int upload_comms(blCtx* ctx, char* err, size_t errlen) {
  if (ctx->peer_mode) return 0;
  for (int g = 0; g < ctx->ngroups; ++g) {
    Comm tmp[kMaxRanks];
    for (int i = 0; i < ctx->group_n[g]; ++i) tmp[i] = ctx->comm_for(ctx->group_ranks[g][i]);
    RT_TRY(cudaSetDevice(ctx->group_dev[g]), "cudaSetDevice");
    RT_TRY(cudaMemcpy(ctx->group_dcomms[g], tmp, sizeof(Comm) * ctx->group_n[g],
                      cudaMemcpyHostToDevice),
           "comm upload");
  }
  return 0;
}

int init_device_state(blCtx* ctx, char* err, size_t errlen) {
  int cur = 0;
  cudaGetDevice(&cur);
  const int nloc = ctx->local_ranks();
  RT_TRY(cudaHostAlloc(reinterpret_cast<void**>(&ctx->h_status), sizeof(blStatus) * kMaxRanks,
                       cudaHostAllocMapped | cudaHostAllocPortable),
         "status block");
  memset(ctx->h_status, 0, sizeof(blStatus) * kMaxRanks);
  RT_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->d_status), ctx->h_status, 0),
         "status alias");
  RT_TRY(cudaHostAlloc(reinterpret_cast<void**>(&ctx->d_bad), sizeof(unsigned long long) * 8,
                       cudaHostAllocMapped | cudaHostAllocPortable),
         "verify counter");
  memset(ctx->d_bad, 0, sizeof(unsigned long long) * 8);
  for (int l = 0; l < nloc; ++l) {
    const int r = ctx->peer_mode ? ctx->rank : l;
    RT_TRY(cudaSetDevice(ctx->arena[r].device), "cudaSetDevice");
    char* base = reinterpret_cast<char*>(ctx->arena[r].va);
    RT_TRY(cudaMemset(base + ctx->layout.sig_off, 0, kSigBytes), "signal pad clear");
    const size_t lam_words = 3 * size_t(ctx->world) * ctx->layout.lamport_slice / 4;
    k_fill_u32<<<256, 256>>>(reinterpret_cast<uint32_t*>(base + ctx->layout.lamport_off), lam_words,
                             kUnwritten);
    RT_TRY(cudaGetLastError(), "inbox fill launch");
    RT_TRY(cudaDeviceSynchronize(), "inbox fill");
  }
  if (!ctx->peer_mode) {
    ctx->ngroups = 0;
    for (int r = 0; r < ctx->world; ++r) {
      int g = -1;
      for (int i = 0; i < ctx->ngroups; ++i)
        if (ctx->group_dev[i] == ctx->arena[r].device) g = i;
      if (g < 0) {
        g = ctx->ngroups++;
        ctx->group_dev[g] = ctx->arena[r].device;
        ctx->group_n[g] = 0;
      }
      ctx->group_ranks[g][ctx->group_n[g]++] = r;
    }
    for (int g = 0; g < ctx->ngroups; ++g) {
      RT_TRY(cudaSetDevice(ctx->group_dev[g]), "cudaSetDevice");
      RT_TRY(cudaMalloc(reinterpret_cast<void**>(&ctx->group_dcomms[g]), sizeof(Comm) * kMaxRanks),
             "comm table");
    }
    if (upload_comms(ctx, err, errlen) != 0) return -1;
  } else {
    RT_TRY(cudaSetDevice(ctx->arena[ctx->rank].device), "cudaSetDevice");
    RT_TRY(cudaStreamCreateWithFlags(&ctx->send_stream, cudaStreamNonBlocking), "send stream");
    RT_TRY(cudaEventCreateWithFlags(&ctx->ev_caller, cudaEventDisableTiming), "event");
    RT_TRY(cudaEventCreateWithFlags(&ctx->ev_send, cudaEventDisableTiming), "event");
  }
  cudaSetDevice(cur);
  return 0;
}

void free_device_state(blCtx* ctx) {
  for (int g = 0; g < ctx->ngroups; ++g)
    if (ctx->group_dcomms[g]) {
      cudaSetDevice(ctx->group_dev[g]);
      cudaFree(ctx->group_dcomms[g]);
      ctx->group_dcomms[g] = nullptr;
    }
  if (ctx->send_stream) cudaStreamDestroy(ctx->send_stream);
  if (ctx->ev_caller) cudaEventDestroy(ctx->ev_caller);
  if (ctx->ev_send) cudaEventDestroy(ctx->ev_send);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  if (ctx->d_bad) cudaFreeHost(ctx->d_bad);
  ctx->send_stream = nullptr;
  ctx->ev_caller = ctx->ev_send = nullptr;
  ctx->h_status = nullptr;
  ctx->d_status = nullptr;
  ctx->d_bad = nullptr;
}

// ---------------------------------------------------------------------------
// host: launching one collective on every local rank
// ---------------------------------------------------------------------------
struct PerRank {
  const void* in = nullptr;
  void* out = nullptr;
  const void* aux_in = nullptr;
  void* aux_out = nullptr;
  const void* gamma = nullptr;
  void* stream = nullptr;
};

static int check_health(blCtx* ctx, char* err, size_t errlen) {
  const int nloc = ctx->local_ranks();
  for (int l = 0; l < nloc; ++l) {
    const volatile blStatus* st = ctx->h_status + l;
    if (st->code != 0) {
      set_err(err, errlen,
              "barlink: an earlier device wait ran out (code %u, protocol %u, waiting for rank %u, "
              "had %u wanted %u); the link state is out of step -- call reset on every rank or "
              "restart the job",
              st->code, st->proto, st->from_rank, st->have, st->want);
      ctx->stats[BL_STAT_TIMEOUTS]++;
      return -1;
    }
  }
  return 0;
}

template <typename K>
static int launch_local(blCtx* ctx, K kernel, CollArgs base, const PerRank* pr, int grid_x,
                        int threads, char* err, size_t errlen, bool join_sends = true, bool pdl = false) {
  if (ctx->peer_mode) {
    // collectives are ordered after every send issued so far
    if (join_sends && ctx->send_pending) {
      cudaStream_t cs = static_cast<cudaStream_t>(pr[0].stream);
      cudaStreamCaptureStatus cst = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(cs, &cst) == cudaSuccess && cst == cudaStreamCaptureStatusNone) {
        cudaStreamWaitEvent(cs, ctx->ev_send, 0);
        ctx->send_pending = false;
      }
      cudaGetLastError();
    }
    CollArgs a = base;
    a.pack.c = ctx->comm_for(ctx->rank);
    a.pack.emu = nullptr;
    a.in[0] = pr[0].in;
    a.out[0] = pr[0].out;
    a.aux_in[0] = pr[0].aux_in;
    a.aux_out[0] = pr[0].aux_out;
    a.gamma[0] = pr[0].gamma;
    static const bool ar_pdl = [] {
      const char* e = getenv("BL_AR_PDL");  // 0: plain stream order for the collective kernels
      return !(e && e[0] == '0');
    }();
    if (pdl && ar_pdl) {
      // only for kernels that execute griddepcontrol.wait before their first read
      RT_TRY(launch_k(kernel, dim3(grid_x, 1, 1), dim3(threads, 1, 1), 0,
                      static_cast<cudaStream_t>(pr[0].stream), a),
             "collective launch");
    } else {
      kernel<<<dim3(grid_x, 1, 1), threads, 0, static_cast<cudaStream_t>(pr[0].stream)>>>(a);
    }
    RT_TRY(cudaGetLastError(), "collective launch");
    // BL_CAPDBG=1 (the reference's per-launch error bisect, torch_ext/barlink_sm86/core.cu:2726-2736):
    // wait for every collective kernel and report the first one that fails; off while capturing
    static const bool capdbg = env_flag_set("BL_CAPDBG");
    if (capdbg) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      cudaStream_t st = static_cast<cudaStream_t>(pr[0].stream);
      if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) {
        const cudaError_t e = cudaStreamSynchronize(st);
        fprintf(stderr, "[barlink capdbg] rank %d collective kernel (grid %d): %s\n", ctx->rank, grid_x,
                cudaGetErrorString(e));
        RT_TRY(e, "collective kernel");
      }
    }
    return 0;
  }
  int cur = 0;
  cudaGetDevice(&cur);
  for (int g = 0; g < ctx->ngroups; ++g) {
    const int n = ctx->group_n[g];
    CollArgs a = base;
    a.pack.c = ctx->comm_for(ctx->group_ranks[g][0]);
    a.pack.emu = ctx->group_dcomms[g];
    for (int i = 0; i < n; ++i) {
      const PerRank& p = pr[ctx->group_ranks[g][i]];
      a.in[i] = p.in;
      a.out[i] = p.out;
      a.aux_in[i] = p.aux_in;
      a.aux_out[i] = p.aux_out;
      a.gamma[i] = p.gamma;
    }
    RT_TRY(cudaSetDevice(ctx->group_dev[g]), "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(pr[ctx->group_ranks[g][0]].stream);
    if (n == 1) {
      kernel<<<dim3(grid_x, 1, 1), threads, 0, st>>>(a);
      RT_TRY(cudaGetLastError(), "collective launch");
    } else {
      // ranks that share a GPU wait on one another: they must be co-resident
      void* params[] = {&a};
      RT_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(grid_x, n, 1),
                                         dim3(threads, 1, 1), params, 0, st),
             "cooperative collective launch");
    }
  }
  cudaSetDevice(cur);
  return 0;
}

static int pick_grid(const blCtx* ctx, size_t work_vecs, int threads, int cap) {
  size_t g = (work_vecs + size_t(threads) - 1) / size_t(threads);
  if (g < 1) g = 1;
  if (!ctx->peer_mode) {
    // cooperative launches of several ranks on one GPU must stay co-resident
    int maxn = 1;
    for (int i = 0; i < ctx->ngroups; ++i) maxn = ctx->group_n[i] > maxn ? ctx->group_n[i] : maxn;
    if (maxn > 1) cap = cap < 8 ? cap : 8;
  }
  if (g > size_t(cap)) g = size_t(cap);
  return int(g);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int V>
using DtTag = std::integral_constant<int, V>;

// calls f(DtTag<dtype>{}) for a supported dtype code
template <typename F>
static int dispatch_dtype(int dtype, char* err, size_t errlen, F&& f) {
  switch (dtype) {
    case BL_DTYPE_FP32: return f(DtTag<BL_DTYPE_FP32>{});
    case BL_DTYPE_BF16: return f(DtTag<BL_DTYPE_BF16>{});
    case BL_DTYPE_FP16: return f(DtTag<BL_DTYPE_FP16>{});
    case BL_DTYPE_FP8E4M3: return f(DtTag<BL_DTYPE_FP8E4M3>{});
    case BL_DTYPE_FP8E5M2: return f(DtTag<BL_DTYPE_FP8E5M2>{});
    case BL_DTYPE_FP64: return f(DtTag<BL_DTYPE_FP64>{});
    case BL_DTYPE_U8: return f(DtTag<BL_DTYPE_U8>{});
    default:
      set_err(err, errlen, "barlink: unsupported dtype code %d", dtype);
      return -1;
  }
}

static int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

static int resolve_algo(const blCtx* ctx, int algo, size_t bytes, int dtype) {
  const bool lamport_ok = dtype != BL_DTYPE_U8 && dtype != BL_DTYPE_FP64 &&
                          bytes <= ctx->layout.lamport_slice;
  const bool nvls_ok = ctx->has_mc && ctx->peer_mode &&
                       (dtype == BL_DTYPE_BF16 || dtype == BL_DTYPE_FP16 || dtype == BL_DTYPE_FP32);
  if (algo == BL_ALGO_AUTO) {
    static int env_algo = -1;
    static int oneshot_max = -1;
    if (env_algo < 0) {
      const char* v = getenv("BL_AR_ALGO");
      env_algo = BL_ALGO_AUTO;
      if (v && !strcmp(v, "oneshot")) env_algo = BL_ALGO_ONESHOT;
      if (v && !strcmp(v, "twoshot")) env_algo = BL_ALGO_TWOSHOT;
      if (v && !strcmp(v, "nvls")) env_algo = BL_ALGO_NVLS;
      if (env_flag_set("BL_AR_NO_FUSED")) env_algo = BL_ALGO_TWOSHOT;
      oneshot_max = env_int("BL_ONESHOT_MAX", 0);
    }
    algo = env_algo;
    if (algo == BL_ALGO_AUTO) {
      // one hop of (world-1) x bytes beats two hops of 2 x bytes/world until
      // the link time outgrows the extra flag round trip
      size_t lim = oneshot_max > 0 ? size_t(oneshot_max)
                                   : (ctx->world <= 2 ? (1u << 20) : (512u << 10));  // measured crossovers
      if (lamport_ok && bytes <= lim) algo = BL_ALGO_ONESHOT;
      else if (nvls_ok && bytes >= (512u << 10)) algo = BL_ALGO_NVLS;
      else algo = BL_ALGO_TWOSHOT;
    }
  }
  if (algo == BL_ALGO_ONESHOT && !lamport_ok) algo = BL_ALGO_TWOSHOT;
  if (algo == BL_ALGO_NVLS && !nvls_ok) algo = BL_ALGO_TWOSHOT;
  return algo;
}

}  // namespace bl
// Algorithm the dispatcher would take for an all-reduce of `bytes` (host-only, no GPU needed):
// 0 auto, 1 one-shot, 2 two-shot, 3 NVLS as in bl_core.h.
extern "C" int bl_algo_for(size_t bytes, int world, int dtype, int has_multicast, size_t pool_bytes, int algo) {
  blCtx* c = new blCtx();
  c->world = world;
  c->peer_mode = true;
  c->has_mc = has_multicast != 0;
  const bl::Layout L = bl::compute_layout(pool_bytes, world);
  c->layout.lamport_slice = L.lamport_slice;
  const int r = bl::resolve_algo(c, algo, bytes, dtype);
  delete c;
  return r;
}
namespace bl {

// all-reduce on every local rank (peer mode: one)
static int allreduce_local(blCtx* ctx, const PerRank* pr, size_t bytes, int dtype, int algo,
                           char* err, size_t errlen) {
  if (check_health(ctx, err, errlen) != 0) return -1;
  const int nloc = ctx->local_ranks();
  if (bytes == 0 || (bytes & 15u)) {
    set_err(err, errlen, "barlink: all-reduce size %zu B is not a non-zero multiple of 16", bytes);
    return -1;
  }
  for (int l = 0; l < nloc; ++l)
    if (!aligned16(pr[l].in) || !aligned16(pr[l].out)) {
      set_err(err, errlen, "barlink: all-reduce pointers must be 16-byte aligned");
      return -1;
    }
  const size_t max_chunk = ctx->layout.stage_slice * size_t(ctx->world);
  if (bytes > max_chunk) {
    set_err(err, errlen, "barlink: all-reduce of %zu B exceeds the %zu B per-call limit (chunk it)",
            bytes, max_chunk);
    return -1;
  }
  algo = resolve_algo(ctx, algo, bytes, dtype);
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  int rc = -1;
  if (algo == BL_ALGO_ONESHOT) {
    const int grid = pick_grid(ctx, a.nvec, kThreads, 32);
    rc = dispatch_dtype(dtype, err, errlen, [&](auto tag) -> int {
      constexpr int DT = decltype(tag)::value;
      if constexpr (DT == BL_DTYPE_U8 || DT == BL_DTYPE_FP64) {
        return -1;
      } else {
        return launch_local(ctx, k_lamport<DT, false>, a, pr, grid, kThreads, err, errlen, true, true);
      }
    });
    ctx->stats[BL_STAT_ONESHOT]++;
  } else if (algo == BL_ALGO_NVLS) {
    const int grid = pick_grid(ctx, (a.nvec + ctx->world - 1) / ctx->world, kThreads, 64);
    rc = dispatch_dtype(dtype, err, errlen, [&](auto tag) -> int {
      constexpr int DT = decltype(tag)::value;
      if constexpr (DT == BL_DTYPE_BF16 || DT == BL_DTYPE_FP16 || DT == BL_DTYPE_FP32) {
        return launch_local(ctx, k_nvls<DT>, a, pr, grid, kThreads, err, errlen);
      } else {
        return -1;
      }
    });
    ctx->stats[BL_STAT_NVLS]++;
  } else {
    a.mode = 0;
    const int grid = pick_grid(ctx, (a.nvec + ctx->world - 1) / ctx->world, kThreads, 128);
    rc = dispatch_dtype(dtype, err, errlen, [&](auto tag) -> int {
      constexpr int DT = decltype(tag)::value;
      return launch_local(ctx, k_staged<DT>, a, pr, grid, kThreads, err, errlen);
    });
    ctx->stats[BL_STAT_TWOSHOT]++;
  }
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_BYTES] += bytes;
  return rc;
}

bool env_flag_set(const char* name) {
  const char* v = getenv(name);
  return v && *v && v[0] != '0';
}

}  // namespace bl

using namespace bl;

// ---------------------------------------------------------------------------
// C API
// ---------------------------------------------------------------------------
extern "C" void bl_set_wait_timeout_ms(blCtx* ctx, unsigned ms) {
  if (!ctx || ms == 0) return;
  ctx->timeout_ms = ms;
  char e[64];
  upload_comms(ctx, e, sizeof(e));
}

extern "C" int bl_status(blCtx* ctx, blStatus* out) {
  if (!ctx || !out || !ctx->h_status) return -1;
  const int nloc = ctx->local_ranks();
  memset(out, 0, sizeof(*out));
  for (int l = 0; l < nloc; ++l)
    if (ctx->h_status[l].code) {
      memcpy(out, const_cast<const blStatus*>(ctx->h_status + l), sizeof(*out));
      break;
    }
  return 0;
}

extern "C" int bl_reset_peer(blCtx* ctx, char* err, size_t errlen) {
  if (!ctx) return -1;
  int cur = 0;
  cudaGetDevice(&cur);
  const int nloc = ctx->local_ranks();
  for (int l = 0; l < nloc; ++l) {
    const int r = ctx->peer_mode ? ctx->rank : l;
    RT_TRY(cudaSetDevice(ctx->arena[r].device), "cudaSetDevice");
    RT_TRY(cudaDeviceSynchronize(), "sync before reset");
  }
  for (int l = 0; l < nloc; ++l) {
    const int r = ctx->peer_mode ? ctx->rank : l;
    RT_TRY(cudaSetDevice(ctx->arena[r].device), "cudaSetDevice");
    char* base = reinterpret_cast<char*>(ctx->arena[r].va);
    RT_TRY(cudaMemset(base + ctx->layout.sig_off, 0, kSigBytes), "signal pad clear");
    const size_t lam_words = 3 * size_t(ctx->world) * ctx->layout.lamport_slice / 4;
    k_fill_u32<<<256, 256>>>(reinterpret_cast<uint32_t*>(base + ctx->layout.lamport_off), lam_words,
                             kUnwritten);
    RT_TRY(cudaDeviceSynchronize(), "inbox fill");
  }
  memset(ctx->h_status, 0, sizeof(blStatus) * kMaxRanks);
  cudaSetDevice(cur);
  return 0;
}

extern "C" int bl_allreduce_into_peer(blCtx* ctx, const void* inPtr, void* outPtr, size_t bytes,
                                      int dtype, int algo, void* stream, char* err, size_t errlen) {
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: allreduce_into needs an SPMD context (init_peer)");
    return -1;
  }
  PerRank pr;
  pr.in = inPtr;
  pr.out = outPtr;
  pr.stream = stream;
  return allreduce_local(ctx, &pr, bytes, dtype, algo, err, errlen);
}

extern "C" int bl_allreduce_(blCtx* ctx, void* const* ptrs, const int* idxs, int n, size_t bytes,
                             int dtype, void* const* streams, char* err, size_t errlen) {
  if (!ctx || ctx->peer_mode) {
    set_err(err, errlen, "barlink: bl_allreduce_ is the single-process call; use allreduce_into in SPMD mode");
    return -1;
  }
  if (n != ctx->world) {
    set_err(err, errlen, "barlink: allreduce_ needs one pool tensor per arena (%d given, %d arenas)",
            n, ctx->world);
    return -1;
  }
  PerRank pr[kMaxRanks];
  bool seen[kMaxRanks] = {};
  for (int i = 0; i < n; ++i) {
    const int r = idxs[i];
    if (r < 0 || r >= ctx->world || seen[r]) {
      set_err(err, errlen, "barlink: allreduce_ arena indices must be a permutation of 0..%d", n - 1);
      return -1;
    }
    seen[r] = true;
    if (bl_pool_offset(ctx, r, ptrs[i]) < 0) {
      set_err(err, errlen, "barlink: allreduce_ tensor %d is not a pool tensor of arena %d", i, r);
      return -1;
    }
    pr[r].in = ptrs[i];
    pr[r].out = ptrs[i];
    pr[r].stream = streams ? streams[i] : nullptr;
  }
  return allreduce_local(ctx, pr, bytes, dtype, BL_ALGO_AUTO, err, errlen);
}

static int staged_local(blCtx* ctx, int mode, const PerRank* pr, size_t per_rank_bytes,
                        size_t stride_bytes, int dtype, int root, char* err, size_t errlen) {
  if (check_health(ctx, err, errlen) != 0) return -1;
  bool al = true;
  for (int l = 0; l < ctx->local_ranks(); ++l) al = al && aligned16(pr[l].in) && aligned16(pr[l].out);
  if (per_rank_bytes == 0 || (per_rank_bytes & 15u) || !al) {
    set_err(err, errlen, "barlink: collective needs 16-byte aligned pointers and a size that is a non-zero multiple of 16 (%zu)",
            per_rank_bytes);
    return -1;
  }
  if (per_rank_bytes > ctx->layout.stage_slice) {
    set_err(err, errlen, "barlink: %zu B per rank exceeds the %zu B staging slice (chunk it)",
            per_rank_bytes, ctx->layout.stage_slice);
    return -1;
  }
  CollArgs a;
  memset(&a, 0, sizeof(a));
  if (stride_bytes & 15u) {
    set_err(err, errlen, "barlink: slice stride %zu is not a multiple of 16", stride_bytes);
    return -1;
  }
  a.nvec = per_rank_bytes / 16;
  a.slice_stride = stride_bytes / 16;
  a.mode = mode;
  a.root = root;
  const int grid = pick_grid(ctx, a.nvec, kThreads, 128);
  int rc = -1;
  rc = dispatch_dtype(dtype, err, errlen, [&](auto tag) -> int {
    constexpr int DT = decltype(tag)::value;
    return launch_local(ctx, k_staged<DT>, a, pr, grid, kThreads, err, errlen);
  });
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_BYTES] += per_rank_bytes;
  return rc;
}

static int staged_peer(blCtx* ctx, int mode, const void* in, void* out, size_t per_rank_bytes,
                       size_t stride_bytes, int dtype, int root, void* stream, char* err,
                       size_t errlen) {
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: this collective needs an SPMD context (init_peer)");
    return -1;
  }
  PerRank pr;
  pr.in = in;
  pr.out = out;
  pr.stream = stream;
  return staged_local(ctx, mode, &pr, per_rank_bytes, stride_bytes, dtype, root, err, errlen);
}

extern "C" int bl_allgather_peer(blCtx* ctx, const void* inPtr, void* outPtr, size_t bytesPerRank,
                                 size_t outStrideBytes, void* stream, char* err, size_t errlen) {
  return staged_peer(ctx, 2, inPtr, outPtr, bytesPerRank, outStrideBytes, BL_DTYPE_U8, 0, stream,
                     err, errlen);
}
extern "C" int bl_reduce_scatter_peer(blCtx* ctx, const void* inPtr, void* outPtr,
                                      size_t bytesPerRank, size_t inStrideBytes, int dtype,
                                      void* stream, char* err, size_t errlen) {
  return staged_peer(ctx, 1, inPtr, outPtr, bytesPerRank, inStrideBytes, dtype, 0, stream, err,
                     errlen);
}
extern "C" int bl_broadcast_peer(blCtx* ctx, void* ptr, size_t bytes, int root, void* stream,
                                 char* err, size_t errlen) {
  if (ctx && (root < 0 || root >= ctx->world)) {
    set_err(err, errlen, "barlink: broadcast root %d out of range", root);
    return -1;
  }
  return staged_peer(ctx, 3, ptr, ptr, bytes, 0, BL_DTYPE_U8, root, stream, err, errlen);
}

extern "C" int bl_barrier_peer(blCtx* ctx, void* stream, char* err, size_t errlen) {
  if (!ctx) return -1;
  if (check_health(ctx, err, errlen) != 0) return -1;
  CollArgs a;
  memset(&a, 0, sizeof(a));
  PerRank pr[kMaxRanks];
  for (auto& p : pr) p.stream = stream;
  return launch_local(ctx, k_barrier, a, pr, 1, 32, err, errlen);
}

static int norm_local(blCtx* ctx, const PerRank* pr, int rows, int hidden, float eps, int dtype,
                      int nsplit, size_t slab, char* err, size_t errlen) {
  if (check_health(ctx, err, errlen) != 0) return -1;
  const int esz = dtype == BL_DTYPE_FP32 ? 4 : 2;
  if (dtype != BL_DTYPE_BF16 && dtype != BL_DTYPE_FP16 && dtype != BL_DTYPE_FP32) {
    set_err(err, errlen, "barlink: allreduce_rmsnorm supports bf16, fp16 and fp32");
    return -1;
  }
  const size_t row_bytes = size_t(hidden) * esz;
  const size_t bytes = row_bytes * size_t(rows);
  if (rows < 1 || hidden < 1 || (row_bytes & 15u) || row_bytes / 16 > size_t(kThreads) * 4) {
    set_err(err, errlen, "barlink: allreduce_rmsnorm needs hidden*itemsize to be a multiple of 16 and at most %d B",
            kThreads * 4 * 16);
    return -1;
  }
  if (bytes > ctx->layout.lamport_slice) {
    set_err(err, errlen, "barlink: allreduce_rmsnorm message of %zu B exceeds the one-shot inbox (%zu B); split the rows",
            bytes, ctx->layout.lamport_slice);
    return -1;
  }
  for (int l = 0; l < ctx->local_ranks(); ++l)
    if (!aligned16(pr[l].in) || !aligned16(pr[l].gamma) || !aligned16(pr[l].aux_out) ||
        !aligned16(pr[l].out) || !aligned16(pr[l].aux_in)) {
      set_err(err, errlen, "barlink: allreduce_rmsnorm pointers must be 16-byte aligned");
      return -1;
    }
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  a.rows = rows;
  a.vec_per_row = int(row_bytes / 16);
  a.eps = eps;
  a.nsplit = nsplit;
  a.slab = slab;
  if (nsplit > 0 && dtype == BL_DTYPE_FP32) {
    set_err(err, errlen, "barlink: slab input to allreduce_rmsnorm needs a 16-bit output type");
    return -1;
  }
  int grid = rows < 64 ? rows : 64;
  if (!ctx->peer_mode && grid > 8) grid = 8;
  int rc = -1;
  // one thread per vector up to the block limit keeps short rows from
  // wasting a 512-thread block
  int threads = (a.vec_per_row + 31) / 32 * 32;
  if (threads > kThreads) threads = kThreads;
  if (threads < 64) threads = 64;
  switch (dtype) {
    case BL_DTYPE_BF16:
      rc = launch_local(ctx, k_lamport<BL_DTYPE_BF16, true>, a, pr, grid, threads, err, errlen, true, true);
      break;
    case BL_DTYPE_FP16:
      rc = launch_local(ctx, k_lamport<BL_DTYPE_FP16, true>, a, pr, grid, threads, err, errlen, true, true);
      break;
    default:
      rc = launch_local(ctx, k_lamport<BL_DTYPE_FP32, true>, a, pr, grid, threads, err, errlen, true, true);
  }
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_FUSED_NORM]++;
  ctx->stats[BL_STAT_BYTES] += bytes;
  return rc;
}

extern "C" int bl_allreduce_rmsnorm_peer(blCtx* ctx, const void* inPtr, const void* residualIn,
                                         const void* gamma, void* residualOut, void* normedOut,
                                         int rows, int hidden, float eps, int dtype, int nsplit,
                                         size_t slab, void* stream, char* err, size_t errlen) {
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: allreduce_rmsnorm needs an SPMD context (init_peer)");
    return -1;
  }
  PerRank pr;
  pr.in = inPtr;
  pr.out = normedOut;
  pr.aux_in = residualIn;
  pr.aux_out = residualOut;
  pr.gamma = gamma;
  pr.stream = stream;
  return norm_local(ctx, &pr, rows, hidden, eps, dtype, nsplit, slab, err, errlen);
}

// Single-process form of the SPMD collectives: one pointer per arena.  With
// ranks that share a GPU this is how an N-rank protocol is exercised on one
// device (one cooperative kernel over all ranks' data).
// kind: 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 broadcast,
//       4 all-reduce + residual + RMSNorm, 5 barrier
extern "C" int bl_sp_collective(blCtx* ctx, int kind, const void* const* in, void* const* out,
                                const void* const* aux_in, void* const* aux_out,
                                const void* const* gamma, size_t bytes, int dtype, int algo, int root,
                                int rows, int hidden, float eps, void* const* streams, char* err,
                                size_t errlen) {
  if (!ctx || ctx->peer_mode) {
    set_err(err, errlen, "barlink: sp_collective is the single-process call (init, not init_peer)");
    return -1;
  }
  PerRank pr[kMaxRanks];
  for (int r = 0; r < ctx->world; ++r) {
    pr[r].in = in ? in[r] : nullptr;
    pr[r].out = out ? out[r] : nullptr;
    pr[r].aux_in = aux_in ? aux_in[r] : nullptr;
    pr[r].aux_out = aux_out ? aux_out[r] : nullptr;
    pr[r].gamma = gamma ? gamma[r] : nullptr;
    pr[r].stream = streams ? streams[r] : nullptr;
  }
  switch (kind) {
    case 0: return allreduce_local(ctx, pr, bytes, dtype, algo, err, errlen);
    case 1: return staged_local(ctx, 1, pr, bytes, 0, dtype, 0, err, errlen);
    case 2: return staged_local(ctx, 2, pr, bytes, 0, BL_DTYPE_U8, 0, err, errlen);
    case 3: return staged_local(ctx, 3, pr, bytes, 0, BL_DTYPE_U8, root, err, errlen);
    case 4: return norm_local(ctx, pr, rows, hidden, eps, dtype, 0, 0, err, errlen);
    case 5: {
      if (check_health(ctx, err, errlen) != 0) return -1;
      CollArgs a;
      memset(&a, 0, sizeof(a));
      return launch_local(ctx, k_barrier, a, pr, 1, 32, err, errlen);
    }
    default:
      set_err(err, errlen, "barlink: unknown collective kind %d", kind);
      return -1;
  }
}

// Single-process p2p: the send runs as rank `src`, then the recv as rank
// `dst`, in that order on one stream (a send never waits for the message it
// carries to be consumed, so the pair cannot block on a shared GPU).
extern "C" int bl_sp_sendrecv(blCtx* ctx, int src, int dst, const void* in, void* out, size_t bytes,
                              void* stream, char* err, size_t errlen) {
  if (!ctx || ctx->peer_mode) {
    set_err(err, errlen, "barlink: sp_sendrecv is the single-process call");
    return -1;
  }
  if (src < 0 || dst < 0 || src >= ctx->world || dst >= ctx->world || src == dst) {
    set_err(err, errlen, "barlink: sp_sendrecv needs two different ranks below %d", ctx->world);
    return -1;
  }
  if (ctx->arena[src].device != ctx->arena[dst].device) {
    set_err(err, errlen, "barlink: sp_sendrecv is for ranks that share a GPU; use copy_ across GPUs");
    return -1;
  }
  if (bytes == 0 || (bytes & 15u) || !aligned16(in) || !aligned16(out) || bytes > ctx->layout.p2p_slice) {
    set_err(err, errlen, "barlink: sp_sendrecv needs aligned pointers and a multiple of 16 bytes up to %zu",
            ctx->layout.p2p_slice);
    return -1;
  }
  if (check_health(ctx, err, errlen) != 0) return -1;
  int cur = 0;
  cudaGetDevice(&cur);
  RT_TRY(cudaSetDevice(ctx->arena[src].device), "cudaSetDevice");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  size_t g = (a.nvec + kThreads - 1) / kThreads;
  const int grid = int(g > 32 ? 32 : g);
  a.pack.c = ctx->comm_for(src);
  a.peer = dst;
  a.in[0] = in;
  k_p2p_send<<<grid, kThreads, 0, st>>>(a);
  RT_TRY(cudaGetLastError(), "send launch");
  a.pack.c = ctx->comm_for(dst);
  a.peer = src;
  a.in[0] = nullptr;
  a.out[0] = out;
  k_p2p_recv<<<grid, kThreads, 0, st>>>(a);
  RT_TRY(cudaGetLastError(), "recv launch");
  cudaSetDevice(cur);
  ctx->stats[BL_STAT_P2P] += 2;
  return 0;
}

// ---- p2p ---------------------------------------------------------------------
static bool stream_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return st != cudaStreamCaptureStatusNone;
}

// work queued later on `stream` must see the sends queued so far
static void join_send_stream(blCtx* ctx, cudaStream_t stream) {
  if (!ctx->send_pending || stream_capturing(stream)) return;
  cudaStreamWaitEvent(stream, ctx->ev_send, 0);
}

static int p2p_check(blCtx* ctx, const void* p, size_t bytes, int peer, char* err, size_t errlen) {
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: send/recv need an SPMD context (init_peer)");
    return -1;
  }
  if (peer < 0 || peer >= ctx->world || peer == ctx->rank) {
    set_err(err, errlen, "barlink: p2p peer %d invalid for rank %d of %d (sending to oneself is not supported)",
            peer, ctx->rank, ctx->world);
    return -1;
  }
  if (bytes == 0 || (bytes & 15u) || !aligned16(p)) {
    set_err(err, errlen, "barlink: p2p needs a 16-byte aligned pointer and a non-zero multiple of 16 bytes (%zu)",
            bytes);
    return -1;
  }
  if (bytes > ctx->layout.p2p_slice) {
    set_err(err, errlen, "barlink: p2p message of %zu B exceeds the %zu B inbox (chunk it)", bytes,
            ctx->layout.p2p_slice);
    return -1;
  }
  return check_health(ctx, err, errlen);
}

extern "C" int bl_send_into_peer(blCtx* ctx, const void* inPtr, size_t bytes, int peerRank,
                                 void* stream, char* err, size_t errlen) {
  if (p2p_check(ctx, inPtr, bytes, peerRank, err, errlen) != 0) return -1;
  cudaStream_t caller = static_cast<cudaStream_t>(stream);
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  a.peer = peerRank;
  PerRank pr;
  pr.in = inPtr;
  const int grid = pick_grid(ctx, a.nvec, kThreads, 64);
  static const bool no_side = env_flag_set("BL_P2P_NO_SIDESTREAM");
  // A send gates on the receipt of the previous message.  On its own stream
  // it cannot block a recv that the caller queues behind it (several sends
  // outstanding before the first recv would otherwise deadlock a pair).
  if (no_side || stream_capturing(caller)) {
    pr.stream = caller;
    if (launch_local(ctx, k_p2p_send, a, &pr, grid, kThreads, err, errlen, false) != 0) return -1;
  } else {
    RT_TRY(cudaEventRecord(ctx->ev_caller, caller), "event record");
    RT_TRY(cudaStreamWaitEvent(ctx->send_stream, ctx->ev_caller, 0), "stream wait");
    pr.stream = ctx->send_stream;
    if (launch_local(ctx, k_p2p_send, a, &pr, grid, kThreads, err, errlen, false) != 0) return -1;
    RT_TRY(cudaEventRecord(ctx->ev_send, ctx->send_stream), "event record");
    ctx->send_pending = true;
  }
  ctx->stats[BL_STAT_P2P]++;
  ctx->stats[BL_STAT_BYTES] += bytes;
  return 0;
}

extern "C" int bl_recv_into_peer(blCtx* ctx, void* outPtr, size_t bytes, int peerRank, void* stream,
                                 char* err, size_t errlen) {
  if (p2p_check(ctx, outPtr, bytes, peerRank, err, errlen) != 0) return -1;
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  a.peer = peerRank;
  PerRank pr;
  pr.out = outPtr;
  pr.stream = stream;
  const int grid = pick_grid(ctx, a.nvec, kThreads, 64);
  if (launch_local(ctx, k_p2p_recv, a, &pr, grid, kThreads, err, errlen, false) != 0) return -1;
  ctx->stats[BL_STAT_P2P]++;
  return 0;
}

// make later work on `stream` wait for sends issued so far (used by the
// binding before a tensor that was sent may be overwritten)
extern "C" void* bl_send_stream(blCtx* ctx) { return ctx && ctx->peer_mode ? ctx->send_stream : nullptr; }

extern "C" int bl_join_sends(blCtx* ctx, void* stream) {
  if (!ctx || !ctx->peer_mode) return 0;
  join_send_stream(ctx, static_cast<cudaStream_t>(stream));
  return 0;
}

// ---- single-process copy ---------------------------------------------------------
extern "C" int bl_copy_(blCtx* ctx, void* dstPtr, int dstIdx, void* srcPtr, int srcIdx, size_t bytes,
                        void* srcStream, void* dstStream, char* err, size_t errlen) {
  if (!ctx || ctx->peer_mode) {
    set_err(err, errlen, "barlink: copy_ is the single-process call; use send/recv in SPMD mode");
    return -1;
  }
  if (bl_pool_offset(ctx, dstIdx, dstPtr) < 0 || bl_pool_offset(ctx, srcIdx, srcPtr) < 0) {
    set_err(err, errlen, "barlink: copy_ needs pool tensors (allocate them with empty())");
    return -1;
  }
  if (bytes == 0 || (bytes & 15u) || !aligned16(dstPtr) || !aligned16(srcPtr)) {
    set_err(err, errlen, "barlink: copy_ needs 16-byte aligned pool tensors and a non-zero multiple of 16 bytes");
    return -1;
  }
  int cur = 0;
  cudaGetDevice(&cur);
  // the source GPU stores straight into the destination arena over NVLink
  RT_TRY(cudaSetDevice(ctx->arena[srcIdx].device), "cudaSetDevice");
  const size_t nvec = bytes / 16;
  int grid = int((nvec + 511) / 512);
  if (grid > 296) grid = 296;
  cudaStream_t ss = static_cast<cudaStream_t>(srcStream), ds = static_cast<cudaStream_t>(dstStream);
  k_copy_vec<<<grid, 512, 0, ss>>>(static_cast<const uint4*>(srcPtr), static_cast<uint4*>(dstPtr), nvec);
  RT_TRY(cudaGetLastError(), "copy launch");
  if (ss != ds || ctx->arena[srcIdx].device != ctx->arena[dstIdx].device) {
    cudaEvent_t ev;
    RT_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "event");
    RT_TRY(cudaEventRecord(ev, ss), "event record");
    RT_TRY(cudaSetDevice(ctx->arena[dstIdx].device), "cudaSetDevice");
    RT_TRY(cudaStreamWaitEvent(ds, ev, 0), "stream wait");
    cudaEventDestroy(ev);
  }
  cudaSetDevice(cur);
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_BYTES] += bytes;
  return 0;
}

// ---- proofs / diagnostics ---------------------------------------------------------
extern "C" uint64_t bl_verify(blCtx* ctx, char* err, size_t errlen) {
  if (!ctx) return ~0ull;
  if (check_health(ctx, err, errlen) != 0) return ~0ull;
  CollArgs a;
  memset(&a, 0, sizeof(a));
  size_t bytes = ctx->layout.stage_slice < (4u << 20) ? ctx->layout.stage_slice : (4u << 20);
  a.nvec = bytes / 16;
  a.bad = ctx->d_bad;
  static unsigned seed = 0x1234;
  a.seed = seed++;
  *ctx->d_bad = 0;
  PerRank pr[kMaxRanks];
  const int grid = pick_grid(ctx, a.nvec, kThreads, 32);
  if (launch_local(ctx, k_verify, a, pr, grid, kThreads, err, errlen) != 0) return ~0ull;
  const int nloc = ctx->local_ranks();
  int cur = 0;
  cudaGetDevice(&cur);
  for (int l = 0; l < nloc; ++l) {
    const int r = ctx->peer_mode ? ctx->rank : l;
    cudaSetDevice(ctx->arena[r].device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      set_err(err, errlen, "barlink: verify kernel failed: %s", cudaGetErrorString(e));
      cudaSetDevice(cur);
      return ~0ull;
    }
  }
  cudaSetDevice(cur);
  if (check_health(ctx, err, errlen) != 0) return ~0ull;
  return *const_cast<volatile unsigned long long*>(ctx->d_bad);
}

extern "C" int bl_readback(blCtx* ctx, int devIdx, void* ptr, size_t bytes, void* dstHost, char* err,
                           size_t errlen) {
  if (!ctx) return -1;
  const int r = ctx->peer_mode ? ctx->rank : devIdx;
  if (r < 0 || r >= ctx->world || bl_pool_offset(ctx, devIdx, ptr) < 0) {
    set_err(err, errlen, "barlink: readback needs a pool tensor of a local arena");
    return -1;
  }
  int cur = 0;
  cudaGetDevice(&cur);
  RT_TRY(cudaSetDevice(ctx->arena[r].device), "cudaSetDevice");
  RT_TRY(cudaDeviceSynchronize(), "sync");
  RT_TRY(cudaMemcpy(dstHost, ptr, bytes, cudaMemcpyDeviceToHost), "readback copy");
  cudaSetDevice(cur);
  return 0;
}

extern "C" int bl_pool_move(blCtx* ctx, void* srcPoolPtr, void* outPtr, size_t bytes, void* stream,
                            char* err, size_t errlen) {
  if (!ctx) return -1;
  if (bytes == 0 || (bytes & 15u) || !aligned16(srcPoolPtr) || !aligned16(outPtr)) {
    set_err(err, errlen, "barlink: pool_move needs 16-byte aligned pointers and a non-zero multiple of 16 bytes");
    return -1;
  }
  const size_t nvec = bytes / 16;
  int grid = int((nvec + 511) / 512);
  if (grid > 296) grid = 296;
  k_copy_vec<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(srcPoolPtr), static_cast<uint4*>(outPtr), nvec);
  RT_TRY(cudaGetLastError(), "pool_move launch");
  return 0;
}

extern "C" int bl_debug_flags(blCtx* ctx, unsigned long long* vals, int n, char* err, size_t errlen) {
  if (!ctx || !vals || n < 1 || n > 4096) return -1;
  const int r = ctx->peer_mode ? ctx->rank : 0;
  std::vector<uint32_t> tmp(n);
  cudaStream_t s;
  RT_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "stream");
  cudaError_t e = cudaMemcpyAsync(tmp.data(),
                                  reinterpret_cast<char*>(ctx->arena[r].va) + ctx->layout.sig_off,
                                  size_t(n) * 4, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaStreamDestroy(s);
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: debug_flags copy failed: %s", cudaGetErrorString(e));
    return -1;
  }
  for (int i = 0; i < n; ++i) vals[i] = tmp[i];
  return 0;
}

extern "C" int bl_probe_signal(blCtx* ctx, unsigned long long* res, int iters, void* stream, char* err,
                               size_t errlen) {
  if (!ctx || !res || iters < 1) return -1;
  if (check_health(ctx, err, errlen) != 0) return -1;
  res[0] = res[1] = res[2] = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long* h = nullptr;
  RT_TRY(cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped), "probe buffer");
  h[0] = 0;
  if (ctx->peer_mode && ctx->world >= 2) {
    CollArgs a;
    memset(&a, 0, sizeof(a));
    a.pack.c = ctx->comm_for(ctx->rank);
    a.iters = iters;
    k_probe<<<1, 32, 0, st>>>(a, h);
    RT_TRY(cudaStreamSynchronize(st), "probe");
    res[0] = h[0];
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  k_empty<<<1, 1, 0, st>>>();
  cudaEventRecord(e0, st);
  for (int i = 0; i < iters; ++i) k_empty<<<1, 1, 0, st>>>();
  cudaEventRecord(e1, st);
  cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  res[1] = (unsigned long long)(double(ms) * 1e6 / iters);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFreeHost(h);
  return 0;
}

// ---------------------------------------------------------------------------
// fused tensor-parallel linears: host side
// ---------------------------------------------------------------------------
extern "C" int bl_tp_units(int n, int k_local, int tokens, int* splits_out) {
  const int tiles = (n + 127) / 128;
  const int kblocks = (k_local + 63) / 64;
  (void)tokens;
  const int splits = pick_splits(tiles, kblocks, sm_count(), 0);
  if (splits_out) *splits_out = splits;
  return tiles * splits;
}

extern "C" int bl_tp_peer_sink(blCtx* ctx, size_t inbox_off, int tokens, blPeerSink* out, char* err,
                               size_t errlen) {
  if (!ctx || !ctx->peer_mode || !out) {
    set_err(err, errlen, "barlink: fused TP linears need an SPMD context (init_peer)");
    return -1;
  }
  if (tokens < ctx->world || tokens % ctx->world) {
    set_err(err, errlen, "barlink: fused reduce-scatter needs a token count that is a multiple of the %d ranks (got %d)",
            ctx->world, tokens);
    return -1;
  }
  if (inbox_off >= ctx->user_bytes || (inbox_off & 15u)) {
    set_err(err, errlen, "barlink: inbox offset %zu is not inside the arena's user zone", inbox_off);
    return -1;
  }
  if (check_health(ctx, err, errlen) != 0) return -1;
  memset(out, 0, sizeof(*out));
  out->world = ctx->world;
  out->rank = ctx->rank;
  out->tokens_per_rank = tokens / ctx->world;
  for (int r = 0; r < ctx->world; ++r) {
    char* base = reinterpret_cast<char*>(ctx->arena[r].va);
    out->inbox[r] = base + inbox_off;
    out->flag[r] = reinterpret_cast<uint32_t*>(base + ctx->layout.sig_off) + sig_flag(P_GEMM_RS, 0, ctx->rank);
  }
  return 0;
}

extern "C" int bl_tp_gate(blCtx* ctx, int tokens, blGemmArgs* a, char* err, size_t errlen) {
  if (!ctx || !ctx->peer_mode || !a) {
    set_err(err, errlen, "barlink: fused TP linears need an SPMD context (init_peer)");
    return -1;
  }
  if (tokens < ctx->world || tokens % ctx->world) {
    set_err(err, errlen, "barlink: fused all-gather needs a token count that is a multiple of the %d ranks (got %d)",
            ctx->world, tokens);
    return -1;
  }
  uint32_t* s = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(ctx->arena[ctx->rank].va) +
                                            ctx->layout.sig_off);
  a->gate_flags = s + sig_flag(P_AG_GEMM, 0, 0);
  a->gate_cum = s + sig_aux(P_AG_GEMM);
  a->gate_ticket = s + sig_ticket(P_AG_GEMM);
  a->gate_add = unsigned(tokens / ctx->world);
  a->gate_n = ctx->world;
  a->gate_timeout_ns = uint64_t(ctx->timeout_ms) * 1000000ull;
  return 0;
}

extern "C" int bl_rs_finish(blCtx* ctx, const blRsFinishArgs* a, void* stream, char* err,
                            size_t errlen) {
  if (!ctx || !ctx->peer_mode || !a) {
    set_err(err, errlen, "barlink: rs_finish needs an SPMD context (init_peer)");
    return -1;
  }
  if (check_health(ctx, err, errlen) != 0) return -1;
  if (a->tokens % ctx->world || a->n % 8 || a->n / 8 > kThreads * 4 || a->splits < 1 || !a->gamma ||
      !a->residual_out) {
    set_err(err, errlen, "barlink: rs_finish needs tokens %% world == 0, n %% 8 == 0, n <= %d, gamma and residual_out",
            kThreads * 32);
    return -1;
  }
  const int tpr = a->tokens / ctx->world;
  const size_t inbox_bytes = size_t(ctx->world) * a->splits * tpr * a->n * 4;
  const size_t gather_bytes = size_t(a->tokens) * a->n * 2;
  if (a->inbox_off + inbox_bytes > ctx->user_bytes || a->gather_off + gather_bytes > ctx->user_bytes) {
    set_err(err, errlen, "barlink: rs_finish buffers do not fit the arena's user zone");
    return -1;
  }
  RsFinishArgs k;
  k.c = ctx->comm_for(ctx->rank);
  k.inbox_off = a->inbox_off;
  k.gather_off = a->gather_off;
  k.tpr = tpr;
  k.n = a->n;
  k.splits = a->splits;
  k.units = a->units;
  k.residual_in = static_cast<const uint4*>(a->residual_in);
  k.residual_out = static_cast<uint4*>(a->residual_out);
  k.gamma = static_cast<const uint4*>(a->gamma);
  k.eps = a->eps;
  int threads = (a->n / 8 + 31) / 32 * 32;
  if (threads > kThreads) threads = kThreads;
  if (threads < 64) threads = 64;
  cudaError_t e = launch_k(k_rs_finish, dim3(tpr), dim3(threads), 0, static_cast<cudaStream_t>(stream), k);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(err, errlen, "barlink: rs_finish launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_FUSED_NORM]++;
  return 0;
}

// ---------------------------------------------------------------------------
// all-reduce whose scatter half is the epilogue of the GEMM that produced the data
// ---------------------------------------------------------------------------
extern "C" int bl_gemm_push_setup(blCtx* ctx, int total_rows, int n, int row0, blRowPush* out, char* err,
                                  size_t errlen) {
  if (!ctx || !ctx->peer_mode || !out) {
    set_err(err, errlen, "barlink: a pushed linear needs an SPMD context (init_peer)");
    return -1;
  }
  if (total_rows < ctx->world || total_rows % ctx->world || n < 8 || (n & 7) || row0 < 0 || row0 >= total_rows) {
    set_err(err, errlen, "barlink: pushed all-reduce needs rows that are a multiple of the %d ranks and n %% 8 == 0 (rows %d, n %d)",
            ctx->world, total_rows, n);
    return -1;
  }
  const size_t per_rank = size_t(total_rows / ctx->world) * size_t(n) * 2;
  if (per_rank > ctx->layout.stage_slice) {
    set_err(err, errlen, "barlink: %zu B per rank exceed the %zu B staging slice (raise BL_POOL_MB or split the rows)",
            per_rank, ctx->layout.stage_slice);
    return -1;
  }
  if (check_health(ctx, err, errlen) != 0) return -1;
  memset(out, 0, sizeof(*out));
  out->world = ctx->world;
  out->rank = ctx->rank;
  out->rows_per_rank = total_rows / ctx->world;
  out->row0 = row0;
  out->stage_off = ctx->layout.stage_off;
  out->stage_slice = ctx->layout.stage_slice;
  char* mine = reinterpret_cast<char*>(ctx->arena[ctx->rank].va);
  out->seq_word = reinterpret_cast<uint32_t*>(mine + ctx->layout.sig_off) + kSigStageSeq;
  for (int r = 0; r < ctx->world; ++r) {
    char* base = reinterpret_cast<char*>(ctx->arena[r].va);
    out->arena[r] = base;
    out->flag[r] = reinterpret_cast<uint32_t*>(base + ctx->layout.sig_off) + sig_flag(P_ROWPUSH, kMaxSlots - 1, ctx->rank);  // the last slot: the blocks' own syncs use slots < 128
  }
  return 0;
}

extern "C" int bl_allreduce_pushed(blCtx* ctx, void* out, int total_rows, int n, int units, void* stream, char* err,
                                   size_t errlen) {
  if (!ctx || !ctx->peer_mode) {
    set_err(err, errlen, "barlink: allreduce_pushed needs an SPMD context (init_peer)");
    return -1;
  }
  if (!out || !aligned16(out) || total_rows % ctx->world || units < 1) {
    set_err(err, errlen, "barlink: allreduce_pushed needs a 16-byte aligned output, rows that split over the ranks and units >= 1");
    return -1;
  }
  if (check_health(ctx, err, errlen) != 0) return -1;
  const size_t bytes = size_t(total_rows) * size_t(n) * 2;
  if (bytes / size_t(ctx->world) > ctx->layout.stage_slice) {
    set_err(err, errlen, "barlink: %zu B per rank exceed the staging slice", bytes / size_t(ctx->world));
    return -1;
  }
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nvec = bytes / 16;
  a.mode = 4;
  a.iters = units;
  PerRank pr;
  pr.in = out;
  pr.out = out;
  pr.stream = stream;
  const int grid = pick_grid(ctx, (a.nvec + ctx->world - 1) / ctx->world, kThreads, 128);
  const int rc = launch_local(ctx, k_staged<BL_DTYPE_BF16>, a, &pr, grid, kThreads, err, errlen);
  ctx->stats[BL_STAT_TWOSHOT]++;
  ctx->stats[BL_STAT_OPS]++;
  ctx->stats[BL_STAT_BYTES] += bytes;
  return rc;
}
