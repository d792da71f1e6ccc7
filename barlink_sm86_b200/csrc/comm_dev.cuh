// SPDX-License-Identifier: MIT
//
// Device-side helpers shared by the collective kernels and by the decode
// linears that fold a collective into their prologue or epilogue: the signal
// pad accessors, bounded waits that record where they gave up, the epoch
// hand-over of a protocol, element packing, and the "payload word is its own
// arrival flag" polling of the one-shot inboxes.  The reference's flag waits
// trap after a clock budget (torch_ext/barlink_sm86/core.cu:376-397); these
// return false and leave a status record instead.
#pragma once

#include <cuda_fp8.h>

#include "bl_ops.h"
#include "heap.h"
#include "ptx.cuh"

namespace bl {

constexpr uint32_t kUnwritten = 0x80000000u;  // -0.0f: "this word has not landed yet"

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ const Comm& comm_of(const CommPack& p) {
  return p.emu ? p.emu[blockIdx.y] : p.c;
}
__device__ __forceinline__ uint32_t* sig_of(const Comm& c, int r) {
  return reinterpret_cast<uint32_t*>(c.base[r] + c.sig_off);
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  return *reinterpret_cast<const volatile uint32_t*>(p);
}

static __device__ __noinline__ void report_timeout(const Comm& c, uint32_t code, int proto, int from,
                                            uint32_t have, uint32_t want) {
  uint32_t* s = sig_of(c, c.rank);
  if (atomicExch(&s[kSigAbort], 1u) == 0u && c.status) {
    volatile blStatus* st = c.status;
    st->proto = uint32_t(proto);
    st->from_rank = uint32_t(from);
    st->have = have;
    st->want = want;
    st->block = blockIdx.x;
    __threadfence_system();
    st->code = code;
  }
}

// Wait until *flag >= want (wrap-safe).  Bounded by the global timer; false
// when it ran out or when another wait of this rank already did.
__device__ __forceinline__ bool wait_flag(const Comm& c, const uint32_t* flag, uint32_t want,
                                          int proto, int from) {
  uint32_t v = ld_acquire_sys(flag);
  if (int32_t(v - want) >= 0) return true;
  const uint32_t* abortw = sig_of(c, c.rank) + kSigAbort;
  uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  for (;;) {
    v = ld_acquire_sys(flag);
    if (int32_t(v - want) >= 0) return true;
    if ((++polls & 255u) == 0u) {
      if (ld_volatile_u32(abortw)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_timeout(c, 1, proto, from, v, want);
        return false;
      }
    }
  }
}

// Block-wide exchange with every rank on slot `slot`: publish `v` to all
// ranks' pads (release: everything this block wrote before is visible to a
// peer that sees the flag), then wait for every rank's `v`.  Uniform result.
__device__ __forceinline__ bool block_sync_peers(const Comm& c, int proto, int slot, uint32_t v) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int p = threadIdx.x;
    st_release_sys(sig_of(c, p) + sig_flag(proto, slot, c.rank), v);
    if (!wait_flag(c, sig_of(c, c.rank) + sig_flag(proto, slot, p), v, proto, p)) s_ok = 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// The last block of this rank to arrive advances the epoch.  All blocks have
// read the epoch before they arrive, so none can see the new value.
__device__ __forceinline__ void finish_epoch(const Comm& c, int proto, uint32_t e, uint32_t aux,
                                             bool set_aux, bool staged = false) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* s = sig_of(c, c.rank);
    __threadfence();
    uint32_t t = atomicAdd(&s[sig_ticket(proto)], 1u);
    if (t == gridDim.x - 1) {
      s[sig_ticket(proto)] = 0;
      if (set_aux) s[sig_aux(proto)] = aux;
      if (staged) s[kSigStageSeq] = s[kSigStageSeq] + 1u;  // every block read it before it arrived here
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&s[sig_epoch(proto)]) = e + 1;
    }
  }
}

// Offset of the staging buffer this call uses (see kSigStageSeq); same on every rank because
// every rank issues the same sequence of staged collectives.
__device__ __forceinline__ size_t stage_buf_off(const Comm& c) {
  const uint32_t seq = ld_volatile_u32(sig_of(c, c.rank) + kSigStageSeq);
  return c.stage_off + size_t(seq & 1u) * (2 * size_t(c.world) * c.stage_slice);
}

// ---- element semantics ------------------------------------------------------
template <int DT>
struct Elem;

template <>
struct Elem<BL_DTYPE_FP32> {
  using acc_t = float;
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
};
template <>
struct Elem<BL_DTYPE_BF16> {
  using acc_t = float;
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
           d = unpack_bf16x2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                      pack_bf16x2(f[6], f[7]));
  }
};
template <>
struct Elem<BL_DTYPE_FP16> {
  using acc_t = float;
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 x = __half22float2(h);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <__nv_fp8_interpretation_t KIND>
struct ElemFp8 {
  using acc_t = float;
  static constexpr int N = 16;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        __half2_raw hr =
            __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t((w[i] >> (16 * j)) & 0xffffu), KIND);
        __half2 h = *reinterpret_cast<__half2*>(&hr);
        float2 x = __half22float2(h);
        f[4 * i + 2 * j] = x.x;
        f[4 * i + 2 * j + 1] = x.y;
      }
    }
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i], f[4 * i + 1]), __NV_SATFINITE, KIND);
      uint32_t hi =
          __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2], f[4 * i + 3]), __NV_SATFINITE, KIND);
      w[i] = (lo & 0xffffu) | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Elem<BL_DTYPE_FP8E4M3> : ElemFp8<__NV_E4M3> {};
template <>
struct Elem<BL_DTYPE_FP8E5M2> : ElemFp8<__NV_E5M2> {};
template <>
struct Elem<BL_DTYPE_FP64> {
  using acc_t = double;
  static constexpr int N = 2;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    f[0] = __hiloint2double(int(v.y), int(v.x));
    f[1] = __hiloint2double(int(v.w), int(v.z));
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    return make_uint4(uint32_t(__double2loint(f[0])), uint32_t(__double2hiint(f[0])),
                      uint32_t(__double2loint(f[1])), uint32_t(__double2hiint(f[1])));
  }
};
template <>
struct Elem<BL_DTYPE_U8> {  // wrapping add: sum in 32 bits, keep the low byte
  using acc_t = uint32_t;
  static constexpr int N = 16;
  static __device__ __forceinline__ void unpack(uint4 v, acc_t* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) f[4 * i + j] = (w[i] >> (8 * j)) & 0xffu;
  }
  static __device__ __forceinline__ uint4 pack(const acc_t* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (f[4 * i] & 0xffu) | ((f[4 * i + 1] & 0xffu) << 8) | ((f[4 * i + 2] & 0xffu) << 16) |
             ((f[4 * i + 3] & 0xffu) << 24);
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <int DT>
__device__ __forceinline__ void acc_add(typename Elem<DT>::acc_t* acc, uint4 v) {
  typename Elem<DT>::acc_t t[Elem<DT>::N];
  Elem<DT>::unpack(v, t);
#pragma unroll
  for (int i = 0; i < Elem<DT>::N; ++i) acc[i] += t[i];
}

__device__ __forceinline__ uint4 scrub(uint4 v) {
  // a payload word equal to the "unwritten" pattern becomes +0.0 (same value)
  if (v.x == kUnwritten) v.x = 0;
  if (v.y == kUnwritten) v.y = 0;
  if (v.z == kUnwritten) v.z = 0;
  if (v.w == kUnwritten) v.w = 0;
  return v;
}
__device__ __forceinline__ bool landed(uint4 v) {
  return v.x != kUnwritten && v.y != kUnwritten && v.z != kUnwritten && v.w != kUnwritten;
}

// Poll one 16-byte vector of a Lamport inbox until all four words landed.
__device__ __forceinline__ bool poll_vec(const Comm& c, const char* p, uint4& v, int from) {
  v = ld_volatile_v4(p);
  if (landed(v)) return true;
  const uint32_t* abortw = sig_of(c, c.rank) + kSigAbort;
  uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  for (;;) {
    v = ld_volatile_v4(p);
    if (landed(v)) return true;
    if ((++polls & 255u) == 0u) {
      if (ld_volatile_u32(abortw)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_timeout(c, 2, P_LAMPORT, from, v.x, kUnwritten);
        return false;
      }
    }
  }
}

}  // namespace bl
