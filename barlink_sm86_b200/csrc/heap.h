// SPDX-License-Identifier: MIT
//
// Symmetric heap: one VMM arena per rank, mapped into every rank, optionally
// bound to one NVLS multicast object.  Takes the place of the reference's
// BAR1 registration chain and pool (torch_ext/barlink_sm86/core.cu:1000-1092
// structs, 1128-1179 allocator, 1188-1507 registration, 2062-2211 peer
// rendezvous): on an NVSwitch box no kernel module, driver patch or
// capability is involved, the arena is shared by POSIX file descriptor.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "bl_core.h"

namespace bl {

// ---- signal pad (u32 words at the tail of every arena) --------------------
constexpr int kMaxRanks = BL_MAX_RANKS;
constexpr int kMaxSlots = 256;        // independently syncing blocks per protocol
constexpr int kNumProtos = 24;
constexpr size_t kSigWords = 256 + size_t(kNumProtos) * kMaxSlots * kMaxRanks;
constexpr size_t kSigBytes = ((kSigWords * 4 + 65535) / 65536) * 65536;

enum Proto : int {
  P_BARRIER = 0,
  P_LAMPORT = 1,
  P_TWOSHOT = 2,
  P_NVLS = 3,
  P_ALLGATHER = 4,
  P_REDSCAT = 5,
  P_BCAST = 6,
  P_VERIFY = 7,
  P_PROBE = 8,
  P_P2P_DATA = 9,   // flag[slot 0][src] = ordinal of the message that landed
  P_P2P_RCPT = 10,  // flag[slot 0][dst] = ordinal that dst has consumed
  P_GEMM_RS = 11,
  P_AG_GEMM = 12,
  P_COPY = 13,
  P_USER0 = 14,
  P_ROWPUSH = 15,  // row-parallel GEMM that scatters its output tiles itself + the kernel that finishes the all-reduce
};

// word indices inside the pad
constexpr int kSigAbort = 0;
// Count of collectives of this rank that went through the staging zone (any protocol).  Call n
// uses staging buffer n & 1: a rank can only be two staged calls ahead of a peer after that
// peer has left the earlier one (every staged kernel waits for all peers at least once), so a
// buffer is never written while a peer still reads the previous call's data from it.
constexpr int kSigStageSeq = 1;
__host__ __device__ constexpr int sig_epoch(int proto) { return 16 + proto; }
__host__ __device__ constexpr int sig_ticket(int proto) { return 48 + proto; }
__host__ __device__ constexpr int sig_aux(int proto) { return 80 + proto; }
// per-peer ordinals of the p2p protocol (send to / recv from peer r)
__host__ __device__ constexpr int sig_p2p_send(int r) { return 112 + r; }
__host__ __device__ constexpr int sig_p2p_recv(int r) { return 120 + r; }
__host__ __device__ constexpr int sig_flag(int proto, int slot, int src) {
  return 256 + (proto * kMaxSlots + slot) * kMaxRanks + src;
}

// What a kernel needs to know about the link.  Passed by value.
struct Comm {
  int rank;
  int world;
  char* base[kMaxRanks];  // every rank's arena as mapped in this process
  char* mc;               // multicast mapping of the arenas, or nullptr
  size_t sig_off;         // signal pad
  size_t stage_off;       // staging zone: two buffers of (inbox half, outbox half), each half
                          // world slices of stage_slice bytes
  size_t stage_slice;     // capacity per source rank
  size_t lamport_off;     // 3 buffers of world * lamport_slice bytes
  size_t lamport_slice;
  size_t p2p_off;         // world inboxes of p2p_slice bytes
  size_t p2p_slice;
  uint64_t timeout_ns;    // bound of every device wait
  blStatus* status;       // host-mapped record of a wait that ran out
};

// Kernel parameter: one rank, or an array of ranks that share this GPU and
// are run as grid.y of one cooperative kernel.
struct CommPack {
  Comm c;
  const Comm* emu;  // device array, indexed by blockIdx.y, or nullptr
};

struct Arena {
  int device = -1;
  CUmemGenericAllocationHandle handle = 0;
  bool owned = false;      // created (not imported) here
  CUdeviceptr va = 0;      // mapping in this process
  int fd = -1;             // exported descriptor (creator only)
  // symmetric allocator over [0, user_bytes)
  size_t bump = 0;
  std::map<size_t, size_t> free_list;  // offset -> bytes
};

}  // namespace bl

struct blCtx {
  bool peer_mode = false;
  int world = 0;
  int rank = -1;              // peer mode only
  size_t pool_bytes = 0;      // per arena, rounded to the granularity
  size_t user_bytes = 0;
  bl::Arena arena[bl::kMaxRanks];
  // multicast
  bool has_mc = false;
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  // layout (same on every rank)
  bl::Comm layout{};          // rank/base filled per rank in comm_for()
  // single-process mode: local ranks grouped by GPU; ranks that share a GPU
  // run as grid.y of one cooperative kernel that reads group_dcomms[g][y]
  int ngroups = 0;
  int group_dev[bl::kMaxRanks] = {};
  int group_n[bl::kMaxRanks] = {};
  int group_ranks[bl::kMaxRanks][bl::kMaxRanks] = {};
  bl::Comm* group_dcomms[bl::kMaxRanks] = {};
  blStatus* h_status = nullptr;            // host-mapped, one per local rank
  blStatus* d_status = nullptr;            // device alias of h_status
  unsigned timeout_ms = 2000;
  // p2p side stream (peer mode)
  cudaStream_t send_stream = nullptr;
  cudaEvent_t ev_caller = nullptr, ev_send = nullptr;
  bool send_pending = false;
  // scratch counters on the device for verify
  unsigned long long* d_bad = nullptr;
  unsigned long long stats[BL_STAT_COUNT] = {};
  std::mutex mu;
  int sock_fd = -1;

  bl::Comm comm_for(int r) const {
    bl::Comm c = layout;
    c.rank = r;
    c.world = world;
    for (int i = 0; i < world; ++i) c.base[i] = reinterpret_cast<char*>(arena[i].va);
    c.mc = has_mc ? reinterpret_cast<char*>(mc_va) : nullptr;
    c.timeout_ns = uint64_t(timeout_ms) * 1000000ull;
    c.status = d_status ? d_status + (peer_mode ? 0 : r) : nullptr;
    return c;
  }
  int local_ranks() const { return peer_mode ? 1 : world; }
};

namespace bl {

void set_err(char* err, size_t errlen, const char* fmt, ...);

// Driver API entry points are looked up at run time so that the library
// loads on a machine without a GPU driver.
struct DriverApi {
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                          unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr,
                                  unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                       unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                            CUmemAllocationGranularity_flags);
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                           CUmemAllocationHandleType, unsigned long long);
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                             CUmemAllocationHandleType);
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t,
                                 CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long);
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                        CUmulticastGranularity_flags);
  CUresult (*cuDeviceGet)(CUdevice*, int);
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*cuGetErrorString)(CUresult, const char**);
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                     const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);
};
// nullptr (and a message) when no driver is present
const DriverApi* driver(char* err, size_t errlen);

// pure layout arithmetic, testable without a GPU
struct Layout {
  size_t pool_bytes, user_bytes, stage_off, stage_slice, lamport_off, lamport_slice, p2p_off,
      p2p_slice, sig_off;
};
Layout compute_layout(size_t pool_bytes, int world);

// host helpers of the GEMM launchers (gemm_kernels.cu)
int sm_count();
int pick_splits(int tiles, int kblocks, int sms, int want);
int make_tmap_kmajor(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t esize, CUtensorMap* out, char* err, size_t errlen, uint32_t box_cols = 64);

// symmetric allocator (host only state)
int64_t arena_alloc(Arena& a, size_t user_bytes, size_t bytes);
bool arena_free(Arena& a, size_t off, size_t bytes);

}  // namespace bl
