#ifndef _GNU_SOURCE
#define _GNU_SOURCE  // struct ucred
#endif
// SPDX-License-Identifier: MIT
//
// Host side of the symmetric heap: driver entry points, arena layout,
// symmetric allocator, single-process bring-up, and the SPMD rendezvous that
// passes VMM file descriptors between rank processes over one unix socket
// (rank 0 is the hub).  Role of the reference's registration + pool +
// rendezvous code (torch_ext/barlink_sm86/core.cu:1128-1179, 1188-1507,
// 1948-2211), with cuMem/NVLS in place of BAR1/dma-buf.
#include "heap.h"

#include <errno.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/prctl.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>

namespace bl {

void set_err(char* err, size_t errlen, const char* fmt, ...) {
  if (!err || errlen == 0) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err, errlen, fmt, ap);
  va_end(ap);
}

// ---------------------------------------------------------------------------
// driver entry points
// ---------------------------------------------------------------------------
static DriverApi g_api;
static int g_api_state = 0;  // 0 unknown, 1 ok, -1 absent
static std::mutex g_api_mu;

template <typename F>
static bool lookup(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

const DriverApi* driver(char* err, size_t errlen) {
  std::lock_guard<std::mutex> g(g_api_mu);
  if (g_api_state == 1) return &g_api;
  if (g_api_state == -1) {
    set_err(err, errlen, "barlink: no CUDA driver on this machine");
    return nullptr;
  }
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    g_api_state = -1;
    set_err(err, errlen, "barlink: no CUDA device visible (cudaGetDeviceCount)");
    return nullptr;
  }
  bool ok = true;
#define BL_LOOKUP(sym) ok = ok && lookup(#sym, &g_api.sym)
  BL_LOOKUP(cuMemCreate);
  BL_LOOKUP(cuMemRelease);
  BL_LOOKUP(cuMemAddressReserve);
  BL_LOOKUP(cuMemAddressFree);
  BL_LOOKUP(cuMemMap);
  BL_LOOKUP(cuMemUnmap);
  BL_LOOKUP(cuMemSetAccess);
  BL_LOOKUP(cuMemGetAllocationGranularity);
  BL_LOOKUP(cuMemExportToShareableHandle);
  BL_LOOKUP(cuMemImportFromShareableHandle);
  BL_LOOKUP(cuMulticastCreate);
  BL_LOOKUP(cuMulticastAddDevice);
  BL_LOOKUP(cuMulticastBindMem);
  BL_LOOKUP(cuMulticastUnbind);
  BL_LOOKUP(cuMulticastGetGranularity);
  BL_LOOKUP(cuDeviceGet);
  BL_LOOKUP(cuDeviceGetAttribute);
  BL_LOOKUP(cuGetErrorString);
  BL_LOOKUP(cuTensorMapEncodeTiled);
#undef BL_LOOKUP
  if (!ok) {
    g_api_state = -1;
    set_err(err, errlen, "barlink: CUDA driver lacks a VMM/multicast/tensor-map entry point");
    return nullptr;
  }
  g_api_state = 1;
  return &g_api;
}

static const char* cu_str(const DriverApi* d, CUresult r) {
  const char* s = nullptr;
  if (d && d->cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown CUresult";
}

#define CU_TRY(call, what)                                                            \
  do {                                                                                \
    CUresult _r = (call);                                                             \
    if (_r != CUDA_SUCCESS) {                                                         \
      set_err(err, errlen, "barlink: %s failed: %s (%d)", what, cu_str(d, _r), (int)_r); \
      return -1;                                                                      \
    }                                                                                 \
  } while (0)

#define RT_TRY(call, what)                                                       \
  do {                                                                           \
    cudaError_t _e = (call);                                                     \
    if (_e != cudaSuccess) {                                                     \
      set_err(err, errlen, "barlink: %s failed: %s", what, cudaGetErrorString(_e)); \
      return -1;                                                                 \
    }                                                                            \
  } while (0)

// ---------------------------------------------------------------------------
// layout and allocator
// ---------------------------------------------------------------------------
static size_t round_down(size_t v, size_t a) { return v / a * a; }
static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

Layout compute_layout(size_t pool_bytes, int world) {
  const size_t K64 = 65536;
  Layout L{};
  L.pool_bytes = pool_bytes;
  L.sig_off = pool_bytes - kSigBytes;
  L.p2p_slice = round_down(std::min<size_t>(std::max<size_t>(pool_bytes / 64, K64), 4u << 20), K64);
  L.p2p_off = L.sig_off - size_t(world) * L.p2p_slice;
  L.lamport_slice =
      round_down(std::min<size_t>(std::max<size_t>(pool_bytes / 256, K64 / 2), 1u << 20), 4096);
  L.lamport_off = round_down(L.p2p_off - 3 * size_t(world) * L.lamport_slice, K64);
  // two staging buffers (taken in turn by successive staged collectives), each with an inbox
  // half and an outbox half of world slices
  L.stage_slice = round_down(pool_bytes / 4 / (4 * size_t(world)), 4096);
  L.stage_off = round_down(L.lamport_off - 4 * size_t(world) * L.stage_slice, K64);
  L.user_bytes = L.stage_off;
  return L;
}

int64_t arena_alloc(Arena& a, size_t user_bytes, size_t bytes) {
  if (bytes == 0) bytes = 16;
  bytes = round_up(bytes, 16);
  const size_t align = bytes >= (2u << 20) ? (2u << 20) : 256;
  // first fit in the free list
  for (auto it = a.free_list.begin(); it != a.free_list.end(); ++it) {
    size_t off = round_up(it->first, align);
    size_t pad = off - it->first;
    if (it->second >= pad + bytes) {
      size_t blk_off = it->first, blk_len = it->second;
      a.free_list.erase(it);
      if (pad) a.free_list[blk_off] = pad;
      size_t rest = blk_len - pad - bytes;
      if (rest) a.free_list[off + bytes] = rest;
      return int64_t(off);
    }
  }
  size_t off = round_up(a.bump, align);
  if (off + bytes > user_bytes) return -1;
  if (off > a.bump) a.free_list[a.bump] = off - a.bump;
  a.bump = off + bytes;
  return int64_t(off);
}

bool arena_free(Arena& a, size_t off, size_t bytes) {
  if (bytes == 0) bytes = 16;
  bytes = round_up(bytes, 16);
  if (off + bytes > a.bump) return false;
  // overlap check against existing free blocks
  auto nx = a.free_list.lower_bound(off);
  if (nx != a.free_list.end() && nx->first < off + bytes) return false;
  if (nx != a.free_list.begin()) {
    auto pv = std::prev(nx);
    if (pv->first + pv->second > off) return false;
  }
  a.free_list[off] = bytes;
  // merge with neighbours
  auto it = a.free_list.find(off);
  if (it != a.free_list.begin()) {
    auto pv = std::prev(it);
    if (pv->first + pv->second == it->first) {
      pv->second += it->second;
      a.free_list.erase(it);
      it = pv;
    }
  }
  auto nn = std::next(it);
  if (nn != a.free_list.end() && it->first + it->second == nn->first) {
    it->second += nn->second;
    a.free_list.erase(nn);
  }
  // give the tail back to the bump pointer
  if (it->first + it->second == a.bump) {
    a.bump = it->first;
    a.free_list.erase(it);
  }
  return true;
}

// ---------------------------------------------------------------------------
// arena creation / mapping
// ---------------------------------------------------------------------------
static CUmemAllocationProp arena_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

static int map_arena(const DriverApi* d, Arena& a, size_t bytes, const int* devs, int ndev,
                     char* err, size_t errlen) {
  CU_TRY(d->cuMemAddressReserve(&a.va, bytes, 2u << 20, 0, 0), "cuMemAddressReserve");
  CU_TRY(d->cuMemMap(a.va, bytes, 0, a.handle, 0), "cuMemMap");
  std::vector<CUmemAccessDesc> acc;
  for (int i = 0; i < ndev; ++i) {
    bool dup = false;
    for (int j = 0; j < i; ++j) dup = dup || devs[j] == devs[i];
    if (dup) continue;
    CUmemAccessDesc ad;
    memset(&ad, 0, sizeof(ad));
    ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    ad.location.id = devs[i];
    ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc.push_back(ad);
  }
  CU_TRY(d->cuMemSetAccess(a.va, bytes, acc.data(), acc.size()), "cuMemSetAccess");
  return 0;
}

static bool env_flag(const char* name, bool dflt) {
  const char* v = getenv(name);
  if (!v || !*v) return dflt;
  return !(v[0] == '0' || v[0] == 'n' || v[0] == 'N' || v[0] == 'f' || v[0] == 'F');
}

static int mc_supported(const DriverApi* d, int device) {
  CUdevice dev;
  int v = 0;
  if (d->cuDeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  if (d->cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
    return 0;
  return v;
}

static size_t pool_granularity(const DriverApi* d, int device, int world, bool want_mc) {
  size_t g = 2u << 20;
  CUmemAllocationProp p = arena_prop(device);
  size_t gm = 0;
  if (d->cuMemGetAllocationGranularity(&gm, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) ==
          CUDA_SUCCESS &&
      gm > g)
    g = gm;
  if (want_mc) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = 2u << 20;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d->cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
            CUDA_SUCCESS &&
        mg > g)
      g = mg;
  }
  return g;
}

// device-side bring-up shared by both modes: signal pad cleared, Lamport
// buffers filled with the "not yet written" word, status block, comm copies.
int init_device_state(blCtx* ctx, char* err, size_t errlen);  // comm_kernels.cu

static void fill_layout(blCtx* ctx) {
  Layout L = compute_layout(ctx->pool_bytes, ctx->world);
  ctx->user_bytes = L.user_bytes;
  Comm& c = ctx->layout;
  memset(&c, 0, sizeof(c));
  c.sig_off = L.sig_off;
  c.stage_off = L.stage_off;
  c.stage_slice = L.stage_slice;
  c.lamport_off = L.lamport_off;
  c.lamport_slice = L.lamport_slice;
  c.p2p_off = L.p2p_off;
  c.p2p_slice = L.p2p_slice;
}

static void read_timeout_env(blCtx* ctx) {
  const char* t = getenv("BL_WAIT_TIMEOUT_MS");
  if (t && *t) {
    long v = strtol(t, nullptr, 10);
    if (v > 0 && v < 600000) ctx->timeout_ms = unsigned(v);
  }
}

}  // namespace bl

using namespace bl;

// ---------------------------------------------------------------------------
// single-process mode
// ---------------------------------------------------------------------------
extern "C" int bl_init(blCtx** out, const int* devices, int ndev, size_t poolBytes, char* err,
                       size_t errlen) {
  if (!out || !devices || ndev < 1 || ndev > kMaxRanks) {
    set_err(err, errlen, "barlink: bl_init needs 1..%d devices (got %d)", kMaxRanks, ndev);
    return -1;
  }
  if (poolBytes < (8u << 20)) {
    set_err(err, errlen, "barlink: pool must be at least 8 MiB per rank");
    return -1;
  }
  const DriverApi* d = driver(err, errlen);
  if (!d) return -1;
  int ngpu = 0;
  RT_TRY(cudaGetDeviceCount(&ngpu), "cudaGetDeviceCount");
  bool distinct = true;
  for (int i = 0; i < ndev; ++i) {
    if (devices[i] < 0 || devices[i] >= ngpu) {
      set_err(err, errlen, "barlink: device ordinal %d out of range (box has %d GPUs)",
              devices[i], ngpu);
      return -1;
    }
    for (int j = 0; j < i; ++j) distinct = distinct && devices[j] != devices[i];
  }
  // peer access between distinct devices
  for (int i = 0; i < ndev; ++i)
    for (int j = 0; j < ndev; ++j) {
      if (devices[i] == devices[j]) continue;
      int can = 0;
      RT_TRY(cudaDeviceCanAccessPeer(&can, devices[i], devices[j]), "cudaDeviceCanAccessPeer");
      if (!can) {
        set_err(err, errlen, "barlink: GPU %d cannot access GPU %d (no P2P path)", devices[i],
                devices[j]);
        return -1;
      }
      RT_TRY(cudaSetDevice(devices[i]), "cudaSetDevice");
      cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        set_err(err, errlen, "barlink: cudaDeviceEnablePeerAccess(%d->%d): %s", devices[i],
                devices[j], cudaGetErrorString(e));
        return -1;
      }
      cudaGetLastError();
    }
  blCtx* ctx = new blCtx();
  ctx->peer_mode = false;
  ctx->world = ndev;
  read_timeout_env(ctx);
  bool want_mc = distinct && ndev > 1 && env_flag("BL_NVLS", false);
  for (int i = 0; i < ndev && want_mc; ++i) want_mc = mc_supported(d, devices[i]) != 0;
  RT_TRY(cudaSetDevice(devices[0]), "cudaSetDevice");
  RT_TRY(cudaFree(0), "context init");
  size_t gran = pool_granularity(d, devices[0], ndev, want_mc);
  ctx->pool_bytes = round_up(poolBytes, gran);
  fill_layout(ctx);
  auto fail = [&](void) {
    bl_shutdown(ctx);
    return -1;
  };
  for (int i = 0; i < ndev; ++i) {
    Arena& a = ctx->arena[i];
    a.device = devices[i];
    if (cudaSetDevice(devices[i]) != cudaSuccess || cudaFree(0) != cudaSuccess) {
      set_err(err, errlen, "barlink: cannot initialise GPU %d", devices[i]);
      return fail();
    }
    CUmemAllocationProp p = arena_prop(devices[i]);
    CUresult r = d->cuMemCreate(&a.handle, ctx->pool_bytes, &p, 0);
    if (r != CUDA_SUCCESS) {
      set_err(err, errlen, "barlink: cuMemCreate(%zu MiB) on GPU %d failed: %s",
              ctx->pool_bytes >> 20, devices[i], cu_str(d, r));
      return fail();
    }
    a.owned = true;
    if (map_arena(d, a, ctx->pool_bytes, devices, ndev, err, errlen) != 0) return fail();
  }
  if (want_mc) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = ndev;
    mp.size = ctx->pool_bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    bool ok = d->cuMulticastCreate(&ctx->mc_handle, &mp) == CUDA_SUCCESS;
    for (int i = 0; i < ndev && ok; ++i) {
      CUdevice dev;
      ok = d->cuDeviceGet(&dev, devices[i]) == CUDA_SUCCESS &&
           d->cuMulticastAddDevice(ctx->mc_handle, dev) == CUDA_SUCCESS;
    }
    for (int i = 0; i < ndev && ok; ++i)
      ok = d->cuMulticastBindMem(ctx->mc_handle, 0, ctx->arena[i].handle, 0, ctx->pool_bytes,
                                 0) == CUDA_SUCCESS;
    if (ok) {
      Arena tmp;
      tmp.handle = ctx->mc_handle;
      ok = map_arena(d, tmp, ctx->pool_bytes, devices, ndev, err, errlen) == 0;
      ctx->mc_va = tmp.va;
    }
    ctx->has_mc = ok;
    if (!ok && ctx->mc_handle) {
      d->cuMemRelease(ctx->mc_handle);
      ctx->mc_handle = 0;
      ctx->mc_va = 0;
    }
  }
  if (init_device_state(ctx, err, errlen) != 0) return fail();
  *out = ctx;
  return 0;
}

// ---------------------------------------------------------------------------
// SPMD rendezvous over one unix socket (rank 0 = hub)
// ---------------------------------------------------------------------------
namespace {

struct Hello {
  uint32_t magic;
  int32_t rank, world;
  uint64_t pool_bytes;
  int32_t mc_ok;
  int32_t pad;
};
constexpr uint32_t kMagic = 0x626c3230;  // "bl20"

int send_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      return -1;
    }
    p += w;
    n -= size_t(w);
  }
  return 0;
}
int recv_all(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n) {
    ssize_t r = recv(fd, p, n, 0);
    if (r == 0) return -1;
    if (r < 0) {
      if (errno == EINTR) continue;
      return -1;
    }
    p += r;
    n -= size_t(r);
  }
  return 0;
}
// one message carrying `nfds` descriptors and a small payload
int send_fds(int sock, const int* fds, int nfds, const void* payload, size_t len) {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov;
  iov.iov_base = const_cast<void*>(payload);
  iov.iov_len = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int) * 16)];
  memset(ctrl, 0, sizeof(ctrl));
  if (nfds > 0) {
    msg.msg_control = ctrl;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * nfds);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * nfds);
    memcpy(CMSG_DATA(c), fds, sizeof(int) * nfds);
  }
  for (;;) {
    ssize_t w = sendmsg(sock, &msg, MSG_NOSIGNAL);
    if (w < 0 && errno == EINTR) continue;
    return w == ssize_t(len) ? 0 : -1;
  }
}
int recv_fds(int sock, int* fds, int nfds, void* payload, size_t len) {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov;
  iov.iov_base = payload;
  iov.iov_len = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int) * 16)];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t r;
  do {
    r = recvmsg(sock, &msg, MSG_WAITALL);
  } while (r < 0 && errno == EINTR);
  if (r != ssize_t(len)) return -1;
  int got = 0;
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int n = int((c->cmsg_len - CMSG_LEN(0)) / sizeof(int));
      for (int i = 0; i < n && got < nfds; ++i)
        memcpy(&fds[got++], CMSG_DATA(c) + sizeof(int) * i, sizeof(int));
    }
  }
  return got == nfds ? 0 : -1;
}

void set_sock_timeout(int fd, int seconds) {
  struct timeval tv;
  tv.tv_sec = seconds;
  tv.tv_usec = 0;
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

struct Hub {
  int rank = 0, world = 1;
  int listen_fd = -1;
  int conn[kMaxRanks];  // hub: socket to each rank; others: conn[0] = socket to hub
  Hub() {
    for (int& c : conn) c = -1;
  }
  void close_all() {
    for (int& c : conn)
      if (c >= 0) {
        close(c);
        c = -1;
      }
    if (listen_fd >= 0) {
      close(listen_fd);
      listen_fd = -1;
    }
  }
  // all-ranks AND of a status byte; doubles as a barrier
  int all_and(int mine, int* result) {
    unsigned char b = mine ? 1 : 0;
    if (rank == 0) {
      unsigned char acc = b;
      for (int r = 1; r < world; ++r) {
        unsigned char x;
        if (recv_all(conn[r], &x, 1) != 0) return -1;
        acc = acc && x;
      }
      for (int r = 1; r < world; ++r)
        if (send_all(conn[r], &acc, 1) != 0) return -1;
      *result = acc;
    } else {
      if (send_all(conn[0], &b, 1) != 0) return -1;
      unsigned char x;
      if (recv_all(conn[0], &x, 1) != 0) return -1;
      *result = x;
    }
    return 0;
  }
};

int rendezvous_timeout_s() {
  const char* t = getenv("BL_RENDEZVOUS_TIMEOUT_S");
  int v = t ? atoi(t) : 0;
  return v > 0 ? v : 120;
}

}  // namespace

extern "C" int bl_init_peer(blCtx** out, int device, size_t poolBytes, const char* sockPath,
                            int rank, int world, char* err, size_t errlen) {
  if (!out || !sockPath || world < 2 || world > kMaxRanks || rank < 0 || rank >= world) {
    set_err(err, errlen, "barlink: bl_init_peer needs 2..%d ranks and 0 <= rank < world (rank %d, world %d)",
            kMaxRanks, rank, world);
    return -1;
  }
  if (poolBytes < (8u << 20)) {
    set_err(err, errlen, "barlink: pool must be at least 8 MiB per rank");
    return -1;
  }
  const DriverApi* d = driver(err, errlen);
  if (!d) return -1;
  RT_TRY(cudaSetDevice(device), "cudaSetDevice");
  RT_TRY(cudaFree(0), "context init");

  blCtx* ctx = new blCtx();
  ctx->peer_mode = true;
  ctx->world = world;
  ctx->rank = rank;
  read_timeout_env(ctx);
  Hub hub;
  hub.rank = rank;
  hub.world = world;
  const int tmo = rendezvous_timeout_s();
  auto fail = [&](void) {
    hub.close_all();
    bl_shutdown(ctx);
    return -1;
  };

  bool want_mc = env_flag("BL_NVLS", false) && mc_supported(d, device) != 0;
  size_t gran = pool_granularity(d, device, world, want_mc);
  ctx->pool_bytes = round_up(poolBytes, gran);
  fill_layout(ctx);

  // my arena
  Arena& mine = ctx->arena[rank];
  mine.device = device;
  {
    CUmemAllocationProp p = arena_prop(device);
    CUresult r = d->cuMemCreate(&mine.handle, ctx->pool_bytes, &p, 0);
    if (r != CUDA_SUCCESS) {
      set_err(err, errlen, "barlink: cuMemCreate(%zu MiB) on GPU %d failed: %s",
              ctx->pool_bytes >> 20, device, cu_str(d, r));
      return fail();
    }
    mine.owned = true;
    r = d->cuMemExportToShareableHandle(&mine.fd, mine.handle,
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
      set_err(err, errlen, "barlink: cuMemExportToShareableHandle failed: %s", cu_str(d, r));
      return fail();
    }
  }

  // ---- connect -----------------------------------------------------------
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  if (strlen(sockPath) >= sizeof(addr.sun_path)) {
    set_err(err, errlen, "barlink: socket path too long: %s", sockPath);
    return fail();
  }
  strcpy(addr.sun_path, sockPath);
  int fds[kMaxRanks + 1];
  for (int& f : fds) f = -1;
  int mc_fd = -1;

  if (rank == 0) {
    unlink(sockPath);
    hub.listen_fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (hub.listen_fd < 0 || bind(hub.listen_fd, (struct sockaddr*)&addr, sizeof(addr)) != 0 ||
        listen(hub.listen_fd, kMaxRanks) != 0) {
      set_err(err, errlen, "barlink: rank 0 cannot listen on %s: %s", sockPath, strerror(errno));
      return fail();
    }
    set_sock_timeout(hub.listen_fd, tmo);
    fds[0] = mine.fd;
    int mc_all = want_mc ? 1 : 0;
    for (int n = 1; n < world; ++n) {
      int c = accept(hub.listen_fd, nullptr, nullptr);
      if (c < 0) {
        set_err(err, errlen,
                "barlink: rank 0 saw only %d of %d ranks connect to %s within %d s (%s)", n,
                world, sockPath, tmo, strerror(errno));
        return fail();
      }
      set_sock_timeout(c, tmo);
      {
        // memory handles go only to processes of the same user
        struct ucred cred;
        socklen_t clen = sizeof(cred);
        if (getsockopt(c, SOL_SOCKET, SO_PEERCRED, &cred, &clen) != 0 || cred.uid != geteuid()) {
          set_err(err, errlen, "barlink: a process of another user connected to %s; refused", sockPath);
          close(c);
          return fail();
        }
      }
      Hello h;
      int fd = -1;
      if (recv_fds(c, &fd, 1, &h, sizeof(h)) != 0 || h.magic != kMagic) {
        set_err(err, errlen, "barlink: bad hello on %s", sockPath);
        close(c);
        return fail();
      }
      if (h.world != world || h.rank <= 0 || h.rank >= world || hub.conn[h.rank] >= 0 ||
          h.pool_bytes != ctx->pool_bytes) {
        set_err(err, errlen,
                "barlink: rank %d joined with world %d pool %llu B, rank 0 has world %d pool "
                "%zu B (every rank must pass the same BL_POOL_MB and world size)",
                h.rank, h.world, (unsigned long long)h.pool_bytes, world, ctx->pool_bytes);
        close(c);
        return fail();
      }
      hub.conn[h.rank] = c;
      fds[h.rank] = fd;
      mc_all = mc_all && h.mc_ok;
    }
    unlink(sockPath);
    want_mc = mc_all != 0;
    if (want_mc) {
      CUmulticastObjectProp mp;
      memset(&mp, 0, sizeof(mp));
      mp.numDevices = world;
      mp.size = ctx->pool_bytes;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      if (d->cuMulticastCreate(&ctx->mc_handle, &mp) != CUDA_SUCCESS ||
          d->cuMemExportToShareableHandle(&mc_fd, ctx->mc_handle,
                                          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                          0) != CUDA_SUCCESS) {
        want_mc = false;
        if (ctx->mc_handle) d->cuMemRelease(ctx->mc_handle);
        ctx->mc_handle = 0;
        mc_fd = -1;
      }
    }
    // hand every rank all descriptors (+ multicast)
    for (int r = 1; r < world; ++r) {
      int send[kMaxRanks + 1];
      int n = 0;
      for (int i = 0; i < world; ++i) send[n++] = fds[i];
      if (want_mc) send[n++] = mc_fd;
      Hello h{kMagic, 0, world, ctx->pool_bytes, want_mc ? 1 : 0, 0};
      if (send_fds(hub.conn[r], send, n, &h, sizeof(h)) != 0) {
        set_err(err, errlen, "barlink: rank 0 could not hand descriptors to rank %d", r);
        return fail();
      }
    }
  } else {
    int c = -1;
    struct timespec ts = {0, 50 * 1000 * 1000};
    for (int tries = 0; tries < tmo * 20; ++tries) {
      c = socket(AF_UNIX, SOCK_STREAM, 0);
      if (c >= 0 && connect(c, (struct sockaddr*)&addr, sizeof(addr)) == 0) break;
      if (c >= 0) close(c);
      c = -1;
      nanosleep(&ts, nullptr);
    }
    if (c < 0) {
      set_err(err, errlen, "barlink: rank %d could not reach rank 0 on %s within %d s", rank,
              sockPath, tmo);
      return fail();
    }
    set_sock_timeout(c, tmo);
    hub.conn[0] = c;
    Hello h{kMagic, rank, world, ctx->pool_bytes, want_mc ? 1 : 0, 0};
    if (send_fds(c, &mine.fd, 1, &h, sizeof(h)) != 0) {
      set_err(err, errlen, "barlink: rank %d could not send its descriptor", rank);
      return fail();
    }
    // The reply carries world (+1) descriptors; its size tells which.
    Hello rh;
    int got[kMaxRanks + 1];
    // try with the multicast descriptor first: the header says whether it is there
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    struct iovec iov;
    iov.iov_base = &rh;
    iov.iov_len = sizeof(rh);
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int) * 16)];
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t rr;
    do {
      rr = recvmsg(c, &msg, MSG_WAITALL);
    } while (rr < 0 && errno == EINTR);
    int ngot = 0;
    if (rr == ssize_t(sizeof(rh))) {
      for (struct cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm; cm = CMSG_NXTHDR(&msg, cm))
        if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) {
          int n = int((cm->cmsg_len - CMSG_LEN(0)) / sizeof(int));
          for (int i = 0; i < n && ngot < kMaxRanks + 1; ++i)
            memcpy(&got[ngot++], CMSG_DATA(cm) + sizeof(int) * i, sizeof(int));
        }
    }
    if (rr != ssize_t(sizeof(rh)) || rh.magic != kMagic || ngot != world + (rh.mc_ok ? 1 : 0)) {
      set_err(err, errlen,
              "barlink: rank %d got no (or a malformed) descriptor table from rank 0 "
              "(a rank died, or pool sizes differ)",
              rank);
      return fail();
    }
    for (int i = 0; i < world; ++i) fds[i] = got[i];
    want_mc = rh.mc_ok != 0;
    if (want_mc) mc_fd = got[world];
  }

  // ---- import + map every peer arena --------------------------------------
  int one_dev[1] = {device};
  for (int r = 0; r < world; ++r) {
    Arena& a = ctx->arena[r];
    if (r != rank) {
      a.device = -1;
      CUresult cr = d->cuMemImportFromShareableHandle(
          &a.handle, (void*)(uintptr_t)fds[r], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (cr != CUDA_SUCCESS) {
        set_err(err, errlen, "barlink: rank %d cannot import rank %d's arena: %s", rank, r,
                cu_str(d, cr));
        return fail();
      }
      if (rank != 0 || true) close(fds[r]);
    }
    if (map_arena(d, a, ctx->pool_bytes, one_dev, 1, err, errlen) != 0) return fail();
  }

  // ---- multicast ---------------------------------------------------------
  int ok = 1, all = 0;
  if (want_mc) {
    if (rank != 0) {
      ok = d->cuMemImportFromShareableHandle(&ctx->mc_handle, (void*)(uintptr_t)mc_fd,
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) ==
           CUDA_SUCCESS;
    }
    if (mc_fd >= 0) close(mc_fd);
    CUdevice dev;
    ok = ok && d->cuDeviceGet(&dev, device) == CUDA_SUCCESS &&
         d->cuMulticastAddDevice(ctx->mc_handle, dev) == CUDA_SUCCESS;
    if (hub.all_and(ok, &all) != 0) {
      set_err(err, errlen, "barlink: rendezvous broke while adding devices to the multicast object");
      return fail();
    }
    if (all) {
      ok = d->cuMulticastBindMem(ctx->mc_handle, 0, mine.handle, 0, ctx->pool_bytes, 0) ==
           CUDA_SUCCESS;
      if (ok) {
        Arena tmp;
        tmp.handle = ctx->mc_handle;
        char e2[128];
        ok = map_arena(d, tmp, ctx->pool_bytes, one_dev, 1, e2, sizeof(e2)) == 0;
        ctx->mc_va = tmp.va;
      }
      if (hub.all_and(ok, &all) != 0) {
        set_err(err, errlen, "barlink: rendezvous broke while binding the multicast object");
        return fail();
      }
    }
    ctx->has_mc = all != 0;
    if (!ctx->has_mc) {
      if (ctx->mc_va) {
        d->cuMemUnmap(ctx->mc_va, ctx->pool_bytes);
        d->cuMemAddressFree(ctx->mc_va, ctx->pool_bytes);
        ctx->mc_va = 0;
      }
      if (ctx->mc_handle) d->cuMemRelease(ctx->mc_handle);
      ctx->mc_handle = 0;
    }
  }

  if (init_device_state(ctx, err, errlen) != 0) return fail();
  // everyone's pad is cleared before anyone signals
  if (hub.all_and(1, &all) != 0 || !all) {
    set_err(err, errlen, "barlink: a rank failed during device bring-up");
    return fail();
  }
  hub.close_all();
  if (mine.fd >= 0) {
    close(mine.fd);
    mine.fd = -1;
  }
  bl_drop_caps();
  *out = ctx;
  return 0;
}

namespace bl {
void free_device_state(blCtx* ctx);  // comm_kernels.cu
}

extern "C" void bl_shutdown(blCtx* ctx) {
  if (!ctx) return;
  char e[64];
  const DriverApi* d = driver(e, sizeof(e));
  int cur = 0;
  cudaGetDevice(&cur);
  for (int r = 0; r < ctx->world; ++r)
    if (ctx->arena[r].device >= 0) {
      cudaSetDevice(ctx->arena[r].device);
      cudaDeviceSynchronize();
    }
  free_device_state(ctx);
  if (d) {
    if (ctx->mc_va) {
      d->cuMemUnmap(ctx->mc_va, ctx->pool_bytes);
      d->cuMemAddressFree(ctx->mc_va, ctx->pool_bytes);
    }
    if (ctx->mc_handle) {
      for (int r = 0; r < ctx->world; ++r)
        if (ctx->arena[r].owned && ctx->arena[r].device >= 0 && ctx->has_mc) {
          CUdevice dev;
          if (d->cuDeviceGet(&dev, ctx->arena[r].device) == CUDA_SUCCESS)
            d->cuMulticastUnbind(ctx->mc_handle, dev, 0, ctx->pool_bytes);
        }
      d->cuMemRelease(ctx->mc_handle);
    }
    for (int r = 0; r < ctx->world; ++r) {
      Arena& a = ctx->arena[r];
      if (a.va) {
        d->cuMemUnmap(a.va, ctx->pool_bytes);
        d->cuMemAddressFree(a.va, ctx->pool_bytes);
      }
      if (a.handle) d->cuMemRelease(a.handle);
      if (a.fd >= 0) close(a.fd);
    }
  }
  cudaSetDevice(cur);
  cudaGetLastError();
  delete ctx;
}

// ---------------------------------------------------------------------------
// small accessors and the allocator front
// ---------------------------------------------------------------------------
extern "C" int bl_is_peer(const blCtx* ctx) { return ctx && ctx->peer_mode; }
extern "C" int bl_world(const blCtx* ctx) { return ctx ? ctx->world : 0; }
extern "C" int bl_rank(const blCtx* ctx) { return ctx ? ctx->rank : -1; }
extern "C" int bl_has_multicast(const blCtx* ctx) { return ctx && ctx->has_mc; }
extern "C" size_t bl_user_bytes(const blCtx* ctx) { return ctx ? ctx->user_bytes : 0; }
extern "C" size_t bl_max_chunk(const blCtx* ctx) {
  return ctx ? ctx->layout.stage_slice * size_t(ctx->world) : 0;
}

extern "C" size_t bl_p2p_chunk(const blCtx* ctx) { return ctx ? ctx->layout.p2p_slice : 0; }
extern "C" size_t bl_oneshot_max(const blCtx* ctx) { return ctx ? ctx->layout.lamport_slice : 0; }
extern "C" size_t bl_pool_bytes(const blCtx* ctx) { return ctx ? ctx->pool_bytes : 0; }

static int arena_index(const blCtx* ctx, int devIdx) {
  return ctx->peer_mode ? ctx->rank : devIdx;
}

extern "C" int bl_pool_alloc(blCtx* ctx, int devIdx, size_t bytes, void** ptrOut, char* err,
                             size_t errlen) {
  if (!ctx || !ptrOut) {
    set_err(err, errlen, "barlink: bl_pool_alloc on a null context");
    return -1;
  }
  int i = arena_index(ctx, devIdx);
  if (i < 0 || i >= ctx->world) {
    set_err(err, errlen, "barlink: arena index %d out of range (world %d)", devIdx, ctx->world);
    return -1;
  }
  std::lock_guard<std::mutex> g(ctx->mu);
  int64_t off = arena_alloc(ctx->arena[i], ctx->user_bytes, bytes);
  if (off < 0) {
    set_err(err, errlen,
            "barlink: pool of arena %d is full (%zu B asked, %zu MiB user zone; raise BL_POOL_MB)",
            i, bytes, ctx->user_bytes >> 20);
    return -1;
  }
  *ptrOut = reinterpret_cast<void*>(ctx->arena[i].va + size_t(off));
  return 0;
}

extern "C" int bl_pool_free(blCtx* ctx, int devIdx, void* ptr, size_t bytes) {
  if (!ctx) return -1;
  int i = arena_index(ctx, devIdx);
  if (i < 0 || i >= ctx->world) return -1;
  int64_t off = bl_pool_offset(ctx, devIdx, ptr);
  if (off < 0) return -1;
  std::lock_guard<std::mutex> g(ctx->mu);
  return arena_free(ctx->arena[i], size_t(off), bytes) ? 0 : -1;
}

extern "C" int64_t bl_pool_offset(const blCtx* ctx, int devIdx, const void* ptr) {
  if (!ctx) return -1;
  int i = arena_index(ctx, devIdx);
  if (i < 0 || i >= ctx->world) return -1;
  CUdeviceptr p = reinterpret_cast<CUdeviceptr>(ptr);
  CUdeviceptr b = ctx->arena[i].va;
  if (!b || p < b || p >= b + ctx->pool_bytes) return -1;
  return int64_t(p - b);
}

extern "C" void* bl_peer_ptr(const blCtx* ctx, int r, size_t offset) {
  if (!ctx || r < 0 || r >= ctx->world || offset >= ctx->pool_bytes) return nullptr;
  return reinterpret_cast<void*>(ctx->arena[r].va + offset);
}
extern "C" void* bl_multicast_ptr(const blCtx* ctx, size_t offset) {
  if (!ctx || !ctx->has_mc || offset >= ctx->pool_bytes) return nullptr;
  return reinterpret_cast<void*>(ctx->mc_va + offset);
}

extern "C" void bl_stats(const blCtx* ctx, unsigned long long* out) {
  for (int i = 0; i < BL_STAT_COUNT; ++i) out[i] = ctx ? ctx->stats[i] : 0;
}

extern "C" void bl_drop_caps(void) {
  // Clear the ambient set and every capability of this thread; harmless
  // when the process has none.
  prctl(PR_CAP_AMBIENT, PR_CAP_AMBIENT_CLEAR_ALL, 0, 0, 0);
  struct {
    uint32_t version;
    int pid;
  } hdr = {0x20080522u /* _LINUX_CAPABILITY_VERSION_3 */, 0};
  struct {
    uint32_t effective, permitted, inheritable;
  } data[2];
  memset(data, 0, sizeof(data));
  syscall(SYS_capset, &hdr, data);
}
