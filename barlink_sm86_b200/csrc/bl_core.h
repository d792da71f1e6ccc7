/* SPDX-License-Identifier: MIT
 *
 * barlink for B200 -- plain-C API of the link core.
 *
 * Capability parity with the reference's C API (torch_ext/barlink_sm86/core.h:
 * 30-195: init, init_peer, pool alloc/free, copy_, allreduce_, zero-copy
 * allreduce on arbitrary tensors, p2p send/recv, verify, readback, pool_move,
 * flag peek), redesigned for N <= 8 GPUs behind NVSwitch: buffers are VMM
 * allocations shared by POSIX file descriptor and mapped into every rank,
 * optionally bound to an NVLS multicast object, and every collective is one
 * kernel that loads and stores peer memory directly.
 *
 * No CUDA types cross this header: streams and pointers are void*.
 * Error convention: 0 on success, -1 on failure with a readable message in
 * err/errlen.  bl_verify returns the number of bad bytes (0 = clean,
 * ~0 = the run itself failed).
 */
#ifndef BARLINK_B200_CORE_H
#define BARLINK_B200_CORE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct blCtx blCtx;

#define BL_MAX_RANKS 8

/* element semantics of reductions (same numbering as the reference) */
#define BL_DTYPE_U8 0      /* wrapping add */
#define BL_DTYPE_FP32 1
#define BL_DTYPE_FP64 2
#define BL_DTYPE_BF16 3    /* summed in fp32, rounded once */
#define BL_DTYPE_FP8E4M3 4 /* summed in fp32, saturating convert */
#define BL_DTYPE_FP8E5M2 5
#define BL_DTYPE_FP16 6

/* all-reduce algorithms (BL_AR_ALGO) */
#define BL_ALGO_AUTO 0
#define BL_ALGO_ONESHOT 1
#define BL_ALGO_TWOSHOT 2
#define BL_ALGO_NVLS 3

/* Single-process mode: this process drives ndev arenas, one per entry of
 * devices[].  An ordinal may repeat: ranks that share a GPU are run as one
 * cooperative kernel over all ranks' data (the way to exercise an N-rank
 * protocol on fewer than N GPUs). */
int bl_init(blCtx** out, const int* devices, int ndev, size_t poolBytes, char* err,
            size_t errlen);

/* SPMD mode: one process per GPU.  Rank 0 listens on the unix socket
 * sockPath, collects every rank's arena descriptor and hands all of them
 * (and the multicast descriptor) to every rank.  After that the processes
 * never talk on the host again. */
int bl_init_peer(blCtx** out, int device, size_t poolBytes, const char* sockPath, int rank,
                 int world, char* err, size_t errlen);
void bl_shutdown(blCtx* ctx);

int bl_is_peer(const blCtx* ctx);
int bl_world(const blCtx* ctx);
int bl_rank(const blCtx* ctx);
int bl_has_multicast(const blCtx* ctx);
size_t bl_user_bytes(const blCtx* ctx);
/* largest message the zero-copy paths move in one call */
size_t bl_max_chunk(const blCtx* ctx);
/* largest p2p message per call, largest one-shot all-reduce message */
size_t bl_p2p_chunk(const blCtx* ctx);
size_t bl_oneshot_max(const blCtx* ctx);
/* the algorithm the dispatcher takes for an all-reduce of `bytes` (host arithmetic only) */
int bl_algo_for(size_t bytes, int world, int dtype, int has_multicast, size_t pool_bytes, int algo);
size_t bl_pool_bytes(const blCtx* ctx);

/* Symmetric allocator over the user zone of arena devIdx (peer mode: devIdx
 * is ignored, the arena is this rank's).  2 MiB alignment for >= 2 MiB,
 * 256 B otherwise; sizes round up to 16 B. */
int bl_pool_alloc(blCtx* ctx, int devIdx, size_t bytes, void** ptrOut, char* err,
                  size_t errlen);
int bl_pool_free(blCtx* ctx, int devIdx, void* ptr, size_t bytes);
/* offset of ptr inside its arena, or -1 when ptr is not arena memory */
int64_t bl_pool_offset(const blCtx* ctx, int devIdx, const void* ptr);
/* address of rank r's arena as mapped in this process (+offset) */
void* bl_peer_ptr(const blCtx* ctx, int r, size_t offset);
void* bl_multicast_ptr(const blCtx* ctx, size_t offset);

/* ---- single-process API (pool tensors) --------------------------------- */
int bl_copy_(blCtx* ctx, void* dstPtr, int dstIdx, void* srcPtr, int srcIdx, size_t bytes,
             void* srcStream, void* dstStream, char* err, size_t errlen);
/* every listed pool tensor ends up holding the elementwise sum of all */
int bl_allreduce_(blCtx* ctx, void* const* ptrs, const int* idxs, int n, size_t bytes,
                  int dtype, void* const* streams, char* err, size_t errlen);

/* the SPMD collectives below in single-process form, one pointer per arena:
 * kind 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 broadcast,
 * 4 all-reduce + residual + RMSNorm, 5 barrier (bytes is per rank for 1, 2) */
int bl_sp_collective(blCtx* ctx, int kind, const void* const* in, void* const* out,
                     const void* const* aux_in, void* const* aux_out, const void* const* gamma,
                     size_t bytes, int dtype, int algo, int root, int rows, int hidden, float eps,
                     void* const* streams, char* err, size_t errlen);
/* send as rank src then recv as rank dst on one stream (ranks sharing a GPU) */
int bl_sp_sendrecv(blCtx* ctx, int src, int dst, const void* in, void* out, size_t bytes,
                   void* stream, char* err, size_t errlen);

/* ---- SPMD collectives on arbitrary device pointers --------------------- */
/* algo: BL_ALGO_*; AUTO picks by size.  in == out allowed. */
int bl_allreduce_into_peer(blCtx* ctx, const void* inPtr, void* outPtr, size_t bytes,
                           int dtype, int algo, void* stream, char* err, size_t errlen);
/* out[r*stride .. r*stride+bytes) = rank r's in (stride 0: dense, = bytes) */
int bl_allgather_peer(blCtx* ctx, const void* inPtr, void* outPtr, size_t bytesPerRank,
                      size_t outStrideBytes, void* stream, char* err, size_t errlen);
/* out = sum over ranks of in[rank*stride .. +bytesPerRank) */
int bl_reduce_scatter_peer(blCtx* ctx, const void* inPtr, void* outPtr, size_t bytesPerRank,
                           size_t inStrideBytes, int dtype, void* stream, char* err,
                           size_t errlen);
int bl_broadcast_peer(blCtx* ctx, void* ptr, size_t bytes, int root, void* stream, char* err,
                      size_t errlen);
int bl_barrier_peer(blCtx* ctx, void* stream, char* err, size_t errlen);
/* out = all-reduce(in) + residual (written to residual_out), then RMSNorm
 * with weight gamma into normed_out.  rows x hidden elements of dtype.
 * nsplit > 0: in is instead nsplit fp32 slabs (slab elements apart) left by a
 * split-K linear; their sum, rounded to dtype, is this rank's contribution. */
int bl_allreduce_rmsnorm_peer(blCtx* ctx, const void* inPtr, const void* residualIn,
                              const void* gamma, void* residualOut, void* normedOut, int rows,
                              int hidden, float eps, int dtype, int nsplit, size_t slab, void* stream,
                              char* err, size_t errlen);
/* byte move; the k-th send to a peer pairs with that peer's k-th recv */
int bl_send_into_peer(blCtx* ctx, const void* inPtr, size_t bytes, int peerRank, void* stream,
                      char* err, size_t errlen);
int bl_recv_into_peer(blCtx* ctx, void* outPtr, size_t bytes, int peerRank, void* stream,
                      char* err, size_t errlen);
/* Sends run on a stream of their own; work queued on `stream` after this call
 * waits for every send issued so far (call it before overwriting a sent
 * buffer). */
int bl_join_sends(blCtx* ctx, void* stream);
/* the stream sends run on (cudaStream_t), or null */
void* bl_send_stream(blCtx* ctx);

/* ---- proofs and diagnostics ------------------------------------------- */
uint64_t bl_verify(blCtx* ctx, char* err, size_t errlen);
int bl_readback(blCtx* ctx, int devIdx, void* ptr, size_t bytes, void* dstHost, char* err,
                size_t errlen);
int bl_pool_move(blCtx* ctx, void* srcPoolPtr, void* outPtr, size_t bytes, void* stream,
                 char* err, size_t errlen);
/* host copy of the first n words of the local signal pad */
int bl_debug_flags(blCtx* ctx, unsigned long long* vals, int n, char* err, size_t errlen);
/* signal round trip and launch baselines in ns: res[0] flag ping-pong per
 * iteration, res[1] empty launch, res[2] multimem ping-pong (0 if none) */
int bl_probe_signal(blCtx* ctx, unsigned long long* res, int iters, void* stream, char* err,
                    size_t errlen);

/* A device wait that ran out leaves a record here instead of trapping.
 * code 0 = healthy.  Reading is free (host-mapped memory, no sync). */
typedef struct blStatus {
  uint32_t code;      /* 0 ok, 1 signal wait ran out, 2 payload wait ran out */
  uint32_t proto;     /* which protocol */
  uint32_t from_rank; /* whom we waited for */
  uint32_t have, want;
  uint32_t block;
  uint32_t reserved[2];
} blStatus;
int bl_status(blCtx* ctx, blStatus* out);
/* clears the record and the local abort word; every rank must then call
 * bl_reset_peer before the next collective */
int bl_reset_peer(blCtx* ctx, char* err, size_t errlen);
void bl_set_wait_timeout_ms(blCtx* ctx, unsigned ms);

/* counters: ops, bytes, per-algorithm picks, timeouts (see BL_STAT_*) */
#define BL_STAT_OPS 0
#define BL_STAT_BYTES 1
#define BL_STAT_ONESHOT 2
#define BL_STAT_TWOSHOT 3
#define BL_STAT_NVLS 4
#define BL_STAT_FUSED_NORM 5
#define BL_STAT_P2P 6
#define BL_STAT_TIMEOUTS 7
#define BL_STAT_COUNT 8
void bl_stats(const blCtx* ctx, unsigned long long* out /* BL_STAT_COUNT */);

/* Nothing privileged is needed on an NVSwitch box; kept so that a payload
 * started by blrun can prove it runs with no capabilities. */
void bl_drop_caps(void);

#ifdef __cplusplus
}
#endif
#endif /* BARLINK_B200_CORE_H */
