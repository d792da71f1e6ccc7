/* SPDX-License-Identifier: MIT
 *
 * Compute ops of barlink for B200: plain-C launchers of the sm_100a kernels
 * (tcgen05 GEMMs, W8A16, norm / RoPE / activation / attention kernels, fused
 * GEMM+collective kernels).  Pointers are device pointers, streams are
 * cudaStream_t passed as void*.  0 on success, -1 with a message otherwise.
 *
 * The reference's compute surface is its W8A16 pair (torch_ext/barlink_sm86/
 * w8a16.cu:165-212); everything else it takes from cuBLAS and HF/vLLM eager
 * kernels (demos/qwen_tp/qwen38_int8/worker.py:84-129, 208-241).
 */
#ifndef BARLINK_B200_OPS_H
#define BARLINK_B200_OPS_H

#include <stddef.h>
#include <stdint.h>

#include "bl_core.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Where the row-parallel linear fused with the reduce-scatter sends its output:
 * the inbox of each token's owner (fp32 [src rank][split][tokens_per_rank][n])
 * and that owner's arrival word for this rank, both as mapped in this process. */
typedef struct blPeerSink {
  void* inbox[BL_MAX_RANKS];
  void* flag[BL_MAX_RANKS];
  int world, rank, tokens_per_rank;
} blPeerSink;

/* Token-major row-parallel linear whose epilogue is the scatter half of a two-shot all-reduce:
 * output row m (global index row0 + m of a [total_rows x n] tensor) is stored, as bf16 16-byte
 * vectors, straight into the staging inbox of the rank that owns that row (rank (row0 + m) /
 * rows_per_rank), and every finished tile bumps the owners' arrival counters.  bl_allreduce_pushed
 * then reduces this rank's rows and hands the sums to every rank.  Filled by bl_gemm_push_setup. */
typedef struct blRowPush {
  void* arena[BL_MAX_RANKS];   /* every rank's arena as mapped here */
  void* flag[BL_MAX_RANKS];    /* each owner's arrival word for this source rank */
  const void* seq_word;        /* this rank's count of staged collectives (selects the staging buffer) */
  size_t stage_off, stage_slice;
  int world, rank, rows_per_rank, row0;
} blRowPush;

/* D[i, j] = sum_k A[i, k] * B[j, k]; A [ra x k] pitch lda, B [rb x k] pitch
 * ldb, bf16, K-major.  swap = 0: out[i, j]; swap = 1: out[j, i] (A = weight
 * rows, B = tokens: the decode orientation).  out is bf16 with pitch ldo.
 * bias is per output feature, residual has out's layout.  silu_mul: output
 * features are interleaved (gate, up) pairs and out gets silu(gate)*up in
 * column feature/2.  bn = 0 and splits = 0 choose automatically.  ws/counters
 * are the split-K scratch: ws_bytes >= tiles*splits*bn*128*4, counters zeroed
 * once (the kernel leaves them zero). */
typedef struct blGemmArgs {
  const void* a;
  int ra, lda;
  const void* b;
  int rb, ldb;
  int k;
  void* out;
  int ldo;
  int swap;
  const void* bias;
  const void* residual;
  int silu_mul;
  int gelu;            /* tanh-GELU on (acc + bias) */
  int bn;
  int splits;
  void* ws;
  size_t ws_bytes;
  void* counters;
  int n_counters;
  void* err_flag; /* u32 in device or host-mapped memory, set to 1 on a wait that ran out */
  int dynamic_weights; /* 1: the weight operand may be written by the kernel just before this
                          one in the stream, so it is not fetched ahead of that kernel's end */
  /* split-K without a reduction in the GEMM: when partial_out is set, split s
   * stores its raw fp32 tile to partial_out[s * partial_stride + token * ldo +
   * feature] and out/bias/residual/silu_mul are ignored; partial_splits is the
   * exact number of splits (see bl_gemm_splits) */
  void* partial_out;
  size_t partial_stride;
  int partial_splits;
  /* fused reduce-scatter (swap orientation only): partial rows go to peers */
  const blPeerSink* peer;
  /* token-major orientation: the output tile goes to the owners' staging inboxes (see blRowPush);
   * out is ignored, ldo must be n, no k-split */
  const blRowPush* push;
  /* fused all-gather in front: wait for gate_n words at gate_flags to reach
   * *gate_cum + gate_add before the first activation tile is requested */
  const void* gate_flags;
  void* gate_cum;
  void* gate_ticket;
  unsigned gate_add;
  int gate_n;
  unsigned long long gate_timeout_ns;
  /* the weight operand (A when swap, else B) is a buffer made by bl_tile_weight
   * (lda/ldb of that operand are ignored) */
  int weight_tiled;
  void* trace; /* debug: u64[8 * grid] global-timer stamps per CTA, or null */
  /* 1: a and b are signed 8-bit (lda/ldb/k in elements, k a multiple of 16); products accumulate in
   * int32 on the tensor cores and the result is acc * feat_scale[feature] * tok_scale[token].
   * Not with weight_tiled, peer, push or gate_flags. */
  int i8;
  const void* feat_scale; /* bf16 per output feature, or null */
  const void* tok_scale;  /* fp32 per token, or null */
  /* i8 with one weight scale per (feature, k-group) instead of feat_scale: bf16 [ra][k / group_k], group_k a
   * multiple of 128.  Weights-first orientation (swap) and at most 64 tokens only: every k-block gets an
   * accumulator of its own and the epilogue warps add acc * scale, k-block by k-block; no k-split. */
  const void* group_scale;
  int group_k;
} blGemmArgs;
int bl_gemm_bf16(const blGemmArgs* a, void* stream, char* err, size_t errlen);
/* Weights in 16 KiB tiles [ceil(n/128)][ceil(k/64)][128 x 128 B], each tile in the
 * swizzled shared-memory image: one bulk copy per tile instead of 128 row requests.
 * dst must be 16-byte aligned and bl_tiled_weight_bytes(n, k) long. */
size_t bl_tiled_weight_bytes(int n, int k);
int bl_tile_weight(const void* src, int n, int k, int ld, void* dst, void* stream, char* err,
                   size_t errlen);
/* k-splits the decode heuristic picks for n output features, k inputs and
 * `tokens` rows (1 = no split) */
int bl_gemm_splits(int n, int k, int tokens);

/* W8A16: x [m x k] bf16, wq [n x k] int8 (row = output channel), scale [n]
 * bf16 (per channel) or scales [k/group x n] fp32 (group > 0).  out [m x n]
 * bf16.  The int8 tile is widened to bf16 in shared memory inside the main
 * loop and multiplied on the tensor cores. */
typedef struct blW8A16Args {
  const void* x;
  int m, ldx;
  const void* wq;
  int n, k;
  const void* scale;  /* bf16 [n] */
  const void* bias;   /* bf16 [n] or null */
  void* out;
  int ldo;
  int silu_mul;
  int splits;
  void* ws;
  size_t ws_bytes;
  void* counters;
  int n_counters;
  void* err_flag;
  /* split-K slabs instead of a reduced output (see blGemmArgs.partial_out); the
   * per-channel scale is applied to every slab */
  void* partial_out;
  size_t partial_stride;
  int partial_splits;
  /* per-group scales applied inside the main loop: group_rel is fp16 [n][k / group_k], each row's
   * group scales divided by that row's largest one, and `scale` then holds the row's largest
   * scale (see bl_w8_group_scales).  group_k must be a multiple of 64.  null = per channel only */
  const void* group_rel;
  int group_k;
  /* activations already quantised per token (bl_w8a16_quant_act): xq int8 [m x k] dense and xs fp32
   * [m].  The product then runs as int8 x int8 on the tensor cores (no widening of the weights); x is
   * ignored, group_rel must be null and partial_out is not supported. */
  const void* xq;
  const void* xs;
  /* with xq: per-group weight scales bf16 [n][k / group_k] (the reference's checkpoint format, group 128)
   * instead of `scale`; at most 64 tokens, group_k a multiple of 128 */
  const void* group_scale;
} blW8A16Args;
/* scales bf16 [n][groups] -> row_max bf16 [n] and rel fp16 [n][groups] = scale / row_max */
int bl_w8_group_scales(const void* scales, int n, int groups, void* row_max, void* rel, void* stream, char* err,
                       size_t errlen);
/* returns -2 (and launches nothing) for more than 256 tokens */
int bl_w8a16_linear(const blW8A16Args* a, void* stream, char* err, size_t errlen);
/* out[n x k] bf16 = wq[n x k] int8 * scale[n]: the prefill path widens once and
 * then uses the bf16 GEMM */
int bl_w8_dequant(const void* wq, const void* scale, void* out, int n, int k, void* stream, char* err,
                  size_t errlen);
/* reference-compatible pair (w8a16.cu:165-212): per-token int8 activation
 * quantisation and the int8 x int8 GEMM with group-128 weight scales */
int bl_w8a16_quant_act(const void* x, int m, int k, void* xq, void* xs, void* stream, char* err,
                       size_t errlen);
int bl_w8a16_gemm(const void* xq, const void* xs, const void* wq_t, const void* sw_t, void* out,
                  int m, int n, int k, int splits, void* ws, void* stream, char* err,
                  size_t errlen);

/* out = RMSNorm(x (+ residual)) * gamma; when residual is given, x + residual
 * is also written to residual_out (may alias residual). */
/* partials != null: x is instead the sum of nsplit fp32 slabs (slab elements
 * apart) left by a split-K linear, rounded to bf16 first */
int bl_rmsnorm(const void* x, const void* residual, const void* gamma, void* out,
               void* residual_out, int rows, int hidden, float eps, const void* partials,
               int nsplit, size_t slab, void* stream, char* err, size_t errlen);
/* qkv [rows x (nq+2*nkv)*hd]: rotate q and k in place (rotate-half RoPE at
 * positions[rows]) and write k, v into the paged cache at slot[rows]
 * (slot = block*block_size + offset; negative = skip).  Cache layout
 * [blocks, nkv, block_size, hd]. */
/* partials != null: the input is the sum of nsplit fp32 slabs of the QKV
 * linear plus bias (bf16 [(nq+2nkv)*hd] or null); qkv is then output only */
int bl_rope_kv_write(void* qkv, const void* partials, int nsplit, size_t slab, const void* bias,
                     const int* positions, const int* slots, void* k_cache, void* v_cache, int rows,
                     int nq, int nkv, int hd, int block_size, float theta, void* stream, char* err,
                     size_t errlen);
/* plain RoPE on [rows x heads x hd] (2-D variant: positions has 2 ints per
 * row and each half of hd rotates by its own axis) */
int bl_rope(void* x, const int* positions, int rows, int heads, int hd, int row_stride, float theta,
            int axes, void* stream, char* err, size_t errlen);
int bl_silu_mul(const void* gate_up, void* out, int rows, int inter, int interleaved, void* stream,
                char* err, size_t errlen);
/* slabs: fp32 [nsplit][rows][2*inter], interleaved (gate, up) columns; out bf16 [rows][inter] */
int bl_silu_mul_slabs(const void* slabs, int nsplit, void* out, int rows, int inter, void* stream, char* err,
                      size_t errlen);
int bl_embedding(const int* ids, const void* table, void* out, int rows, int hidden, int vocab_lo,
                 int vocab_hi, void* stream, char* err, size_t errlen);
/* Decode attention over a paged KV cache.  q rows live in qkv (pitch
 * q_stride elements), nq query heads share nkv KV heads (nq % nkv == 0,
 * group <= 16).  block_tables [batch x max_blocks], ctx_lens [batch].
 * scratch: fp32, batch*nq*splits*(hd+2) floats (splits = 0: chosen here;
 * returns the number used through *splits_out). */
int bl_paged_attn_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                         const int* block_tables, const int* ctx_lens, void* out, int batch, int nq,
                         int nkv, int hd, int block_size, int max_blocks, float scale, int splits,
                         void* scratch, size_t scratch_bytes, void* stream, char* err,
                         size_t errlen);
/* RoPE + KV write + paged attention in one launch (decode).  qkv: bf16 rows, or null with
 * slabs = nsplit_in fp32 slabs of the QKV linear `slab` floats apart (+ bias).
 * counters: batch * nkv zeroed u32 words (left zero); with them the splits are merged by the
 * last block of each (sequence, KV head) inside the kernel, without them by a second kernel. */
int bl_rope_attn_decode(const void* qkv, int q_stride, const void* slabs, int nsplit_in, size_t slab,
                        const void* bias, const int* positions, const int* slots, float theta, void* k_cache,
                        void* v_cache, const int* block_tables, const int* ctx_lens, void* out, int batch, int nq,
                        int nkv, int hd, int block_size, int max_blocks, float scale, int splits, void* scratch,
                        size_t scratch_bytes, void* counters, void* stream, char* err, size_t errlen);
/* Dense attention (prefill / joint attention): q [tq x nq x hd], k, v
 * [tk x nkv x hd] per sequence, sequences given by cu_seqlens (batch+1);
 * causal aligns the last query with the last key. */
int bl_attn_fwd(const void* q, const void* k, const void* v, void* out, const int* cu_q,
                const int* cu_k, int batch, int max_q, int nq, int nkv, int hd, int q_stride,
                int k_stride, int v_stride, int o_stride, float scale, int causal, void* stream,
                char* err, size_t errlen);
/* same contract on the tcgen05 tensor cores (head_dim 128).  vt: scratch of
 * bl_attn_tc_scratch_bytes(); total_q / total_k: rows of q and k; err_flag: a
 * device word set to 1 if a bounded wait inside the kernel ran out */
size_t bl_attn_tc_scratch_bytes(int batch, int max_k, int nkv);
int bl_attn_fwd_tc(const void* q, const void* k, const void* v, void* out, const int* cu_q, const int* cu_k,
                   int batch, int max_q, int max_k, int total_q, int total_k, int nq, int nkv, int hd,
                   int q_stride, int k_stride, int v_stride, int o_stride, float scale, int causal, void* vt,
                   void* err_flag, void* stream, char* err, size_t errlen);
/* arg max over the last dim of [rows x n] bf16 logits -> idx (int32) and
 * value (fp32); `offset` is added to the index (vocab-parallel shards). */
int bl_argmax(const void* logits, int rows, int n, int ld, int offset, int* idx, float* val,
              void* scratch, size_t scratch_bytes, void* stream, char* err, size_t errlen);
/* first stage only: parts[bl_argmax_chunks()][rows] (value, index bits) pairs, one per slice of a
 * row -- the layout bl_argmax_merge reads, so per-rank parts of a vocabulary-parallel head can be
 * all-gathered and merged without any repacking */
int bl_argmax_parts(const void* logits, int rows, int n, int ld, int offset, void* parts, void* stream,
                    char* err, size_t errlen);
int bl_argmax_chunks(void);
/* merge [parts x rows] (value, index bits) pairs: highest value, lowest index */
int bl_argmax_merge(const void* pairs, int parts, int rows, int* idx, void* stream, char* err,
                    size_t errlen);
/* device-side bookkeeping of one decode step (positions, context lengths,
 * KV slots, next input ids) so that a captured step can be replayed */
int bl_decode_advance(int* positions, int* ctx_lens, int* slots, const int* block_tables, int* ids,
                      const int* sampled, int batch, int max_blocks, int block_size, void* stream,
                      char* err, size_t errlen);

/* ---- W4A16: GPTQ-v1 int4 weights, bf16 activations -------------------------- */
/* y[m, n] = sum_k x[m, k] * (nibble(n, k) - zero(g, n)) * scale(g, n); 1..16 rows;
 * splits <= 0: chosen here; a k-split needs ws of splits*m*n floats.  -2: too many rows */
int bl_w4a16_gemv(const void* x, const void* qweight, const void* scales, const void* qzeros, void* out,
                  int m, int n, int k, int group, int splits, void* ws, size_t ws_bytes, void* stream,
                  char* err, size_t errlen);
/* packed tensors -> bf16 [n, k] */
int bl_w4_dequant(const void* qweight, const void* scales, const void* qzeros, void* w, int n, int k,
                  int group, void* stream, char* err, size_t errlen);

/* ---- MMDiT (Flux-style) elementwise kernels --------------------------------- */
/* per-head RMSNorm of the q and k heads of a fused qkv row (weights gq, gk of
 * head_dim 128, null = no norm), then RoPE with 1 or 2 position axes */
int bl_qknorm_rope(void* qkv, const void* gq, const void* gk, const int* positions, int rows, int heads,
                   int hd, int row_stride, float eps, float theta, int axes, void* stream, char* err,
                   size_t errlen);
/* out = LayerNorm(x) * (1 + scale[b]) + shift[b], b = row / rows_per_batch */
int bl_layernorm_modulate(const void* x, const void* shift, const void* scale, void* out, int rows,
                          int hidden, int rows_per_batch, int mod_stride, float eps, void* stream,
                          char* err, size_t errlen);
/* x += gate[b] * y */
int bl_gate_residual(void* x, const void* y, const void* gate, int rows, int hidden, int rows_per_batch,
                     int mod_stride, void* stream, char* err, size_t errlen);

/* ---- fused GEMM + collective (tensor-parallel linears) -------------------
 * Decode with T tokens on `world` ranks, T % world == 0: token m belongs to
 * rank m / (T / world).
 *
 *  1. row-parallel linear + reduce-scatter: bl_gemm_bf16 in swap orientation
 *     with `peer` filled by bl_tp_peer_sink -- every k-split of every tile
 *     stores its fp32 partial rows into the owners' inboxes over NVLink and
 *     bumps their arrival counters;
 *  2. bl_rs_finish on every rank: wait for `units` arrivals from each rank,
 *     sum world x splits partial rows of my tokens (rank order, split order),
 *     add the residual of my tokens, RMS-normalise, and store the normed rows
 *     into every rank's all-gather buffer (+ arrival counter);
 *  3. all-gather + column-parallel linear: bl_gemm_bf16 whose activation
 *     operand is the all-gather buffer and whose gate_* fields come from
 *     bl_tp_gate: the weight tiles stream while it waits for the rows.
 * Offsets are into the symmetric arena (bl_pool_offset). */
int bl_tp_peer_sink(blCtx* ctx, size_t inbox_off, int tokens, blPeerSink* out, char* err,
                    size_t errlen);
/* rows of a [total_rows x n] bf16 all-reduce that a linear starting at row0 will push; fails when
 * total_rows is not a multiple of the ranks or a rank's rows do not fit its staging slice */
int bl_gemm_push_setup(blCtx* ctx, int total_rows, int n, int row0, blRowPush* out, char* err, size_t errlen);
/* tiles (arrival counts per owner) that bl_gemm_bf16 will produce for a pushed linear of `rows` rows */
int bl_gemm_push_units(int rows, int n);
/* second half: wait for `units` arrivals from every rank, reduce this rank's rows in rank order in
 * fp32, give the sums to every rank and write the whole [total_rows x n] result to out */
int bl_allreduce_pushed(blCtx* ctx, void* out, int total_rows, int n, int units, void* stream, char* err,
                        size_t errlen);
int bl_tp_gate(blCtx* ctx, int tokens, blGemmArgs* a, char* err, size_t errlen);
typedef struct blRsFinishArgs {
  size_t inbox_off;        /* fp32 [world][splits][tokens/world][n] in my arena */
  int tokens, n, splits;
  int units;               /* arrivals expected from each rank: tiles x splits of step 1 */
  const void* residual_in; /* bf16 [tokens/world][n], my tokens, or null */
  void* residual_out;      /* bf16 [tokens/world][n] (may alias residual_in) */
  const void* gamma;       /* bf16 [n] */
  float eps;
  size_t gather_off;       /* bf16 [tokens][n] in every rank's arena */
} blRsFinishArgs;
int bl_rs_finish(blCtx* ctx, const blRsFinishArgs* a, void* stream, char* err, size_t errlen);
/* tiles x splits that bl_gemm_bf16 will use for a peer-sink linear (the
 * `units` of bl_rs_finish and the slab count the inbox must hold) */
int bl_tp_units(int n, int k_local, int tokens, int* splits_out);

/* ---- decode linears with the surrounding collective folded in (dlin_kernels.cu) ----------
 * y[tokens, n] = x[tokens, k] @ w[n, k]^T for 1..64 tokens.  A cluster of CTAs shares one
 * 128-row tile of w and sums its k-split partials through distributed shared memory.
 *   pro = 1: x is first produced by this kernel as RMSNorm(residual_in + sum over ranks of the
 *            rows in this GPU's one-shot inbox) * gamma; the new residual goes to residual_out,
 *            the rows to x (k must be the hidden size).  This is the second half of an
 *            all-reduce whose first half is the epi = 2 epilogue of the linear before.
 *   epi = 0: out[tokens, ldo] = y (+ bias); 1: rows of w are interleaved (gate, up) pairs and
 *            out[tokens, n/2] = SiLU(gate) * up; 2: y is rounded to bf16 and stored into every
 *            rank's inbox as this rank's partial of a [tokens, hidden] all-reduce.
 * The inboxes are the link's (ctx in peer mode) or, for a single GPU, a buffer of
 * bl_dlin_local_link_bytes() prepared once by bl_dlin_local_link_init().  sync: 528 zeroed u32
 * words (counters, then per-segment sums of squares) that belong to this call site family (any number of launches may share them as long
 * as they are in one stream).  cluster = 0 chooses the cluster size. */
typedef struct blDlinArgs {
  const void* w;
  int n, k, ldw;
  const void* x; /* [tokens, k] bf16, pitch ldx; written first when pro = 1 */
  int tokens, ldx;
  int pro, epi;
  int hidden;    /* row length of the all-reduced tensor (pro = 1: == k; epi = 2: >= n) */
  const void* residual_in; /* pro = 1; null = no residual */
  void* residual_out;
  const void* gamma;
  float eps;
  void* sync;
  void* out;
  int ldo;
  const void* bias;
  int cluster;
  void* local_link;
  void* err_flag;
  void* trace; /* debug: u64[12 * grid] global-timer stamps per CTA, or null */
} blDlinArgs;
int bl_dlin(blCtx* ctx, const blDlinArgs* a, void* stream, char* err, size_t errlen);
/* the prologue of pro = 1 as a kernel of its own (in front of a linear that keeps its kernel) */
int bl_gather_norm(blCtx* ctx, const blDlinArgs* a, void* stream, char* err, size_t errlen);
int bl_dlin_cluster(int n, int k, int tokens, int want);
size_t bl_dlin_local_link_bytes(int tokens, int hidden);
int bl_dlin_local_link_init(void* buf, int tokens, int hidden, void* stream, char* err, size_t errlen);

#ifdef __cplusplus
}
#endif
#endif
