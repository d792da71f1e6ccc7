// SPDX-License-Identifier: MIT
//
// Python binding `_C`: the op surface of the reference's extension
// (torch_ext/barlink_sm86/binding.cpp:531-563 -- init, init_peer, shutdown,
// empty, copy_, allreduce_, allreduce_into, send_into, recv_into, verify,
// readback, debug_flags, pool_move, w8a16_quant_act, w8a16_gemm) plus what
// N-rank tensor parallelism on B200 adds: all-gather / reduce-scatter /
// broadcast / barrier, the fused all-reduce+RMSNorm, tcgen05 linears,
// decode kernels, fused GEMM+collective linears and the c10d backend class.
// One link context per process; argument errors are raised with actionable
// messages before any traffic; the GIL is released around every launch.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "backend.h"
#include "bl_core.h"
#include "bl_ops.h"

namespace py = pybind11;
using blpg::global_ctx;

namespace {

constexpr size_t kErr = 512;
#define BL_CHECK(expr)                                                 \
  do {                                                                 \
    char _e[kErr] = {0};                                               \
    char* err = _e;                                                    \
    size_t errlen = kErr;                                              \
    (void)err; (void)errlen;                                           \
    int _rc = (expr);                                                  \
    TORCH_CHECK(_rc == 0, _e[0] ? _e : "barlink: call failed: " #expr); \
  } while (0)

blCtx* ctx_or_throw() {
  blCtx* c = global_ctx();
  TORCH_CHECK(c != nullptr, "barlink: not initialised -- call init(devices, pool_mb) or init_peer(...) first");
  return c;
}
void* stream_of(const at::Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}
void check_cuda_contig(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "barlink: ", name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), "barlink: ", name, " must be contiguous");
}
void check_bf16(const at::Tensor& t, const char* name) {
  check_cuda_contig(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, "barlink: ", name, " must be bfloat16");
}

// ---------------------------------------------------------------------------
// link
// ---------------------------------------------------------------------------
std::vector<int> g_devices;   // single-process mode: arena index -> CUDA ordinal
int g_pool_mb = 0;

void init(std::vector<int> devices, int pool_mb) {
  blCtx* c = global_ctx();
  if (c) {
    // idempotent for the same arguments, like the reference (binding.cpp:96-104)
    TORCH_CHECK(!bl_is_peer(c) && devices == g_devices && pool_mb == g_pool_mb,
                "barlink: already initialised with different arguments; call shutdown() first");
    return;
  }
  TORCH_CHECK(pool_mb >= 8 && pool_mb <= 65536, "barlink: pool_mb must be in [8, 65536]");
  TORCH_CHECK(!devices.empty() && devices.size() <= BL_MAX_RANKS, "barlink: init needs 1..",
              BL_MAX_RANKS, " devices");
  blCtx* out = nullptr;
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_init(&out, devices.data(), int(devices.size()), size_t(pool_mb) << 20, err, errlen));
  }
  g_devices = devices;
  g_pool_mb = pool_mb;
  blpg::set_global_ctx(out);
  bl_drop_caps();
}

void init_peer(int device, int pool_mb, const std::string& sock_path, int rank, int world) {
  blCtx* c = global_ctx();
  if (c) {
    TORCH_CHECK(bl_is_peer(c) && bl_rank(c) == rank && bl_world(c) == world && pool_mb == g_pool_mb,
                "barlink: already initialised with different arguments; call shutdown() first");
    return;
  }
  TORCH_CHECK(pool_mb >= 8 && pool_mb <= 65536, "barlink: pool_mb must be in [8, 65536]");
  blCtx* out = nullptr;
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_init_peer(&out, device, size_t(pool_mb) << 20, sock_path.c_str(), rank, world, err,
                          errlen));
  }
  g_devices = {device};
  g_pool_mb = pool_mb;
  blpg::set_global_ctx(out);
}

void py_shutdown() {
  blCtx* c = global_ctx();
  if (!c) return;
  blpg::set_global_ctx(nullptr);
  bl_shutdown(c);
  g_devices.clear();
  g_pool_mb = 0;
}

py::dict info() {
  py::dict d;
  blCtx* c = global_ctx();
  d["initialized"] = c != nullptr;
  if (!c) return d;
  d["peer_mode"] = bool(bl_is_peer(c));
  d["world"] = bl_world(c);
  d["rank"] = bl_rank(c);
  d["multicast"] = bool(bl_has_multicast(c));
  d["pool_bytes"] = bl_pool_bytes(c);
  d["user_bytes"] = bl_user_bytes(c);
  d["max_chunk"] = bl_max_chunk(c);
  d["p2p_chunk"] = bl_p2p_chunk(c);
  d["oneshot_max"] = bl_oneshot_max(c);
  d["devices"] = g_devices;
  return d;
}

int arena_device(blCtx* c, int idx) {
  if (bl_is_peer(c)) return g_devices[0];
  TORCH_CHECK(idx >= 0 && idx < int(g_devices.size()), "barlink: arena index ", idx, " out of range");
  return g_devices[idx];
}

// pool tensor (never individually freed unless free_ is called)
at::Tensor empty(int64_t nbytes, int device_index, py::object dtype) {
  blCtx* c = ctx_or_throw();
  TORCH_CHECK(nbytes > 0, "barlink: empty() needs a positive byte count");
  at::ScalarType st = at::kByte;
  if (!dtype.is_none()) st = torch::python::detail::py_object_to_dtype(dtype);
  const int64_t isz = c10::elementSize(st);
  TORCH_CHECK(nbytes % isz == 0, "barlink: nbytes must be a multiple of the dtype's size");
  void* p = nullptr;
  BL_CHECK(bl_pool_alloc(c, device_index, size_t(nbytes), &p, err, errlen));
  const int dev = arena_device(c, device_index);
  auto opts = at::TensorOptions().dtype(st).device(at::kCUDA, dev);
  return at::from_blob(p, {nbytes / isz}, [](void*) {}, opts);
}
void free_(const at::Tensor& t, int device_index) {
  blCtx* c = ctx_or_throw();
  TORCH_CHECK(bl_pool_free(c, device_index, t.data_ptr(), t.nbytes()) == 0,
              "barlink: free_() needs a pool tensor exactly as empty() returned it");
}
int64_t pool_offset(const at::Tensor& t, int device_index) {
  return bl_pool_offset(ctx_or_throw(), device_index, t.data_ptr());
}

int arena_of(blCtx* c, const at::Tensor& t, const char* name) {
  for (int i = 0; i < bl_world(c); ++i)
    if (bl_pool_offset(c, i, t.data_ptr()) >= 0 && (bl_is_peer(c) || g_devices[i] == t.device().index()))
      return i;
  TORCH_CHECK(false, "barlink: ", name, " is not a pool tensor (allocate it with empty())");
}

void copy_(const at::Tensor& dst, const at::Tensor& src) {
  blCtx* c = ctx_or_throw();
  check_cuda_contig(dst, "dst");
  check_cuda_contig(src, "src");
  TORCH_CHECK(dst.nbytes() == src.nbytes() && dst.scalar_type() == src.scalar_type(),
              "barlink: copy_ needs same-size, same-dtype tensors");
  const int di = arena_of(c, dst, "dst"), si = arena_of(c, src, "src");
  void* ss = at::cuda::getCurrentCUDAStream(src.device().index()).stream();
  void* ds = at::cuda::getCurrentCUDAStream(dst.device().index()).stream();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_copy_(c, dst.data_ptr(), di, src.data_ptr(), si, src.nbytes(), ss, ds, err, errlen));
}

void allreduce_(std::vector<at::Tensor> ts) {
  blCtx* c = ctx_or_throw();
  TORCH_CHECK(int(ts.size()) == bl_world(c), "barlink: allreduce_ needs one pool tensor per arena (",
              bl_world(c), ")");
  std::vector<void*> ptrs, streams;
  std::vector<int> idxs;
  const int code = blpg::dtype_code(ts[0].scalar_type());
  TORCH_CHECK(code >= 0, "barlink: allreduce_ does not support dtype ", ts[0].scalar_type());
  std::vector<bool> used(ts.size(), false);
  for (auto& t : ts) {
    check_cuda_contig(t, "tensor");
    TORCH_CHECK(t.nbytes() == ts[0].nbytes() && t.scalar_type() == ts[0].scalar_type(),
                "barlink: allreduce_ tensors must match in size and dtype");
    int idx = -1;
    for (int i = 0; i < bl_world(c); ++i)
      if (!used[i] && bl_pool_offset(c, i, t.data_ptr()) >= 0 && g_devices[i] == t.device().index()) {
        idx = i;
        break;
      }
    TORCH_CHECK(idx >= 0, "barlink: allreduce_ needs one pool tensor from each arena");
    used[idx] = true;
    ptrs.push_back(t.data_ptr());
    idxs.push_back(idx);
    streams.push_back(at::cuda::getCurrentCUDAStream(t.device().index()).stream());
  }
  py::gil_scoped_release nogil;
  BL_CHECK(bl_allreduce_(c, ptrs.data(), idxs.data(), int(ptrs.size()), ts[0].nbytes(), code,
                         streams.data(), err, errlen));
}

int algo_code(const std::string& a) {
  if (a == "auto" || a.empty()) return BL_ALGO_AUTO;
  if (a == "oneshot") return BL_ALGO_ONESHOT;
  if (a == "twoshot") return BL_ALGO_TWOSHOT;
  if (a == "nvls") return BL_ALGO_NVLS;
  TORCH_CHECK(false, "barlink: unknown all-reduce algorithm '", a, "' (auto, oneshot, twoshot, nvls)");
}

void check_zero_copy(const at::Tensor& t, const char* name) {
  check_cuda_contig(t, name);
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0, "barlink: ", name,
              " must be 16-byte aligned");
  TORCH_CHECK(t.nbytes() > 0 && (t.nbytes() & 15u) == 0, "barlink: ", name,
              " must have a byte size that is a non-zero multiple of 16");
}

void allreduce_into(const at::Tensor& out, const at::Tensor& in, const std::string& algo) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(out, "out");
  check_zero_copy(in, "in");
  TORCH_CHECK(out.nbytes() == in.nbytes() && out.scalar_type() == in.scalar_type(),
              "barlink: allreduce_into needs same-size, same-dtype tensors");
  const int code = blpg::dtype_code(in.scalar_type());
  TORCH_CHECK(code >= 0, "barlink: allreduce_into does not support dtype ", in.scalar_type());
  const int a = algo_code(algo);
  c10::cuda::CUDAGuard guard(in.device());
  void* st = stream_of(in);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_allreduce_into_peer(c, in.data_ptr(), out.data_ptr(), in.nbytes(), code, a, st, err,
                                  errlen));
}

void allgather_into(const at::Tensor& out, const at::Tensor& in) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(out, "out");
  check_zero_copy(in, "in");
  TORCH_CHECK(out.nbytes() == in.nbytes() * size_t(bl_world(c)), "barlink: allgather_into needs out = world x in");
  c10::cuda::CUDAGuard guard(in.device());
  void* st = stream_of(in);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_allgather_peer(c, in.data_ptr(), out.data_ptr(), in.nbytes(), 0, st, err, errlen));
}

void reduce_scatter_into(const at::Tensor& out, const at::Tensor& in) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(out, "out");
  check_zero_copy(in, "in");
  TORCH_CHECK(in.nbytes() == out.nbytes() * size_t(bl_world(c)), "barlink: reduce_scatter_into needs in = world x out");
  const int code = blpg::dtype_code(in.scalar_type());
  TORCH_CHECK(code >= 0, "barlink: reduce_scatter_into does not support dtype ", in.scalar_type());
  c10::cuda::CUDAGuard guard(in.device());
  void* st = stream_of(in);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_reduce_scatter_peer(c, in.data_ptr(), out.data_ptr(), out.nbytes(), 0, code, st, err,
                                  errlen));
}

void broadcast_(const at::Tensor& t, int root) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(t, "tensor");
  c10::cuda::CUDAGuard guard(t.device());
  void* st = stream_of(t);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_broadcast_peer(c, t.data_ptr(), t.nbytes(), root, st, err, errlen));
}

void barrier() {
  blCtx* c = ctx_or_throw();
  void* st = at::cuda::getCurrentCUDAStream().stream();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_barrier_peer(c, st, err, errlen));
}

// normed, residual_out = allreduce_rmsnorm(x, residual, gamma, eps)
std::tuple<at::Tensor, at::Tensor> allreduce_rmsnorm(const at::Tensor& x,
                                                     const c10::optional<at::Tensor>& residual,
                                                     const at::Tensor& gamma, double eps,
                                                     c10::optional<at::Tensor> normed_out,
                                                     c10::optional<at::Tensor> residual_out) {
  blCtx* c = ctx_or_throw();
  check_cuda_contig(x, "x");
  check_cuda_contig(gamma, "gamma");
  const bool from_slabs = x.scalar_type() == at::kFloat && gamma.scalar_type() != at::kFloat;
  TORCH_CHECK(x.dim() >= 1 && gamma.numel() == x.size(-1) &&
                  (from_slabs ? x.dim() == 3 : gamma.scalar_type() == x.scalar_type()),
              "barlink: gamma must match the last dim (and, unless x is fp32 split-K slabs "
              "[splits, rows, hidden], the dtype) of x");
  const int code = blpg::dtype_code(gamma.scalar_type());
  const int hidden = int(x.size(-1));
  const int nsplit = from_slabs ? int(x.size(0)) : 0;
  const int rows = int(x.numel() / hidden / (from_slabs ? nsplit : 1));
  auto oopt = x.options().dtype(gamma.scalar_type());
  at::Tensor normed = normed_out ? *normed_out : at::empty({rows, hidden}, oopt);
  at::Tensor res = residual_out ? *residual_out : at::empty({rows, hidden}, oopt);
  const void* rin = nullptr;
  if (residual) {
    check_cuda_contig(*residual, "residual");
    TORCH_CHECK(residual->numel() == int64_t(rows) * hidden &&
                    residual->scalar_type() == gamma.scalar_type(),
                "barlink: residual must be [rows, hidden] of the output dtype");
    rin = residual->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  void* st = stream_of(x);
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_allreduce_rmsnorm_peer(c, x.data_ptr(), rin, gamma.data_ptr(), res.data_ptr(),
                                       normed.data_ptr(), rows, hidden, float(eps), code, nsplit,
                                       size_t(rows) * hidden, st, err, errlen));
  }
  return {normed, res};
}

void send_into(const at::Tensor& t, int peer) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(t, "tensor");
  c10::cuda::CUDAGuard guard(t.device());
  void* st = stream_of(t);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_send_into_peer(c, t.data_ptr(), t.nbytes(), peer, st, err, errlen));
}
void join_sends() {
  blCtx* c = ctx_or_throw();
  bl_join_sends(c, at::cuda::getCurrentCUDAStream().stream());
}
void recv_into(const at::Tensor& t, int peer) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(t, "tensor");
  c10::cuda::CUDAGuard guard(t.device());
  void* st = stream_of(t);
  py::gil_scoped_release nogil;
  BL_CHECK(bl_recv_into_peer(c, t.data_ptr(), t.nbytes(), peer, st, err, errlen));
}

uint64_t verify() {
  blCtx* c = ctx_or_throw();
  char e[kErr] = {0};
  uint64_t bad;
  {
    py::gil_scoped_release nogil;
    bad = bl_verify(c, e, kErr);
  }
  TORCH_CHECK(bad != ~0ull, e[0] ? e : "barlink: verify failed to run");
  return bad;
}

at::Tensor readback(const at::Tensor& t) {
  blCtx* c = ctx_or_throw();
  check_cuda_contig(t, "tensor");
  const int idx = arena_of(c, t, "tensor");
  at::Tensor out = at::empty(t.sizes(), t.options().device(at::kCPU));
  py::gil_scoped_release nogil;
  BL_CHECK(bl_readback(c, idx, t.data_ptr(), t.nbytes(), out.data_ptr(), err, errlen));
  return out;
}

void pool_move(const at::Tensor& out, const at::Tensor& src) {
  blCtx* c = ctx_or_throw();
  check_zero_copy(out, "out");
  check_zero_copy(src, "src");
  TORCH_CHECK(out.nbytes() == src.nbytes(), "barlink: pool_move needs same-size tensors");
  c10::cuda::CUDAGuard guard(out.device());
  void* st = stream_of(out);
  BL_CHECK(bl_pool_move(c, src.data_ptr(), out.data_ptr(), out.nbytes(), st, err, errlen));
}

std::vector<uint64_t> debug_flags(int n) {
  blCtx* c = ctx_or_throw();
  std::vector<unsigned long long> v(n);
  BL_CHECK(bl_debug_flags(c, v.data(), n, err, errlen));
  return std::vector<uint64_t>(v.begin(), v.end());
}

std::vector<uint64_t> signal_probe(int iters) {
  blCtx* c = ctx_or_throw();
  unsigned long long r[3] = {0, 0, 0};
  void* st = at::cuda::getCurrentCUDAStream().stream();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_probe_signal(c, r, iters, st, err, errlen));
  }
  return {r[0], r[1], r[2]};
}

py::dict status() {
  py::dict d;
  blCtx* c = ctx_or_throw();
  blStatus s;
  bl_status(c, &s);
  d["code"] = s.code;
  d["proto"] = s.proto;
  d["from_rank"] = s.from_rank;
  d["have"] = s.have;
  d["want"] = s.want;
  d["block"] = s.block;
  return d;
}
void reset() {
  blCtx* c = ctx_or_throw();
  BL_CHECK(bl_reset_peer(c, err, errlen));
}
void set_wait_timeout_ms(unsigned ms) { bl_set_wait_timeout_ms(ctx_or_throw(), ms); }
py::dict stats() {
  unsigned long long v[BL_STAT_COUNT];
  bl_stats(global_ctx(), v);
  py::dict d;
  d["ops"] = v[BL_STAT_OPS];
  d["bytes"] = v[BL_STAT_BYTES];
  d["oneshot"] = v[BL_STAT_ONESHOT];
  d["twoshot"] = v[BL_STAT_TWOSHOT];
  d["nvls"] = v[BL_STAT_NVLS];
  d["fused_norm"] = v[BL_STAT_FUSED_NORM];
  d["p2p"] = v[BL_STAT_P2P];
  d["timeouts"] = v[BL_STAT_TIMEOUTS];
  return d;
}

// ---------------------------------------------------------------------------
// compute ops
// ---------------------------------------------------------------------------
struct Scratch {
  at::Tensor ws, counters, err_flag, attn, attn_counters;
};
Scratch& scratch_for(int dev) {
  static std::map<int, Scratch> m;
  auto it = m.find(dev);
  if (it != m.end()) return it->second;
  Scratch s;
  auto o = at::TensorOptions().device(at::kCUDA, dev);
  s.ws = at::empty({int64_t(64) << 20}, o.dtype(at::kByte));
  s.counters = at::zeros({16384}, o.dtype(at::kInt));
  s.err_flag = at::zeros({4}, o.dtype(at::kInt));
  s.attn = at::empty({int64_t(64) << 20}, o.dtype(at::kByte));
  s.attn_counters = at::zeros({65536}, o.dtype(at::kInt));
  return m.emplace(dev, s).first->second;
}

int gemm_error_flag(int dev) {
  Scratch& s = scratch_for(dev);
  return s.err_flag.cpu()[0].item<int>();
}

// y[tokens, n] = x[tokens, k] @ w[n, k]^T (+bias) (+residual) (silu_mul: w rows
// are interleaved gate/up pairs and y is [tokens, n/2])
at::Tensor linear(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                  const c10::optional<at::Tensor>& residual, bool silu_mul,
                  c10::optional<at::Tensor> out_opt, int force_swap, int bn, int splits,
                  bool dynamic_weights, c10::optional<at::Tensor> trace, int gate_tokens, int tiled_n,
                  int tiled_k, bool gelu) {
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
              "barlink: x must be a 2-D bfloat16 CUDA tensor with unit inner stride");
  const bool tiled = tiled_n > 0;
  if (tiled) {
    TORCH_CHECK(tiled_k == x.size(1) && size_t(w.nbytes()) >= bl_tiled_weight_bytes(tiled_n, tiled_k) &&
                    (reinterpret_cast<uintptr_t>(w.data_ptr()) & 15u) == 0,
                "barlink: tiled weight buffer does not match (n, k) = (", tiled_n, ", ", tiled_k, ")");
  } else {
    TORCH_CHECK(w.dim() == 2 && w.size(1) == x.size(1), "barlink: weight must be [n, k] with k = x.shape[1]");
  }
  const int tokens = int(x.size(0)), k = int(x.size(1)), n = tiled ? tiled_n : int(w.size(0));
  const int n_out = silu_mul ? n / 2 : n;
  at::Tensor out = out_opt ? *out_opt : at::empty({tokens, n_out}, x.options());
  TORCH_CHECK(out.is_contiguous() && out.size(0) == tokens && out.size(1) == n_out &&
                  out.scalar_type() == at::kBFloat16,
              "barlink: out must be a contiguous [tokens, n] bfloat16 tensor");
  if (tokens == 0) return out;
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  Scratch& s = scratch_for(dev);
  const bool swap = force_swap >= 0 ? force_swap != 0 : tokens <= 128;
  blGemmArgs a;
  memset(&a, 0, sizeof(a));
  if (swap) {
    a.a = w.data_ptr(); a.ra = n; a.lda = k;
    a.b = x.data_ptr(); a.rb = tokens; a.ldb = int(x.stride(0));
  } else {
    a.a = x.data_ptr(); a.ra = tokens; a.lda = int(x.stride(0));
    a.b = w.data_ptr(); a.rb = n; a.ldb = k;
  }
  a.k = k;
  a.out = out.data_ptr();
  a.ldo = n_out;
  a.swap = swap ? 1 : 0;
  if (bias) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == n, "barlink: bias must have n elements");
    a.bias = bias->data_ptr();
  }
  if (residual) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->sizes() == out.sizes(), "barlink: residual must match the output");
    a.residual = residual->data_ptr();
  }
  a.silu_mul = silu_mul ? 1 : 0;
  a.gelu = gelu ? 1 : 0;
  a.bn = bn;
  a.splits = splits;
  a.ws = s.ws.data_ptr();
  a.ws_bytes = size_t(s.ws.nbytes());
  a.counters = s.counters.data_ptr();
  a.n_counters = int(s.counters.numel());
  a.err_flag = s.err_flag.data_ptr();
  a.dynamic_weights = dynamic_weights ? 1 : 0;
  a.weight_tiled = tiled ? 1 : 0;
  if (gate_tokens > 0) BL_CHECK(bl_tp_gate(ctx_or_throw(), gate_tokens, &a, err, errlen));
  if (trace) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->numel() >= 8 * 296,
                "barlink: trace must be an int64 CUDA tensor of at least 2368 entries");
    a.trace = trace->data_ptr();
  }
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_gemm_bf16(&a, st, err, errlen));
  }
  return out;
}

// Row-parallel linear whose epilogue scatters the output tiles into the owners' staging inboxes
// (first half of a two-shot all-reduce over a [total_rows, n] tensor; this call covers rows
// row0 .. row0 + x.shape[0]).  Returns the arrival count to pass to allreduce_pushed.
int linear_push(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                const c10::optional<at::Tensor>& residual, bool gelu, int total_rows, int row0) {
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 &&
                  w.dim() == 2 && w.size(1) == x.size(1),
              "barlink: linear_push needs bf16 x [rows, k] and w [n, k]");
  const int rows = int(x.size(0)), k = int(x.size(1)), n = int(w.size(0));
  TORCH_CHECK(rows > 128 && n >= 256 && row0 >= 0 && row0 + rows <= total_rows,
              "barlink: linear_push is for token-major products (more than 128 rows, n >= 256) inside total_rows");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  Scratch& s = scratch_for(dev);
  blRowPush push;
  BL_CHECK(bl_gemm_push_setup(ctx_or_throw(), total_rows, n, row0, &push, err, errlen));
  blGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.a = x.data_ptr(); a.ra = rows; a.lda = int(x.stride(0));
  a.b = w.data_ptr(); a.rb = n; a.ldb = k;
  a.k = k;
  a.ldo = n;
  a.push = &push;
  if (bias) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == n, "barlink: bias must have n elements");
    a.bias = bias->data_ptr();
  }
  if (residual) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == rows && residual->size(1) == n,
                "barlink: residual must be [rows, n]");
    a.residual = residual->data_ptr();
  }
  a.gelu = gelu ? 1 : 0;
  a.err_flag = s.err_flag.data_ptr();
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_gemm_bf16(&a, st, err, errlen));
  }
  return bl_gemm_push_units(rows, n);
}

// second half: out [total_rows, n] bf16 receives the all-reduced tensor on every rank
void allreduce_pushed(const at::Tensor& out, int units) {
  check_bf16(out, "out");
  TORCH_CHECK(out.dim() == 2, "barlink: allreduce_pushed needs a [rows, n] output");
  c10::cuda::CUDAGuard guard(out.device());
  void* st = at::cuda::getCurrentCUDAStream(out.device().index()).stream();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_allreduce_pushed(ctx_or_throw(), out.data_ptr(), int(out.size(0)), int(out.size(1)), units, st, err,
                               errlen));
}

int gemm_splits(int n, int k, int tokens) { return bl_gemm_splits(n, k, tokens); }

// [n, k] bf16 -> flat buffer of 16 KiB tiles in the swizzled shared-memory image
at::Tensor tile_weight(const at::Tensor& w) {
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1,
              "barlink: tile_weight needs a 2-D bfloat16 CUDA tensor with unit inner stride");
  const int n = int(w.size(0)), k = int(w.size(1));
  at::Tensor out = at::empty({int64_t(bl_tiled_weight_bytes(n, k) / 2)}, w.options());
  c10::cuda::CUDAGuard guard(w.device());
  BL_CHECK(bl_tile_weight(w.data_ptr(), n, k, int(w.stride(0)), out.data_ptr(), stream_of(w), err, errlen));
  return out;
}

// Split-K linear without a reduction: returns fp32 slabs [splits, tokens, n] that
// the next kernel (rmsnorm / rope_kv_write / the fused all-reduce) sums as it reads.
at::Tensor linear_partial(const at::Tensor& x, const at::Tensor& w, int splits,
                          c10::optional<at::Tensor> out_opt, int gate_tokens, int tiled_n, int tiled_k) {
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
              "barlink: x must be a 2-D bfloat16 CUDA tensor with unit inner stride");
  const bool tiled = tiled_n > 0;
  if (tiled) {
    TORCH_CHECK(tiled_k == x.size(1) && size_t(w.nbytes()) >= bl_tiled_weight_bytes(tiled_n, tiled_k),
                "barlink: tiled weight buffer does not match (n, k)");
  } else {
    TORCH_CHECK(w.dim() == 2 && w.size(1) == x.size(1), "barlink: weight must be [n, k] with k = x.shape[1]");
  }
  const int tokens = int(x.size(0)), k = int(x.size(1)), n = tiled ? tiled_n : int(w.size(0));
  TORCH_CHECK(tokens >= 1 && tokens <= 256, "barlink: linear_partial is the decode path (1..256 tokens)");
  if (splits <= 0) splits = bl_gemm_splits(n, k, tokens);
  at::Tensor out = out_opt ? *out_opt
                           : at::empty({splits, tokens, n}, x.options().dtype(at::kFloat));
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kFloat && out.dim() == 3 &&
                  out.size(0) == splits && out.size(1) == tokens && out.size(2) == n,
              "barlink: out must be a contiguous float32 [splits, tokens, n] tensor");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  Scratch& s = scratch_for(dev);
  blGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.a = w.data_ptr(); a.ra = n; a.lda = k;
  a.b = x.data_ptr(); a.rb = tokens; a.ldb = int(x.stride(0));
  a.k = k;
  a.ldo = n;
  a.swap = 1;
  a.partial_out = out.data_ptr();
  a.partial_stride = size_t(tokens) * n;
  a.partial_splits = splits;
  a.splits = splits;
  a.err_flag = s.err_flag.data_ptr();
  a.weight_tiled = tiled ? 1 : 0;
  if (gate_tokens > 0) BL_CHECK(bl_tp_gate(ctx_or_throw(), gate_tokens, &a, err, errlen));
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_gemm_bf16(&a, st, err, errlen));
  }
  return out;
}

// Row-parallel linear fused with the reduce-scatter: partial rows of x @ w.T go
// straight into the inbox of each token's owner (inbox: fp32 arena tensor of
// world*splits*tokens/world*n elements at the same offset on every rank).
// Returns (units, splits) for tp_rs_finish.
std::tuple<int, int> tp_gemm_rs(const at::Tensor& x, const at::Tensor& w, const at::Tensor& inbox,
                                int tiled_n, int tiled_k) {
  blCtx* c = ctx_or_throw();
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
              "barlink: x must be a 2-D bfloat16 CUDA tensor with unit inner stride");
  const bool tiled = tiled_n > 0;
  if (!tiled) {
    TORCH_CHECK(w.dim() == 2 && w.size(1) == x.size(1), "barlink: weight must be [n, k_local]");
  }
  const int tokens = int(x.size(0)), k = int(x.size(1)), n = tiled ? tiled_n : int(w.size(0));
  TORCH_CHECK(tokens <= 256, "barlink: the fused reduce-scatter linear is the decode path (<= 256 tokens)");
  int splits = 1;
  const int units = bl_tp_units(n, k, tokens, &splits);
  const int64_t off = bl_pool_offset(c, 0, inbox.data_ptr());
  TORCH_CHECK(off >= 0 && inbox.scalar_type() == at::kFloat &&
                  inbox.numel() >= int64_t(bl_world(c)) * splits * (tokens / bl_world(c)) * n,
              "barlink: inbox must be a float32 arena tensor (empty()) of at least world*splits*tokens/world*n elements");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  Scratch& s = scratch_for(dev);
  blPeerSink ps;
  BL_CHECK(bl_tp_peer_sink(c, size_t(off), tokens, &ps, err, errlen));
  blGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.a = w.data_ptr(); a.ra = n; a.lda = k;
  a.b = x.data_ptr(); a.rb = tokens; a.ldb = int(x.stride(0));
  a.k = k;
  a.ldo = n;
  a.swap = 1;
  a.peer = &ps;
  a.weight_tiled = tiled ? 1 : 0;
  a.partial_splits = splits;
  a.splits = splits;
  a.err_flag = s.err_flag.data_ptr();
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_gemm_bf16(&a, st, err, errlen));
  }
  return {units, splits};
}

// Reduce my tokens from the inbox, add the residual (updated in place), norm,
// and all-gather the normed rows into `gather` (bf16 arena tensor [tokens, n]).
void tp_rs_finish(const at::Tensor& inbox, const at::Tensor& gather, const at::Tensor& residual,
                  const at::Tensor& gamma, double eps, int tokens, int splits, int units,
                  bool add_residual) {
  blCtx* c = ctx_or_throw();
  check_bf16(gamma, "gamma");
  check_bf16(residual, "residual");
  check_bf16(gather, "gather");
  const int n = int(gamma.numel());
  const int64_t ioff = bl_pool_offset(c, 0, inbox.data_ptr());
  const int64_t goff = bl_pool_offset(c, 0, gather.data_ptr());
  TORCH_CHECK(ioff >= 0 && goff >= 0, "barlink: inbox and gather must be arena tensors (empty())");
  TORCH_CHECK(gather.numel() >= int64_t(tokens) * n, "barlink: gather must hold tokens x n elements");
  TORCH_CHECK(residual.numel() == int64_t(tokens / bl_world(c)) * n,
              "barlink: residual holds this rank's tokens: [tokens/world, n]");
  blRsFinishArgs a;
  memset(&a, 0, sizeof(a));
  a.inbox_off = size_t(ioff);
  a.tokens = tokens;
  a.n = n;
  a.splits = splits;
  a.units = units;
  a.residual_in = add_residual ? residual.data_ptr() : nullptr;
  a.residual_out = residual.data_ptr();
  a.gamma = gamma.data_ptr();
  a.eps = float(eps);
  a.gather_off = size_t(goff);
  c10::cuda::CUDAGuard guard(gather.device());
  void* st = at::cuda::getCurrentCUDAStream(gather.device().index()).stream();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_rs_finish(c, &a, st, err, errlen));
}

std::tuple<at::Tensor, at::Tensor> rmsnorm(const at::Tensor& x, const at::Tensor& gamma, double eps,
                                           const c10::optional<at::Tensor>& residual,
                                           c10::optional<at::Tensor> out_opt) {
  check_bf16(gamma, "gamma");
  const bool from_slabs = x.scalar_type() == at::kFloat;
  if (from_slabs) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 3,
                "barlink: split-K slabs must be a contiguous float32 [splits, rows, hidden] CUDA tensor");
  } else {
    check_bf16(x, "x");
  }
  const int hidden = int(x.size(-1));
  const int nsplit = from_slabs ? int(x.size(0)) : 0;
  const int rows = int(x.numel() / hidden / (from_slabs ? nsplit : 1));
  TORCH_CHECK(gamma.numel() == hidden, "barlink: gamma must have hidden elements");
  at::Tensor out = out_opt ? *out_opt
                           : at::empty({rows, hidden}, x.options().dtype(at::kBFloat16));
  at::Tensor res_out;
  const void* rin = nullptr;
  void* rout = nullptr;
  if (residual) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->numel() == int64_t(rows) * hidden, "barlink: residual must match x");
    res_out = *residual;  // updated in place
    rin = residual->data_ptr();
    rout = res_out.data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  if (rows > 0)
    BL_CHECK(bl_rmsnorm(from_slabs ? nullptr : x.data_ptr(), rin, gamma.data_ptr(), out.data_ptr(),
                        rout, rows, hidden, float(eps), from_slabs ? x.data_ptr() : nullptr, nsplit,
                        size_t(rows) * hidden, stream_of(x), err, errlen));
  return {out, res_out};
}

at::Tensor rope_kv_write(const at::Tensor& qkv_in, const at::Tensor& positions,
                         const c10::optional<at::Tensor>& slots,
                         const c10::optional<at::Tensor>& k_cache,
                         const c10::optional<at::Tensor>& v_cache, int nq, int nkv, int hd,
                         int block_size, double theta, const c10::optional<at::Tensor>& bias,
                         c10::optional<at::Tensor> out_opt) {
  const bool from_slabs = qkv_in.scalar_type() == at::kFloat;
  at::Tensor qkv = qkv_in;
  const void* slabs = nullptr;
  int nsplit = 0;
  size_t slab = 0;
  const void* bias_p = nullptr;
  if (from_slabs) {
    TORCH_CHECK(qkv_in.is_cuda() && qkv_in.is_contiguous() && qkv_in.dim() == 3,
                "barlink: split-K slabs must be a contiguous float32 [splits, rows, width] CUDA tensor");
    nsplit = int(qkv_in.size(0));
    slab = size_t(qkv_in.size(1)) * size_t(qkv_in.size(2));
    slabs = qkv_in.data_ptr();
    qkv = out_opt ? *out_opt
                  : at::empty({qkv_in.size(1), qkv_in.size(2)}, qkv_in.options().dtype(at::kBFloat16));
    if (bias) {
      check_bf16(*bias, "bias");
      TORCH_CHECK(bias->numel() == qkv_in.size(2), "barlink: bias must match the qkv width");
      bias_p = bias->data_ptr();
    }
  } else {
    TORCH_CHECK(!bias, "barlink: bias is applied only when the input is split-K slabs");
  }
  check_bf16(qkv, "qkv");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.is_contiguous(),
              "barlink: positions must be a contiguous int32 CUDA tensor");
  const int rows = int(qkv.numel() / (int64_t(nq + 2 * nkv) * hd));
  TORCH_CHECK(int64_t(rows) * (nq + 2 * nkv) * hd == qkv.numel() && positions.numel() == rows,
              "barlink: qkv must be [rows, (nq + 2 nkv) * hd] and positions [rows]");
  const int* sl = nullptr;
  void *kc = nullptr, *vc = nullptr;
  if (slots) {
    TORCH_CHECK(slots->is_cuda() && slots->scalar_type() == at::kInt && slots->numel() == rows,
                "barlink: slots must be int32 [rows]");
    TORCH_CHECK(k_cache && v_cache, "barlink: slots given without caches");
    check_bf16(*k_cache, "k_cache");
    check_bf16(*v_cache, "v_cache");
    sl = slots->data_ptr<int>();
    kc = k_cache->data_ptr();
    vc = v_cache->data_ptr();
  }
  c10::cuda::CUDAGuard guard(qkv.device());
  if (rows > 0)
    BL_CHECK(bl_rope_kv_write(qkv.data_ptr(), slabs, nsplit, slab, bias_p, positions.data_ptr<int>(),
                              sl, kc, vc, rows, nq, nkv, hd, block_size, float(theta), stream_of(qkv),
                              err, errlen));
  return qkv;
}

void rope(const at::Tensor& x, const at::Tensor& positions, int heads, int hd, double theta, int axes) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() >= 2 && x.stride(-1) == 1,
              "barlink: rope needs a bfloat16 CUDA tensor");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.is_contiguous(),
              "barlink: positions must be a contiguous int32 CUDA tensor");
  const int rows = int(positions.numel() / axes);
  at::Tensor x2 = x.dim() == 2 ? x : x.view({rows, -1});
  TORCH_CHECK(x2.size(0) == rows && x2.size(1) >= int64_t(heads) * hd, "barlink: rope shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  if (rows > 0)
    BL_CHECK(bl_rope(x2.data_ptr(), positions.data_ptr<int>(), rows, heads, hd, int(x2.stride(0)),
                     float(theta), axes, stream_of(x), err, errlen));
}

at::Tensor silu_mul(const at::Tensor& gate_up, bool interleaved) {
  if (gate_up.scalar_type() == at::kFloat && gate_up.dim() == 3) {
    // k-split slabs [split][rows][2*inter] of the gate/up linear (interleaved columns)
    TORCH_CHECK(gate_up.is_cuda() && gate_up.is_contiguous() && interleaved && gate_up.size(2) % 8 == 0,
                "barlink: silu_mul over slabs needs contiguous float32 CUDA slabs with interleaved gate/up columns");
    const int rows = int(gate_up.size(1)), inter = int(gate_up.size(2) / 2);
    at::Tensor out = at::empty({rows, inter}, gate_up.options().dtype(at::kBFloat16));
    c10::cuda::CUDAGuard guard(gate_up.device());
    if (rows > 0)
      BL_CHECK(bl_silu_mul_slabs(gate_up.data_ptr(), int(gate_up.size(0)), out.data_ptr(), rows, inter,
                                 stream_of(gate_up), err, errlen));
    return out;
  }
  check_bf16(gate_up, "gate_up");
  const int two = int(gate_up.size(-1));
  TORCH_CHECK(two % 2 == 0, "barlink: silu_mul needs an even last dim");
  const int rows = int(gate_up.numel() / two);
  auto sizes = gate_up.sizes().vec();
  sizes.back() = two / 2;
  at::Tensor out = at::empty(sizes, gate_up.options());
  c10::cuda::CUDAGuard guard(gate_up.device());
  if (rows > 0)
    BL_CHECK(bl_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, two / 2, interleaved ? 1 : 0,
                         stream_of(gate_up), err, errlen));
  return out;
}

at::Tensor embedding(const at::Tensor& ids, const at::Tensor& table, int vocab_lo,
                     c10::optional<at::Tensor> out_opt) {
  check_bf16(table, "table");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.is_contiguous(),
              "barlink: ids must be a contiguous int32 CUDA tensor");
  const int rows = int(ids.numel()), hidden = int(table.size(1));
  at::Tensor out = out_opt ? *out_opt : at::empty({rows, hidden}, table.options());
  c10::cuda::CUDAGuard guard(table.device());
  if (rows > 0)
    BL_CHECK(bl_embedding(ids.data_ptr<int>(), table.data_ptr(), out.data_ptr(), rows, hidden,
                          vocab_lo, vocab_lo + int(table.size(0)), stream_of(table), err, errlen));
  return out;
}

std::tuple<at::Tensor, at::Tensor> argmax(const at::Tensor& logits, int offset) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 &&
                  logits.stride(1) == 1,
              "barlink: argmax needs 2-D bfloat16 CUDA logits");
  const int rows = int(logits.size(0)), n = int(logits.size(1));
  at::Tensor idx = at::empty({rows}, logits.options().dtype(at::kInt));
  at::Tensor val = at::empty({rows}, logits.options().dtype(at::kFloat));
  c10::cuda::CUDAGuard guard(logits.device());
  if (rows > 0)
  {
    Scratch& s = scratch_for(logits.device().index());
    BL_CHECK(bl_argmax(logits.data_ptr(), rows, n, int(logits.stride(0)), offset,
                       idx.data_ptr<int>(), val.data_ptr<float>(), s.attn.data_ptr(),
                       size_t(s.attn.nbytes()), stream_of(logits), err, errlen));
  }
  return {idx, val};
}

void decode_advance(const at::Tensor& positions, const at::Tensor& ctx_lens, const at::Tensor& slots,
                    const at::Tensor& block_tables, const at::Tensor& ids,
                    const c10::optional<at::Tensor>& sampled, int block_size) {
  auto chk = [](const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), "barlink: ", name,
                " must be a contiguous int32 CUDA tensor");
  };
  chk(positions, "positions");
  chk(ctx_lens, "ctx_lens");
  chk(slots, "slots");
  chk(block_tables, "block_tables");
  chk(ids, "ids");
  const int batch = int(positions.numel());
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.size(0) == batch && ctx_lens.numel() == batch &&
                  slots.numel() == batch && ids.numel() == batch,
              "barlink: decode_advance batch mismatch");
  const int* sp = nullptr;
  if (sampled) {
    chk(*sampled, "sampled");
    sp = sampled->data_ptr<int>();
  }
  c10::cuda::CUDAGuard guard(positions.device());
  BL_CHECK(bl_decode_advance(positions.data_ptr<int>(), ctx_lens.data_ptr<int>(), slots.data_ptr<int>(),
                             block_tables.data_ptr<int>(), ids.data_ptr<int>(), sp, batch,
                             int(block_tables.size(1)), block_size, stream_of(positions), err, errlen));
}

// per-slice (value, index bits) pairs of every row: float32 [chunks, rows, 2]
at::Tensor argmax_parts(const at::Tensor& logits, int offset, c10::optional<at::Tensor> out_opt) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 &&
                  logits.stride(1) == 1,
              "barlink: argmax needs 2-D bfloat16 CUDA logits");
  const int rows = int(logits.size(0)), n = int(logits.size(1));
  at::Tensor parts = out_opt ? *out_opt
                             : at::empty({bl_argmax_chunks(), rows, 2}, logits.options().dtype(at::kFloat));
  TORCH_CHECK(parts.is_cuda() && parts.is_contiguous() && parts.scalar_type() == at::kFloat &&
                  parts.numel() == int64_t(bl_argmax_chunks()) * rows * 2,
              "barlink: argmax_parts out must be contiguous float32 [chunks, rows, 2]");
  c10::cuda::CUDAGuard guard(logits.device());
  if (rows > 0)
    BL_CHECK(bl_argmax_parts(logits.data_ptr(), rows, n, int(logits.stride(0)), offset, parts.data_ptr(),
                             stream_of(logits), err, errlen));
  return parts;
}

at::Tensor argmax_merge(const at::Tensor& pairs, c10::optional<at::Tensor> out_opt) {
  TORCH_CHECK(pairs.is_cuda() && pairs.scalar_type() == at::kFloat && pairs.dim() == 3 &&
                  pairs.size(2) == 2 && pairs.is_contiguous(),
              "barlink: argmax_merge needs float32 [world, rows, 2] (value, index bits)");
  const int world = int(pairs.size(0)), rows = int(pairs.size(1));
  at::Tensor idx = out_opt ? *out_opt : at::empty({rows}, pairs.options().dtype(at::kInt));
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.is_contiguous() && idx.numel() == rows,
              "barlink: argmax_merge out must be contiguous int32 [rows]");
  c10::cuda::CUDAGuard guard(pairs.device());
  BL_CHECK(bl_argmax_merge(pairs.data_ptr(), world, rows, idx.data_ptr<int>(), stream_of(pairs), err,
                           errlen));
  return idx;
}

at::Tensor paged_attn_decode(const at::Tensor& qkv, const at::Tensor& k_cache,
                             const at::Tensor& v_cache, const at::Tensor& block_tables,
                             const at::Tensor& ctx_lens, int nq, int nkv, int hd, double scale,
                             int splits, c10::optional<at::Tensor> out_opt) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 &&
                  qkv.stride(1) == 1,
              "barlink: q/qkv must be a 2-D bfloat16 CUDA tensor");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(1) == nkv && k_cache.size(3) == hd,
              "barlink: cache layout is [blocks, nkv, block_size, head_dim]");
  TORCH_CHECK(block_tables.is_cuda() && block_tables.scalar_type() == at::kInt &&
                  block_tables.dim() == 2 && block_tables.is_contiguous(),
              "barlink: block_tables must be contiguous int32 [batch, max_blocks]");
  TORCH_CHECK(ctx_lens.is_cuda() && ctx_lens.scalar_type() == at::kInt, "barlink: ctx_lens must be int32");
  const int batch = int(qkv.size(0));
  TORCH_CHECK(block_tables.size(0) == batch && ctx_lens.numel() == batch, "barlink: batch mismatch");
  TORCH_CHECK(qkv.size(1) >= int64_t(nq) * hd, "barlink: q rows too short");
  at::Tensor out = out_opt ? *out_opt : at::empty({batch, int64_t(nq) * hd}, qkv.options());
  const int dev = qkv.device().index();
  c10::cuda::CUDAGuard guard(qkv.device());
  Scratch& s = scratch_for(dev);
  if (batch > 0)
    BL_CHECK(bl_paged_attn_decode(qkv.data_ptr(), int(qkv.stride(0)), k_cache.data_ptr(),
                                  v_cache.data_ptr(), block_tables.data_ptr<int>(),
                                  ctx_lens.data_ptr<int>(), out.data_ptr(), batch, nq, nkv, hd,
                                  int(k_cache.size(2)), int(block_tables.size(1)), float(scale),
                                  splits, s.attn.data_ptr(), size_t(s.attn.nbytes()),
                                  stream_of(qkv), err, errlen));
  return out;
}

// qkv: bf16 [batch, width] or fp32 k-split slabs [splits, batch, width] of the QKV linear
at::Tensor rope_attn_decode(const at::Tensor& qkv, const c10::optional<at::Tensor>& bias,
                            const at::Tensor& positions, const at::Tensor& slots, at::Tensor& k_cache,
                            at::Tensor& v_cache, const at::Tensor& block_tables, const at::Tensor& ctx_lens,
                            int nq, int nkv, int hd, double theta, double scale, int splits,
                            bool merge_in_kernel) {
  const bool slabs = qkv.scalar_type() == at::kFloat && qkv.dim() == 3;
  TORCH_CHECK(qkv.is_cuda() && qkv.is_contiguous() &&
                  (slabs || (qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2)),
              "barlink: qkv must be contiguous bfloat16 [batch, width] or float32 slabs [splits, batch, width]");
  const int batch = int(qkv.size(slabs ? 1 : 0)), width = int(qkv.size(slabs ? 2 : 1));
  TORCH_CHECK(width == (nq + 2 * nkv) * hd, "barlink: qkv rows must hold nq + 2 nkv heads");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(1) == nkv && k_cache.size(3) == hd,
              "barlink: cache layout is [blocks, nkv, block_size, head_dim]");
  TORCH_CHECK(block_tables.is_cuda() && block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 &&
                  block_tables.is_contiguous() && block_tables.size(0) == batch,
              "barlink: block_tables must be contiguous int32 [batch, max_blocks]");
  for (const at::Tensor* t : {&positions, &slots, &ctx_lens})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous() && t->numel() == batch,
                "barlink: positions / slots / ctx_lens must be contiguous int32 [batch]");
  if (bias) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == width, "barlink: bias must have one entry per qkv column");
  }
  at::Tensor out = at::empty({batch, int64_t(nq) * hd}, k_cache.options());
  const int dev = qkv.device().index();
  c10::cuda::CUDAGuard guard(qkv.device());
  Scratch& s = scratch_for(dev);
  if (batch > 0)
    BL_CHECK(bl_rope_attn_decode(slabs ? nullptr : qkv.data_ptr(), width, slabs ? qkv.data_ptr() : nullptr,
                                 slabs ? int(qkv.size(0)) : 0, size_t(batch) * width,
                                 bias ? bias->data_ptr() : nullptr, positions.data_ptr<int>(),
                                 slots.data_ptr<int>(), float(theta), k_cache.data_ptr(), v_cache.data_ptr(),
                                 block_tables.data_ptr<int>(), ctx_lens.data_ptr<int>(), out.data_ptr(), batch,
                                 nq, nkv, hd, int(k_cache.size(2)), int(block_tables.size(1)), float(scale),
                                 splits, s.attn.data_ptr(), size_t(s.attn.nbytes()),
                                 merge_in_kernel ? s.attn_counters.data_ptr() : nullptr, stream_of(qkv), err,
                                 errlen));
  return out;
}

}  // namespace

void bind_extra(py::module_& m);  // binding_extra.cc: attention prefill, W8A16, fused TP linears

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "barlink for B200: NVLink peer-memory collectives, tcgen05 linears, decode kernels";
  m.def("init", &init, py::arg("devices"), py::arg("pool_mb") = 64);
  m.def("init_peer", &init_peer, py::arg("device"), py::arg("pool_mb") = 64, py::arg("sock_path"),
        py::arg("rank"), py::arg("world") = 2);
  m.def("shutdown", &py_shutdown);
  m.def("info", &info);
  m.def("empty", &empty, py::arg("nbytes"), py::arg("device") = 0, py::arg("dtype") = py::none());
  m.def("free_", &free_, py::arg("tensor"), py::arg("device") = 0);
  m.def("pool_offset", &pool_offset, py::arg("tensor"), py::arg("device") = 0);
  m.def("copy_", &copy_);
  m.def("allreduce_", &allreduce_);
  m.def("allreduce_into", &allreduce_into, py::arg("out"), py::arg("in"), py::arg("algo") = "auto");
  m.def("allgather_into", &allgather_into, py::arg("out"), py::arg("in"));
  m.def("reduce_scatter_into", &reduce_scatter_into, py::arg("out"), py::arg("in"));
  m.def("broadcast_", &broadcast_, py::arg("tensor"), py::arg("root"));
  m.def("barrier", &barrier);
  m.def("allreduce_rmsnorm", &allreduce_rmsnorm, py::arg("x"), py::arg("residual"), py::arg("gamma"),
        py::arg("eps"), py::arg("normed_out") = py::none(), py::arg("residual_out") = py::none());
  m.def("send_into", &send_into, py::arg("t"), py::arg("peer_rank"));
  m.def("recv_into", &recv_into, py::arg("t"), py::arg("peer_rank"));
  m.def("join_sends", &join_sends);
  m.def("verify", &verify);
  m.def("readback", &readback);
  m.def("pool_move", &pool_move, py::arg("out"), py::arg("src"));
  m.def("debug_flags", &debug_flags, py::arg("n") = 64);
  m.def("signal_probe", &signal_probe, py::arg("iters") = 1000);
  m.def("status", &status);
  m.def("reset", &reset);
  m.def("set_wait_timeout_ms", &set_wait_timeout_ms);
  m.def("stats", &stats);

  m.def("linear", &linear, py::arg("x"), py::arg("weight"), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("silu_mul") = false, py::arg("out") = py::none(),
        py::arg("force_swap") = -1, py::arg("bn") = 0, py::arg("splits") = 0,
        py::arg("dynamic_weights") = false, py::arg("trace") = py::none(), py::arg("gate_tokens") = 0,
        py::arg("tiled_n") = 0, py::arg("tiled_k") = 0, py::arg("gelu") = false);
  m.def("linear_push", &linear_push, py::arg("x"), py::arg("weight"), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("gelu") = false, py::arg("total_rows"), py::arg("row0") = 0);
  m.def("allreduce_pushed", &allreduce_pushed, py::arg("out"), py::arg("units"));
  m.def("gemm_error_flag", &gemm_error_flag, py::arg("device") = 0);
  m.def("rmsnorm", &rmsnorm, py::arg("x"), py::arg("gamma"), py::arg("eps"),
        py::arg("residual") = py::none(), py::arg("out") = py::none());
  m.def("rope_kv_write", &rope_kv_write, py::arg("qkv"), py::arg("positions"),
        py::arg("slots") = py::none(), py::arg("k_cache") = py::none(),
        py::arg("v_cache") = py::none(), py::arg("nq"), py::arg("nkv"), py::arg("hd"),
        py::arg("block_size") = 16, py::arg("theta") = 1e6, py::arg("bias") = py::none(),
        py::arg("out") = py::none());
  m.def("linear_partial", &linear_partial, py::arg("x"), py::arg("weight"), py::arg("splits") = 0,
        py::arg("out") = py::none(), py::arg("gate_tokens") = 0, py::arg("tiled_n") = 0,
        py::arg("tiled_k") = 0);
  m.def("tile_weight", &tile_weight, py::arg("weight"));
  m.def("tp_gemm_rs", &tp_gemm_rs, py::arg("x"), py::arg("weight"), py::arg("inbox"),
        py::arg("tiled_n") = 0, py::arg("tiled_k") = 0);
  m.def("tp_rs_finish", &tp_rs_finish, py::arg("inbox"), py::arg("gather"), py::arg("residual"),
        py::arg("gamma"), py::arg("eps"), py::arg("tokens"), py::arg("splits"), py::arg("units"),
        py::arg("add_residual") = true);
  m.def("gemm_splits", &gemm_splits, py::arg("n"), py::arg("k"), py::arg("tokens"));
  m.def("rope", &rope, py::arg("x"), py::arg("positions"), py::arg("heads"), py::arg("hd"),
        py::arg("theta") = 1e4, py::arg("axes") = 1);
  m.def("silu_mul", &silu_mul, py::arg("gate_up"), py::arg("interleaved") = false);
  m.def("embedding", &embedding, py::arg("ids"), py::arg("table"), py::arg("vocab_lo") = 0,
        py::arg("out") = py::none());
  m.def("argmax", &argmax, py::arg("logits"), py::arg("offset") = 0);
  m.def("argmax_merge", &argmax_merge, py::arg("pairs"), py::arg("out") = py::none());
  m.def("argmax_parts", &argmax_parts, py::arg("logits"), py::arg("offset") = 0, py::arg("out") = py::none());
  m.def("decode_advance", &decode_advance, py::arg("positions"), py::arg("ctx_lens"), py::arg("slots"),
        py::arg("block_tables"), py::arg("ids"), py::arg("sampled") = py::none(),
        py::arg("block_size") = 16);
  m.def("rope_attn_decode", &rope_attn_decode, py::arg("qkv"), py::arg("bias"), py::arg("positions"),
        py::arg("slots"), py::arg("k_cache"), py::arg("v_cache"), py::arg("block_tables"), py::arg("ctx_lens"),
        py::arg("nq"), py::arg("nkv"), py::arg("hd"), py::arg("theta"), py::arg("scale"), py::arg("splits") = 0,
        py::arg("merge_in_kernel") = true);
  m.def("paged_attn_decode", &paged_attn_decode, py::arg("qkv"), py::arg("k_cache"),
        py::arg("v_cache"), py::arg("block_tables"), py::arg("ctx_lens"), py::arg("nq"),
        py::arg("nkv"), py::arg("hd"), py::arg("scale"), py::arg("splits") = 0,
        py::arg("out") = py::none());

  py::class_<blpg::BarlinkBackend, c10::intrusive_ptr<blpg::BarlinkBackend>, c10d::Backend>(
      m, "BarlinkBackend")
      .def(py::init([](int rank, int size, const c10::intrusive_ptr<c10d::Backend>& cpu_backend,
                       bool use_link) {
             return c10::make_intrusive<blpg::BarlinkBackend>(rank, size, cpu_backend, use_link);
           }),
           py::arg("rank"), py::arg("size"), py::arg("cpu_backend") = py::none(),
           py::arg("use_link") = false)
      .def_readonly("n_zero_copy", &blpg::BarlinkBackend::n_zero_copy)
      .def_readonly("n_staged", &blpg::BarlinkBackend::n_staged)
      .def_readonly("n_cpu", &blpg::BarlinkBackend::n_cpu)
      .def_readonly("n_local", &blpg::BarlinkBackend::n_local)
      .def_readonly("n_host_staged", &blpg::BarlinkBackend::n_host_staged);

  bind_extra(m);
}
