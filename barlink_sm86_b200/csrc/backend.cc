// SPDX-License-Identifier: MIT
//
// c10d backend "barlink": routes torch.distributed collectives onto the link
// core (CUDA tensors) or onto an inner gloo backend (CPU tensors).
// See backend.h for the contract kept from the reference's Python backend
// (torch_ext/barlink_sm86/process_group.py:134-520).
#include <stdio.h>
#include <stdlib.h>

#include "backend.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

namespace blpg {

static blCtx* g_ctx = nullptr;
blCtx* global_ctx() { return g_ctx; }
void set_global_ctx(blCtx* ctx) { g_ctx = ctx; }

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kByte: return BL_DTYPE_U8;
    case at::kFloat: return BL_DTYPE_FP32;
    case at::kDouble: return BL_DTYPE_FP64;
    case at::kBFloat16: return BL_DTYPE_BF16;
    case at::kHalf: return BL_DTYPE_FP16;
    case at::kFloat8_e4m3fn: return BL_DTYPE_FP8E4M3;
    case at::kFloat8_e5m2: return BL_DTYPE_FP8E5M2;
    default: return -1;
  }
}

DoneWork::DoneWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs)
    : c10d::Work(rank, op), outputs_(std::move(outputs)) {
  future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
  future_->markCompleted(c10::IValue(outputs_));
}
c10::intrusive_ptr<c10::ivalue::Future> DoneWork::getFuture() { return future_; }

BarlinkBackend::BarlinkBackend(int rank, int size, c10::intrusive_ptr<c10d::Backend> cpu_backend,
                               bool use_link)
    : c10d::Backend(rank, size), cpu_(std::move(cpu_backend)), use_link_(use_link) {
  if (use_link_ && size > 1) {
    blCtx* c = global_ctx();
    TORCH_CHECK(c != nullptr, "barlink: the link is not initialised (call init_peer first)");
    TORCH_CHECK(bl_is_peer(c), "barlink: a process group needs the SPMD link (init_peer), not init()");
    TORCH_CHECK(bl_world(c) == size && bl_rank(c) == rank,
                "barlink: process group (rank ", rank, " of ", size,
                ") does not match the link (rank ", bl_rank(c), " of ", bl_world(c),
                "); groups smaller than the world are supported only with one member");
  }
}

void BarlinkBackend::drain_sends() {
  for (auto& e : inflight_) {
    cudaEventSynchronize(e.first);
    cudaEventDestroy(e.first);
  }
  cudaGetLastError();
  inflight_.clear();
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::done(c10d::OpType op, std::vector<at::Tensor> outs) {
  return c10::make_intrusive<DoneWork>(getRank(), op, std::move(outs));
}

c10d::Backend& BarlinkBackend::cpu(const char* what) {
  TORCH_CHECK(cpu_, "barlink: ", what, " on a CPU tensor needs the gloo companion backend, which this group was created without");
  ++n_cpu;
  return *cpu_;
}

// A CUDA tensor in a group that the link does not serve (a subgroup of 2..world-1 ranks, e.g. the
// tensor-parallel group of a TP x PP job): staged through host memory and the gloo companion.
// Slow, but the group works; the hot groups (the whole world) never take this path.
bool BarlinkBackend::host_staged(const at::Tensor& t) {
  if (!t.is_cuda() || use_link_ || !cpu_) return false;
  ++n_host_staged;
  return true;
}

static void* cur_stream(const at::Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}
static bool aligned_ok(const at::Tensor& t) {
  return t.is_contiguous() && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0 &&
         (t.nbytes() & 15u) == 0 && t.nbytes() > 0;
}
#define BL_CALL(expr)                              \
  do {                                             \
    char _e[512] = {0};                            \
    char* err = _e;                                \
    size_t errlen = sizeof(_e);                    \
    int _rc = (expr);                              \
    TORCH_CHECK(_rc == 0, _e[0] ? _e : "barlink: link call failed"); \
  } while (0)

blCtx* BarlinkBackend::link() {
  TORCH_CHECK(use_link_,
              "barlink: this group has no GPU link (it was created on a host without CUDA, with "
              "BL_CPU_ONLY=1, or it is a subgroup of 2..world-1 ranks, which the link does not serve); "
              "CUDA tensors cannot be communicated through it");
  blCtx* c = global_ctx();
  TORCH_CHECK(c != nullptr, "barlink: the link is not initialised");
  return c;
}

// padded flat staging copy of a tensor: numel rounded up so that bytes % 16 == 0
static at::Tensor padded_copy(const at::Tensor& t) {
  const int64_t isz = t.element_size();
  const int64_t per = 16 / std::min<int64_t>(16, isz) > 0 ? 16 / std::min<int64_t>(16, isz) : 1;
  const int64_t n = t.numel();
  const int64_t np = (n + per - 1) / per * per;
  at::Tensor tmp = at::zeros({np}, t.options());
  tmp.narrow(0, 0, n).copy_(t.reshape({-1}));
  return tmp;
}

void BarlinkBackend::allreduce_cuda(at::Tensor& t) {
  const int code = dtype_code(t.scalar_type());
  TORCH_CHECK(code >= 0, "barlink: all_reduce does not support dtype ", t.scalar_type(),
              " (supported: uint8, float16, bfloat16, float32, float64, float8_e4m3fn, float8_e5m2)");
  if (t.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(t.device());
  void* st = cur_stream(t);
  const size_t chunk = bl_max_chunk(c) & ~size_t(15);
  auto run = [&](char* p, size_t bytes) {
    for (size_t off = 0; off < bytes; off += chunk) {
      const size_t len = std::min(chunk, bytes - off);
      BL_CALL(bl_allreduce_into_peer(c, p + off, p + off, len, code, BL_ALGO_AUTO, st, err, errlen));
    }
  };
  // ablation / debug switches of the reference's backend (torch_ext/barlink_sm86/process_group.py:
  // 137-148 BL_AR_TRACE, :185 BL_AR_NO_ZC): force the staged path; print a checksum per call
  static const bool no_zc = getenv("BL_AR_NO_ZC") && getenv("BL_AR_NO_ZC")[0] != '0';
  static const bool trace = getenv("BL_AR_TRACE") && getenv("BL_AR_TRACE")[0] != '0';
  double before = 0.0;
  if (trace) before = t.to(at::kDouble).sum().item<double>();
  if (aligned_ok(t) && !no_zc) {
    ++n_zero_copy;
    run(static_cast<char*>(t.data_ptr()), t.nbytes());
  } else {
    ++n_staged;
    at::Tensor tmp = padded_copy(t);
    run(static_cast<char*>(tmp.data_ptr()), tmp.nbytes());
    t.copy_(tmp.narrow(0, 0, t.numel()).view(t.sizes()));
  }
  if (trace) {
    // synchronises: a debugging aid, never on in a timed run
    const double after = t.to(at::kDouble).sum().item<double>();
    fprintf(stderr, "[barlink rank %d] all_reduce #%llu %s %lld elements: checksum %.6g -> %.6g (%s)\n", getRank(),
            (unsigned long long)(n_zero_copy + n_staged), c10::toString(t.scalar_type()), (long long)t.numel(),
            before, after, (aligned_ok(t) && !no_zc) ? "zero-copy" : "staged");
  }
}

void BarlinkBackend::allgather_cuda(at::Tensor& out, const at::Tensor& in) {
  const int world = getSize();
  TORCH_CHECK(out.numel() == in.numel() * world && out.scalar_type() == in.scalar_type(),
              "barlink: all_gather output must hold world x input elements of the same dtype");
  if (in.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(in.device());
  void* st = cur_stream(in);
  const size_t slice = (bl_max_chunk(c) / size_t(world)) & ~size_t(15);
  auto run = [&](const char* ip, char* op, size_t bytes) {
    for (size_t off = 0; off < bytes; off += slice) {
      const size_t len = std::min(slice, bytes - off);
      BL_CALL(bl_allgather_peer(c, ip + off, op + off, len, bytes, st, err, errlen));
    }
  };
  if (aligned_ok(in) && aligned_ok(out)) {
    ++n_zero_copy;
    run(static_cast<const char*>(in.data_ptr()), static_cast<char*>(out.data_ptr()), in.nbytes());
  } else {
    ++n_staged;
    at::Tensor ti = padded_copy(in);
    at::Tensor to = at::empty({world, ti.numel()}, ti.options());
    run(static_cast<const char*>(ti.data_ptr()), static_cast<char*>(to.data_ptr()), ti.nbytes());
    out.copy_(to.narrow(1, 0, in.numel()).reshape(out.sizes()));
  }
}

void BarlinkBackend::reduce_scatter_cuda(at::Tensor& out, const at::Tensor& in) {
  const int world = getSize();
  const int code = dtype_code(in.scalar_type());
  TORCH_CHECK(code >= 0, "barlink: reduce_scatter does not support dtype ", in.scalar_type());
  TORCH_CHECK(in.numel() == out.numel() * world && out.scalar_type() == in.scalar_type(),
              "barlink: reduce_scatter input must hold world x output elements of the same dtype");
  if (out.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(in.device());
  void* st = cur_stream(in);
  const size_t slice = (bl_max_chunk(c) / size_t(world)) & ~size_t(15);
  auto run = [&](const char* ip, char* op, size_t bytes) {
    for (size_t off = 0; off < bytes; off += slice) {
      const size_t len = std::min(slice, bytes - off);
      BL_CALL(bl_reduce_scatter_peer(c, ip + off, op + off, len, bytes, code, st, err, errlen));
    }
  };
  if (aligned_ok(in) && aligned_ok(out)) {
    ++n_zero_copy;
    run(static_cast<const char*>(in.data_ptr()), static_cast<char*>(out.data_ptr()), out.nbytes());
  } else {
    ++n_staged;
    const int64_t n = out.numel();
    at::Tensor to = padded_copy(out);
    at::Tensor ti = at::zeros({world, to.numel()}, in.options());
    ti.narrow(1, 0, n).copy_(in.reshape({world, n}));
    run(static_cast<const char*>(ti.data_ptr()), static_cast<char*>(to.data_ptr()), to.nbytes());
    out.copy_(to.narrow(0, 0, n).view(out.sizes()));
  }
}

void BarlinkBackend::broadcast_cuda(at::Tensor& t, int root) {
  if (t.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(t.device());
  void* st = cur_stream(t);
  const size_t slice = (bl_max_chunk(c) / size_t(getSize())) & ~size_t(15);
  auto run = [&](char* p, size_t bytes) {
    for (size_t off = 0; off < bytes; off += slice) {
      const size_t len = std::min(slice, bytes - off);
      BL_CALL(bl_broadcast_peer(c, p + off, len, root, st, err, errlen));
    }
  };
  if (aligned_ok(t)) {
    ++n_zero_copy;
    run(static_cast<char*>(t.data_ptr()), t.nbytes());
  } else {
    ++n_staged;
    at::Tensor tmp = padded_copy(t);
    run(static_cast<char*>(tmp.data_ptr()), tmp.nbytes());
    if (getRank() != root) t.copy_(tmp.narrow(0, 0, t.numel()).view(t.sizes()));
  }
}

static size_t p2p_chunk(blCtx* c) { return bl_p2p_chunk(c) & ~size_t(15); }

void BarlinkBackend::send_cuda(const at::Tensor& t, int dst) {
  TORCH_CHECK(dst != getRank(), "barlink: send to self is not supported");
  TORCH_CHECK(dst >= 0 && dst < getSize(), "barlink: send destination ", dst, " out of range");
  if (t.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(t.device());
  void* st = cur_stream(t);
  const size_t chunk = p2p_chunk(c);
  at::Tensor src = t;
  if (!aligned_ok(t)) {
    ++n_staged;
    src = padded_copy(t);
  } else {
    ++n_zero_copy;
  }
  const char* p = static_cast<const char*>(src.data_ptr());
  const size_t bytes = src.nbytes();
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    BL_CALL(bl_send_into_peer(c, p + off, len, dst, st, err, errlen));
  }
  // Sends run on the link's own stream so that a recv queued behind them can
  // make progress (several sends outstanding before the first recv would
  // otherwise deadlock a pair).  The buffer is kept alive here until that
  // stream has read it; any later collective joins the stream.
  if (void* ss = bl_send_stream(c)) {
    while (!inflight_.empty() && cudaEventQuery(inflight_.front().first) == cudaSuccess) {
      cudaEventDestroy(inflight_.front().first);
      inflight_.pop_front();
    }
    cudaGetLastError();
    cudaEvent_t ev;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
      cudaEventRecord(ev, static_cast<cudaStream_t>(ss));
      inflight_.emplace_back(ev, src);
    }
  }
}

void BarlinkBackend::recv_cuda(at::Tensor& t, int src) {
  TORCH_CHECK(src != getRank(), "barlink: recv from self is not supported");
  TORCH_CHECK(src >= 0 && src < getSize(), "barlink: recv source ", src, " out of range");
  if (t.numel() == 0) return;
  blCtx* c = link();
  c10::cuda::CUDAGuard guard(t.device());
  void* st = cur_stream(t);
  const size_t chunk = p2p_chunk(c);
  const bool direct = aligned_ok(t);
  at::Tensor dst = direct ? t : padded_copy(t);
  direct ? ++n_zero_copy : ++n_staged;
  char* p = static_cast<char*>(dst.data_ptr());
  const size_t bytes = dst.nbytes();
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    BL_CALL(bl_recv_into_peer(c, p + off, len, src, st, err, errlen));
  }
  if (!direct) t.copy_(dst.narrow(0, 0, t.numel()).view(t.sizes()));
}

// MAX / MIN / PRODUCT / AVG: the reduce kernels of the link only add, so these
// (control-plane sized in practice: loss scales, timings, flags) gather every
// rank's tensor over the link and reduce locally.
void BarlinkBackend::allreduce_other_cuda(at::Tensor& t, const c10d::ReduceOp& op) {
  // argument errors surface before any rank has put traffic on the link
  TORCH_CHECK(op == c10d::ReduceOp::MAX || op == c10d::ReduceOp::MIN || op == c10d::ReduceOp::PRODUCT ||
                  op == c10d::ReduceOp::AVG,
              "barlink: all_reduce on CUDA tensors supports SUM, AVG, MAX, MIN and PRODUCT");
  TORCH_CHECK(t.is_contiguous(), "barlink: all_reduce needs a contiguous tensor");
  c10::cuda::CUDAGuard guard(t.device());
  const int64_t n = t.numel();
  if (n == 0) return;
  // pad to a 16-byte multiple so that the gather runs zero-copy sized chunks
  const int64_t esz = int64_t(t.element_size());
  const int64_t padded = (n * esz + 15) / 16 * 16 / esz;
  at::Tensor in = at::zeros({padded}, t.options());
  in.narrow(0, 0, n).copy_(t.view({-1}));
  at::Tensor all = at::empty({int64_t(getSize()) * padded}, t.options());
  allgather_cuda(all, in);
  at::Tensor rows = all.view({int64_t(getSize()), padded}).narrow(1, 0, n);
  at::Tensor r;
  if (op == c10d::ReduceOp::MAX) r = rows.amax(0);
  else if (op == c10d::ReduceOp::MIN) r = rows.amin(0);
  else if (op == c10d::ReduceOp::PRODUCT) r = rows.prod(0);
  else r = at::isFloatingType(t.scalar_type()) ? rows.mean(0) : rows.sum(0).floor_divide(int64_t(getSize()));
  t.view({-1}).copy_(r);
}

// ---------------------------------------------------------------------------

static void check_sum(const c10d::ReduceOp& op, const char* what) {
  TORCH_CHECK(op == c10d::ReduceOp::SUM, "barlink: ", what,
              " supports only ReduceOp.SUM on CUDA tensors");
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::allreduce(std::vector<at::Tensor>& tensors,
                                                         const c10d::AllreduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "barlink: all_reduce takes one tensor");
  at::Tensor& t = tensors[0];
  if (getSize() == 1) {
    ++n_local;
    return done(c10d::OpType::ALLREDUCE, tensors);
  }
  if (host_staged(t)) {
    std::vector<at::Tensor> h{t.cpu()};
    cpu_->allreduce(h, opts)->wait();
    t.copy_(h[0]);
    return done(c10d::OpType::ALLREDUCE, tensors);
  }
  if (t.is_cuda()) {
    if (opts.reduceOp == c10d::ReduceOp::SUM) {
      allreduce_cuda(t);
    } else {
      allreduce_other_cuda(t, opts.reduceOp);
    }
    return done(c10d::OpType::ALLREDUCE, tensors);
  }
  return cpu("all_reduce").allreduce(tensors, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::allreduce_coalesced(
    std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) {
  if (getSize() == 1) return done(c10d::OpType::ALLREDUCE_COALESCED, tensors);
  if (!tensors.empty() && tensors[0].is_cuda()) {
    check_sum(opts.reduceOp, "all_reduce_coalesced");
    for (auto& t : tensors) allreduce_cuda(t);
    return done(c10d::OpType::ALLREDUCE_COALESCED, tensors);
  }
  return cpu("all_reduce_coalesced").allreduce_coalesced(tensors, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::broadcast(std::vector<at::Tensor>& tensors,
                                                         const c10d::BroadcastOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "barlink: broadcast takes one tensor");
  if (getSize() == 1) {
    ++n_local;
    return done(c10d::OpType::BROADCAST, tensors);
  }
  if (host_staged(tensors[0])) {
    std::vector<at::Tensor> h{tensors[0].cpu()};
    cpu_->broadcast(h, opts)->wait();
    tensors[0].copy_(h[0]);
    return done(c10d::OpType::BROADCAST, tensors);
  }
  if (tensors[0].is_cuda()) {
    TORCH_CHECK(opts.rootRank >= 0 && opts.rootRank < getSize(), "barlink: broadcast root out of range");
    broadcast_cuda(tensors[0], int(opts.rootRank));
    return done(c10d::OpType::BROADCAST, tensors);
  }
  return cpu("broadcast").broadcast(tensors, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::barrier(const c10d::BarrierOptions& opts) {
  if (getSize() == 1) {
    ++n_local;
    return done(c10d::OpType::BARRIER, {});
  }
  if (use_link_) {
    blCtx* c = link();
    void* st = at::cuda::getCurrentCUDAStream().stream();
    BL_CALL(bl_barrier_peer(c, st, err, errlen));
    // a c10d barrier is a host-side meeting point as well
    AT_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(st)));
    return done(c10d::OpType::BARRIER, {});
  }
  return cpu("barrier").barrier(opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::_allgather_base(at::Tensor& output, at::Tensor& input,
                                                               const c10d::AllgatherOptions& opts) {
  if (getSize() == 1) {
    ++n_local;
    output.copy_(input.reshape(output.sizes()));
    return done(c10d::OpType::_ALLGATHER_BASE, {output});
  }
  if (host_staged(input)) {
    at::Tensor ho = at::empty(output.sizes(), output.options().device(at::kCPU)), hi = input.cpu();
    cpu_->_allgather_base(ho, hi, opts)->wait();
    output.copy_(ho);
    return done(c10d::OpType::_ALLGATHER_BASE, {output});
  }
  if (input.is_cuda()) {
    allgather_cuda(output, input);
    return done(c10d::OpType::_ALLGATHER_BASE, {output});
  }
  return cpu("all_gather_into_tensor")._allgather_base(output, input, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::allgather(
    std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
    const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "barlink: all_gather takes one input tensor");
  TORCH_CHECK(int(outputs[0].size()) == getSize(), "barlink: all_gather output list must have world entries");
  if (getSize() == 1) {
    ++n_local;
    outputs[0][0].copy_(inputs[0]);
    return done(c10d::OpType::ALLGATHER, outputs[0]);
  }
  if (host_staged(inputs[0])) {
    std::vector<std::vector<at::Tensor>> ho(1);
    for (auto& o : outputs[0]) ho[0].push_back(at::empty(o.sizes(), o.options().device(at::kCPU)));
    std::vector<at::Tensor> hi{inputs[0].cpu()};
    cpu_->allgather(ho, hi, opts)->wait();
    for (size_t r = 0; r < outputs[0].size(); ++r) outputs[0][r].copy_(ho[0][r]);
    return done(c10d::OpType::ALLGATHER, outputs[0]);
  }
  if (inputs[0].is_cuda()) {
    at::Tensor flat = at::empty({getSize(), inputs[0].numel()}, inputs[0].options());
    at::Tensor in = inputs[0].contiguous();
    allgather_cuda(flat, in);
    for (int r = 0; r < getSize(); ++r) outputs[0][r].copy_(flat[r].view(outputs[0][r].sizes()));
    return done(c10d::OpType::ALLGATHER, outputs[0]);
  }
  return cpu("all_gather").allgather(outputs, inputs, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::allgather_into_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
    const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size(), "barlink: coalesced all_gather needs matching lists");
  if (!inputs.empty() && !inputs[0].is_cuda() && getSize() > 1)
    return cpu("all_gather_into_tensor_coalesced").allgather_into_tensor_coalesced(outputs, inputs, opts);
  for (size_t i = 0; i < inputs.size(); ++i) {
    if (getSize() == 1) outputs[i].copy_(inputs[i].reshape(outputs[i].sizes()));
    else allgather_cuda(outputs[i], inputs[i]);
  }
  return done(c10d::OpType::ALLGATHER_COALESCED, outputs);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::_reduce_scatter_base(
    at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) {
  if (getSize() == 1) {
    ++n_local;
    output.copy_(input.reshape(output.sizes()));
    return done(c10d::OpType::_REDUCE_SCATTER_BASE, {output});
  }
  if (host_staged(input)) {
    at::Tensor ho = at::empty(output.sizes(), output.options().device(at::kCPU)), hi = input.cpu();
    cpu_->_reduce_scatter_base(ho, hi, opts)->wait();
    output.copy_(ho);
    return done(c10d::OpType::_REDUCE_SCATTER_BASE, {output});
  }
  if (input.is_cuda()) {
    check_sum(opts.reduceOp, "reduce_scatter");
    reduce_scatter_cuda(output, input);
    return done(c10d::OpType::_REDUCE_SCATTER_BASE, {output});
  }
  return cpu("reduce_scatter_tensor")._reduce_scatter_base(output, input, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::reduce_scatter(
    std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
    const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1, "barlink: reduce_scatter takes one output tensor");
  TORCH_CHECK(int(inputs[0].size()) == getSize(), "barlink: reduce_scatter input list must have world entries");
  if (getSize() == 1) {
    ++n_local;
    outputs[0].copy_(inputs[0][0]);
    return done(c10d::OpType::REDUCE_SCATTER, outputs);
  }
  if (outputs[0].is_cuda()) {
    check_sum(opts.reduceOp, "reduce_scatter");
    std::vector<at::Tensor> flat;
    for (auto& t : inputs[0]) flat.push_back(t.reshape({-1}));
    at::Tensor in = at::cat(flat, 0);
    reduce_scatter_cuda(outputs[0], in);
    return done(c10d::OpType::REDUCE_SCATTER, outputs);
  }
  return cpu("reduce_scatter").reduce_scatter(outputs, inputs, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::reduce_scatter_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
    const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size(), "barlink: coalesced reduce_scatter needs matching lists");
  if (!inputs.empty() && !inputs[0].is_cuda() && getSize() > 1)
    return cpu("reduce_scatter_tensor_coalesced").reduce_scatter_tensor_coalesced(outputs, inputs, opts);
  if (getSize() > 1) check_sum(opts.reduceOp, "reduce_scatter");
  for (size_t i = 0; i < inputs.size(); ++i) {
    if (getSize() == 1) outputs[i].copy_(inputs[i].reshape(outputs[i].sizes()));
    else reduce_scatter_cuda(outputs[i], inputs[i]);
  }
  return done(c10d::OpType::COALESCED, outputs);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::reduce(std::vector<at::Tensor>& tensors,
                                                      const c10d::ReduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "barlink: reduce takes one tensor");
  if (getSize() == 1) return done(c10d::OpType::REDUCE, tensors);
  if (tensors[0].is_cuda()) {
    check_sum(opts.reduceOp, "reduce");
    // every rank computes the sum; only the root keeps it
    at::Tensor tmp = tensors[0].clone();
    allreduce_cuda(tmp);
    if (getRank() == opts.rootRank) tensors[0].copy_(tmp);
    return done(c10d::OpType::REDUCE, tensors);
  }
  return cpu("reduce").reduce(tensors, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::gather(std::vector<std::vector<at::Tensor>>& outputs,
                                                      std::vector<at::Tensor>& inputs,
                                                      const c10d::GatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1, "barlink: gather takes one input tensor");
  if (getSize() == 1) {
    if (!outputs.empty()) outputs[0][0].copy_(inputs[0]);
    return done(c10d::OpType::GATHER, {});
  }
  if (inputs[0].is_cuda()) {
    at::Tensor flat = at::empty({getSize(), inputs[0].numel()}, inputs[0].options());
    at::Tensor in = inputs[0].contiguous();
    allgather_cuda(flat, in);
    if (getRank() == opts.rootRank) {
      TORCH_CHECK(outputs.size() == 1 && int(outputs[0].size()) == getSize(),
                  "barlink: gather root needs a list of world output tensors");
      for (int r = 0; r < getSize(); ++r) outputs[0][r].copy_(flat[r].view(outputs[0][r].sizes()));
    }
    return done(c10d::OpType::GATHER, {});
  }
  return cpu("gather").gather(outputs, inputs, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::scatter(std::vector<at::Tensor>& outputs,
                                                       std::vector<std::vector<at::Tensor>>& inputs,
                                                       const c10d::ScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1, "barlink: scatter takes one output tensor");
  if (getSize() == 1) {
    outputs[0].copy_(inputs[0][0]);
    return done(c10d::OpType::SCATTER, outputs);
  }
  if (outputs[0].is_cuda()) {
    // the root broadcasts the concatenation, every rank keeps its part
    at::Tensor all = at::empty({getSize(), outputs[0].numel()}, outputs[0].options());
    if (getRank() == opts.rootRank) {
      TORCH_CHECK(inputs.size() == 1 && int(inputs[0].size()) == getSize(),
                  "barlink: scatter root needs a list of world input tensors");
      for (int r = 0; r < getSize(); ++r) all[r].copy_(inputs[0][r].reshape({-1}));
    }
    broadcast_cuda(all, int(opts.rootRank));
    outputs[0].copy_(all[getRank()].view(outputs[0].sizes()));
    return done(c10d::OpType::SCATTER, outputs);
  }
  return cpu("scatter").scatter(outputs, inputs, opts);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::alltoall_base(at::Tensor& output, at::Tensor& input,
                                                             std::vector<int64_t>& outSplit,
                                                             std::vector<int64_t>& inSplit,
                                                             const c10d::AllToAllOptions& opts) {
  if (getSize() == 1) {
    output.copy_(input.reshape(output.sizes()));
    return done(c10d::OpType::ALLTOALL_BASE, {output});
  }
  if (!input.is_cuda()) return cpu("all_to_all").alltoall_base(output, input, outSplit, inSplit, opts);
  // Equal splits only: every rank gathers every input over the link and keeps the
  // slices addressed to it (world x the minimal traffic; the models of this library
  // have no all-to-all on their hot path, so this is a convenience, not a tuned kernel).
  TORCH_CHECK(outSplit.empty() && inSplit.empty(),
              "barlink: all_to_all on CUDA tensors supports equal splits only");
  const int64_t w = getSize();
  TORCH_CHECK(input.numel() == output.numel() && input.numel() % w == 0 && input.is_contiguous() &&
                  output.is_contiguous() && input.scalar_type() == output.scalar_type(),
              "barlink: all_to_all needs contiguous tensors of equal size, divisible by the world size");
  const int64_t per = input.numel() / w;
  at::Tensor all = at::empty({w, w, per}, input.options());
  at::Tensor in = input.view({-1});
  at::Tensor flat = all.view({-1});
  allgather_cuda(flat, in);
  // all[r][me] is what rank r addressed to this rank
  output.view({w, per}).copy_(all.select(1, getRank()));
  return done(c10d::OpType::ALLTOALL_BASE, {output});
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::send(std::vector<at::Tensor>& tensors, int dstRank,
                                                    int tag) {
  TORCH_CHECK(tensors.size() == 1, "barlink: send takes one tensor");
  if (host_staged(tensors[0])) {
    std::vector<at::Tensor> h{tensors[0].cpu()};
    cpu_->send(h, dstRank, tag)->wait();
    return done(c10d::OpType::SEND, {});
  }
  if (tensors[0].is_cuda()) {
    send_cuda(tensors[0], dstRank);
    return done(c10d::OpType::SEND, {});
  }
  return cpu("send").send(tensors, dstRank, tag);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::recv(std::vector<at::Tensor>& tensors, int srcRank,
                                                    int tag) {
  TORCH_CHECK(tensors.size() == 1, "barlink: recv takes one tensor");
  if (host_staged(tensors[0])) {
    std::vector<at::Tensor> h{at::empty(tensors[0].sizes(), tensors[0].options().device(at::kCPU))};
    cpu_->recv(h, srcRank, tag)->wait();
    tensors[0].copy_(h[0]);
    return done(c10d::OpType::RECV, tensors);
  }
  if (tensors[0].is_cuda()) {
    recv_cuda(tensors[0], srcRank);
    return done(c10d::OpType::RECV, tensors);
  }
  return cpu("recv").recv(tensors, srcRank, tag);
}

c10::intrusive_ptr<c10d::Work> BarlinkBackend::recvAnysource(std::vector<at::Tensor>& tensors,
                                                             int tag) {
  TORCH_CHECK(!tensors.empty() && !tensors[0].is_cuda(),
              "barlink: recv from any source is not supported on CUDA tensors (messages are matched by per-pair order)");
  return cpu("recv").recvAnysource(tensors, tag);
}

}  // namespace blpg
