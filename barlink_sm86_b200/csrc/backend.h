// SPDX-License-Identifier: MIT
//
// c10d backend "barlink" as a C++ class.  The reference implements its
// backend as a Python subclass of torch._C._distributed_c10d.Backend
// (torch_ext/barlink_sm86/process_group.py:69-520); that base has no Python
// constructor in current torch builds, so the class lives here and Python
// only registers a creator.  Semantics kept from the reference: collectives
// are stream-ordered and host-asynchronous and return an already completed
// Work (process_group.py:44-66); CUDA tensors go zero-copy when aligned and
// through a staged copy otherwise (:184-256); size-1 groups are honest local
// no-ops (:523-565); errors are raised before any traffic (:149-152).
// New: N <= 8 ranks, reduce_scatter, and CPU tensors served by an inner gloo
// backend so that the same group object works for host-side plumbing.
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/torch.h>

#include <cuda_runtime.h>

#include <deque>

#include "bl_core.h"

namespace blpg {

// singleton link context of this process (set by init / init_peer)
blCtx* global_ctx();
void set_global_ctx(blCtx* ctx);

int dtype_code(at::ScalarType t);  // BL_DTYPE_* or -1

class DoneWork : public c10d::Work {
 public:
  DoneWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs);
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override { return true; }
  void synchronize() override {}
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;

 private:
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class BarlinkBackend : public c10d::Backend {
 public:
  // cpu_backend may be null (CPU tensors then raise)
  BarlinkBackend(int rank, int size, c10::intrusive_ptr<c10d::Backend> cpu_backend, bool use_link);

  const std::string getBackendName() const override { return "barlink"; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(
      std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                           const c10d::BroadcastOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                           std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(
      at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors,
                                        const c10d::ReduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs,
                                        std::vector<at::Tensor>& inputs,
                                        const c10d::GatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs,
                                         std::vector<std::vector<at::Tensor>>& inputs,
                                         const c10d::ScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input,
                                               std::vector<int64_t>& outSplit,
                                               std::vector<int64_t>& inSplit,
                                               const c10d::AllToAllOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dstRank,
                                      int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int srcRank,
                                      int tag) override;
  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor>& tensors, int tag) override;

  void shutdown() override { drain_sends(); }
  void abort() override { drain_sends(); }
  ~BarlinkBackend() override { drain_sends(); }

  // counters for tests: how many ops took which path
  int64_t n_zero_copy = 0, n_staged = 0, n_cpu = 0, n_local = 0, n_host_staged = 0;

 private:
  c10::intrusive_ptr<c10d::Work> done(c10d::OpType op, std::vector<at::Tensor> outs);
  bool host_staged(const at::Tensor& t);
  void allreduce_cuda(at::Tensor& t);
  void allreduce_other_cuda(at::Tensor& t, const c10d::ReduceOp& op);
  void allgather_cuda(at::Tensor& out, const at::Tensor& in);
  void reduce_scatter_cuda(at::Tensor& out, const at::Tensor& in);
  void broadcast_cuda(at::Tensor& t, int root);
  void send_cuda(const at::Tensor& t, int dst);
  void recv_cuda(at::Tensor& t, int src);
  c10d::Backend& cpu(const char* what);
  blCtx* link();

  void drain_sends();

  c10::intrusive_ptr<c10d::Backend> cpu_;
  bool use_link_;
  // tensors handed to send() whose copy on the send stream may still be running
  std::deque<std::pair<cudaEvent_t, at::Tensor>> inflight_;
};

}  // namespace blpg
