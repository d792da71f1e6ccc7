// SPDX-License-Identifier: MIT
//
// Second half of the `_C` binding: single-process forms of the collectives
// (ranks that share a GPU), dense attention, W8A16 and the fused
// GEMM+collective tensor-parallel linears.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "backend.h"
#include "bl_core.h"
#include "bl_ops.h"

namespace py = pybind11;

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
  blCtx* c = blpg::global_ctx();
  TORCH_CHECK(c != nullptr, "barlink: not initialised -- call init(devices, pool_mb) or init_peer(...) first");
  return c;
}

int kind_code(const std::string& k) {
  if (k == "allreduce") return 0;
  if (k == "reduce_scatter") return 1;
  if (k == "allgather") return 2;
  if (k == "broadcast") return 3;
  if (k == "allreduce_rmsnorm") return 4;
  if (k == "barrier") return 5;
  TORCH_CHECK(false, "barlink: unknown collective '", k, "'");
}
int algo_code2(const std::string& a) {
  if (a == "oneshot") return BL_ALGO_ONESHOT;
  if (a == "twoshot") return BL_ALGO_TWOSHOT;
  if (a == "nvls") return BL_ALGO_NVLS;
  return BL_ALGO_AUTO;
}

// one tensor per rank in every list; lists may be empty when the collective
// does not use them
void sp_collective(const std::string& kind, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs,
                   std::vector<at::Tensor> aux_in, std::vector<at::Tensor> aux_out,
                   std::vector<at::Tensor> gamma, const std::string& algo, int root, double eps) {
  blCtx* c = ctx_or_throw();
  const int world = bl_world(c);
  const int k = kind_code(kind);
  auto ptrs = [&](std::vector<at::Tensor>& v, const char* name) {
    std::vector<void*> p;
    if (v.empty()) return p;
    TORCH_CHECK(int(v.size()) == world, "barlink: ", name, " needs one tensor per rank (", world, ")");
    for (auto& t : v) {
      TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "barlink: ", name, " tensors must be contiguous CUDA tensors");
      p.push_back(t.data_ptr());
    }
    return p;
  };
  std::vector<void*> pi = ptrs(ins, "ins"), po = ptrs(outs, "outs"), pai = ptrs(aux_in, "aux_in"),
                     pao = ptrs(aux_out, "aux_out"), pg = ptrs(gamma, "gamma");
  std::vector<void*> streams(world, nullptr);
  int dtype = BL_DTYPE_U8;
  size_t bytes = 0;
  int rows = 0, hidden = 0;
  if (k != 5) {
    TORCH_CHECK(!ins.empty() && !outs.empty(), "barlink: ins and outs are required");
    dtype = blpg::dtype_code(ins[0].scalar_type());
    TORCH_CHECK(dtype >= 0, "barlink: unsupported dtype ", ins[0].scalar_type());
    bytes = (k == 1) ? outs[0].nbytes() : ins[0].nbytes();
    if (k == 4) {
      hidden = int(ins[0].size(-1));
      rows = int(ins[0].numel() / hidden);
    }
    for (int r = 0; r < world; ++r)
      streams[r] = at::cuda::getCurrentCUDAStream(ins[r].device().index()).stream();
  } else {
    for (int r = 0; r < world; ++r) streams[r] = at::cuda::getCurrentCUDAStream().stream();
  }
  py::gil_scoped_release nogil;
  BL_CHECK(bl_sp_collective(c, k, pi.empty() ? nullptr : pi.data(), po.empty() ? nullptr : po.data(),
                            pai.empty() ? nullptr : pai.data(), pao.empty() ? nullptr : pao.data(),
                            pg.empty() ? nullptr : pg.data(), bytes, dtype, algo_code2(algo), root,
                            rows, hidden, float(eps), streams.data(), err, errlen));
}

void sp_sendrecv(int src, int dst, const at::Tensor& in, const at::Tensor& out) {
  blCtx* c = ctx_or_throw();
  TORCH_CHECK(in.is_cuda() && out.is_cuda() && in.is_contiguous() && out.is_contiguous() &&
                  in.nbytes() == out.nbytes(),
              "barlink: sp_sendrecv needs contiguous CUDA tensors of equal size");
  void* st = at::cuda::getCurrentCUDAStream(in.device().index()).stream();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_sp_sendrecv(c, src, dst, in.data_ptr(), out.data_ptr(), in.nbytes(), st, err, errlen));
}

// q [T, nq, hd], k / v [Tk, nkv, hd] (token stride free, heads and dims dense)
at::Tensor attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                    const at::Tensor& cu_q, const at::Tensor& cu_k, int max_q, double scale,
                    bool causal) {
  auto chk = [](const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.stride(2) == 1 &&
                    t.stride(1) == t.size(2),
                "barlink: ", name, " must be a bfloat16 CUDA tensor [tokens, heads, head_dim] with dense heads");
  };
  chk(q, "q");
  chk(k, "k");
  chk(v, "v");
  TORCH_CHECK(cu_q.is_cuda() && cu_q.scalar_type() == at::kInt && cu_k.is_cuda() &&
                  cu_k.scalar_type() == at::kInt && cu_q.numel() == cu_k.numel() && cu_q.numel() >= 2,
              "barlink: cu_q / cu_k must be int32 CUDA tensors of batch + 1 entries");
  const int batch = int(cu_q.numel()) - 1;
  const int nq = int(q.size(1)), nkv = int(k.size(1)), hd = int(q.size(2));
  at::Tensor out = at::empty({q.size(0), nq, hd}, q.options());
  c10::cuda::CUDAGuard guard(q.device());
  void* st = at::cuda::getCurrentCUDAStream(q.device().index()).stream();
  if (q.size(0) > 0)
    BL_CHECK(bl_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                         cu_q.data_ptr<int>(), cu_k.data_ptr<int>(), batch, max_q, nq, nkv, hd,
                         int(q.stride(0)), int(k.stride(0)), int(v.stride(0)), nq * hd, float(scale),
                         causal ? 1 : 0, st, err, errlen));
  return out;
}

}  // namespace

void bind_extra(py::module_& m) {
  m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("cu_q"),
        py::arg("cu_k"), py::arg("max_q"), py::arg("scale"), py::arg("causal"));
  m.def("sp_collective", &sp_collective, py::arg("kind"), py::arg("ins") = std::vector<at::Tensor>{},
        py::arg("outs") = std::vector<at::Tensor>{}, py::arg("aux_in") = std::vector<at::Tensor>{},
        py::arg("aux_out") = std::vector<at::Tensor>{}, py::arg("gamma") = std::vector<at::Tensor>{},
        py::arg("algo") = "auto", py::arg("root") = 0, py::arg("eps") = 1e-6);
  m.def("sp_sendrecv", &sp_sendrecv, py::arg("src"), py::arg("dst"), py::arg("inp"), py::arg("out"));
}
