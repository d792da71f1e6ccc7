// SPDX-License-Identifier: MIT
//
// Second half of the `_C` binding: single-process forms of the collectives
// (ranks that share a GPU), dense attention, W8A16 and the fused
// GEMM+collective tensor-parallel linears.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include <map>

#include "backend.h"
#include "bl_core.h"
#include "bl_ops.h"
#include "heap.h"

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
at::Tensor& attn_err(int dev) {
  static std::map<int, at::Tensor> m;
  auto it = m.find(dev);
  if (it != m.end()) return it->second;
  return m.emplace(dev, at::zeros({4}, at::TensorOptions().device(at::kCUDA, dev).dtype(at::kInt))).first->second;
}
int attn_error_flag(int dev) { return attn_err(dev).cpu()[0].item<int>(); }

// max_k > 0 (longest key sequence) selects the tcgen05 kernel; BL_ATTN_TC=0 keeps the mma.sync kernel
at::Tensor attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                    const at::Tensor& cu_q, const at::Tensor& cu_k, int max_q, double scale,
                    bool causal, int max_k) {
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
  static const bool tc_on = [] {
    const char* e = getenv("BL_ATTN_TC");
    return !(e && e[0] == '0');
  }();
  if (q.size(0) > 0 && tc_on && max_k > 0 && hd == 128) {
    at::Tensor vt = at::empty({int64_t(bl_attn_tc_scratch_bytes(batch, max_k, nkv) / 2)}, q.options());
    BL_CHECK(bl_attn_fwd_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), cu_q.data_ptr<int>(),
                            cu_k.data_ptr<int>(), batch, max_q, max_k, int(q.size(0)), int(k.size(0)), nq, nkv,
                            hd, int(q.stride(0)), int(k.stride(0)), int(v.stride(0)), nq * hd, float(scale),
                            causal ? 1 : 0, vt.data_ptr(), attn_err(q.device().index()).data_ptr(), st, err,
                            errlen));
    return out;
  }
  if (q.size(0) > 0)
    BL_CHECK(bl_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                         cu_q.data_ptr<int>(), cu_k.data_ptr<int>(), batch, max_q, nq, nkv, hd,
                         int(q.stride(0)), int(k.stride(0)), int(v.stride(0)), nq * hd, float(scale),
                         causal ? 1 : 0, st, err, errlen));
  return out;
}

void check_bf16x(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kBFloat16, "barlink: ", name,
              " must be a contiguous bfloat16 CUDA tensor");
}

struct W8Scratch {
  at::Tensor ws, counters, err_flag;
};
W8Scratch& w8_scratch(int dev) {
  static std::map<int, W8Scratch> m;
  auto it = m.find(dev);
  if (it != m.end()) return it->second;
  auto o = at::TensorOptions().device(at::kCUDA, dev);
  W8Scratch s;
  s.ws = at::empty({int64_t(64) << 20}, o.dtype(at::kByte));
  s.counters = at::zeros({16384}, o.dtype(at::kInt));
  s.err_flag = at::zeros({4}, o.dtype(at::kInt));
  return m.emplace(dev, s).first->second;
}

// y = x @ (wq * scale[:, None]).T (+ bias): bf16 activations, int8 per-channel
// weights widened to bf16 inside the tcgen05 main loop (<= 256 tokens); more
// tokens widen the weight once and use the bf16 GEMM.
// bf16 group scales [n, groups] -> (row_max bf16 [n], rel fp16 [n, groups]): done once per weight
std::tuple<at::Tensor, at::Tensor> w8_group_scales(const at::Tensor& scales) {
  check_bf16x(scales, "scales");
  TORCH_CHECK(scales.dim() == 2, "barlink: group scales must be [n, groups]");
  const int n = int(scales.size(0)), groups = int(scales.size(1));
  at::Tensor row = at::empty({n}, scales.options());
  at::Tensor rel = at::empty({n, groups}, scales.options().dtype(at::kHalf));
  c10::cuda::CUDAGuard guard(scales.device());
  void* st = at::cuda::getCurrentCUDAStream(scales.device().index()).stream();
  BL_CHECK(bl_w8_group_scales(scales.data_ptr(), n, groups, row.data_ptr(), rel.data_ptr(), st, err, errlen));
  return {row, rel};
}

at::Tensor w8a16_linear(const at::Tensor& x, const at::Tensor& wq, const at::Tensor& scale,
                        const c10::optional<at::Tensor>& bias, bool silu_mul, int splits,
                        const c10::optional<at::Tensor>& group_rel, bool act_int8,
                        const c10::optional<at::Tensor>& group_scale) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
              "barlink: x must be a 2-D bfloat16 CUDA tensor with unit inner stride");
  TORCH_CHECK(wq.is_cuda() && wq.is_contiguous() && wq.scalar_type() == at::kChar && wq.dim() == 2 &&
                  wq.size(1) == x.size(1),
              "barlink: wq must be a contiguous int8 [n, k] CUDA tensor with k = x.shape[1]");
  check_bf16x(scale, "scale");
  const int m = int(x.size(0)), k = int(x.size(1)), n = int(wq.size(0));
  TORCH_CHECK(group_scale || scale.numel() == n, "barlink: scale must have one entry per output channel");
  if (group_scale) {
    TORCH_CHECK(act_int8 && m <= 64, "barlink: group_scale goes with act_int8 and at most 64 tokens");
    TORCH_CHECK(group_scale->is_cuda() && group_scale->is_contiguous() && group_scale->scalar_type() == at::kBFloat16 &&
                    group_scale->dim() == 2 && group_scale->size(0) == n && k % group_scale->size(1) == 0 &&
                    (k / group_scale->size(1)) % 128 == 0,
                "barlink: group_scale must be contiguous bfloat16 [n, k / group] with a group size that is a multiple of 128");
  }
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  at::Tensor out = at::empty({m, silu_mul ? n / 2 : n}, x.options());
  if (m == 0) return out;
  if (group_rel) {
    TORCH_CHECK(group_rel->is_cuda() && group_rel->is_contiguous() && group_rel->scalar_type() == at::kHalf &&
                    group_rel->dim() == 2 && group_rel->size(0) == n && k % group_rel->size(1) == 0,
                "barlink: group_rel must be contiguous float16 [n, k / group] (see w8_group_scales)");
    TORCH_CHECK(m <= 256, "barlink: in-kernel group scales take at most 256 tokens");
  }
  if (act_int8) {
    // the reference's numerics (w8a16.cu:37-92 there quantises the activations per token and
    // multiplies int8 by int8): both operands go to the tensor cores as int8
    TORCH_CHECK(!group_rel, "barlink: int8 activations go with per-channel weight scales");
    TORCH_CHECK(k % 16 == 0, "barlink: int8 activations need K % 16 == 0");
    at::Tensor xc = x.is_contiguous() ? x : x.contiguous();
    at::Tensor xq = at::empty({m, k}, x.options().dtype(at::kChar));
    at::Tensor xs = at::empty({m}, x.options().dtype(at::kFloat));
    BL_CHECK(bl_w8a16_quant_act(xc.data_ptr(), m, k, xq.data_ptr(), xs.data_ptr(), st, err, errlen));
    W8Scratch& s = w8_scratch(dev);
    if (bias) {
      check_bf16x(*bias, "bias");
      TORCH_CHECK(bias->numel() == n, "barlink: bias must have n entries");
    }
    if (m <= 256) {
      blW8A16Args a;
      memset(&a, 0, sizeof(a));
      a.xq = xq.data_ptr();
      a.xs = xs.data_ptr();
      a.m = m;
      a.ldx = k;
      a.wq = wq.data_ptr();
      a.n = n;
      a.k = k;
      a.scale = scale.data_ptr();
      if (group_scale) {
        a.group_scale = group_scale->data_ptr();
        a.group_k = k / int(group_scale->size(1));
      }
      a.bias = bias ? bias->data_ptr() : nullptr;
      a.out = out.data_ptr();
      a.ldo = silu_mul ? n / 2 : n;
      a.silu_mul = silu_mul ? 1 : 0;
      a.splits = splits;
      a.ws = s.ws.data_ptr();
      a.ws_bytes = size_t(s.ws.nbytes());
      a.counters = s.counters.data_ptr();
      a.n_counters = int(s.counters.numel());
      a.err_flag = s.err_flag.data_ptr();
      py::gil_scoped_release nogil;
      BL_CHECK(bl_w8a16_linear(&a, st, err, errlen));
    } else {
      // prefill: token-major tiles
      blGemmArgs g;
      memset(&g, 0, sizeof(g));
      g.a = xq.data_ptr(); g.ra = m; g.lda = k;
      g.b = wq.data_ptr(); g.rb = n; g.ldb = k;
      g.k = k;
      g.out = out.data_ptr();
      g.ldo = silu_mul ? n / 2 : n;
      g.bias = bias ? bias->data_ptr() : nullptr;
      g.silu_mul = silu_mul ? 1 : 0;
      g.splits = 1;
      g.err_flag = s.err_flag.data_ptr();
      g.i8 = 1;
      g.feat_scale = scale.data_ptr();
      g.tok_scale = xs.data_ptr();
      py::gil_scoped_release nogil;
      BL_CHECK(bl_gemm_bf16(&g, st, err, errlen));
    }
    return out;
  }
  if (m > 256) {
    at::Tensor w = at::empty({n, k}, x.options());
    BL_CHECK(bl_w8_dequant(wq.data_ptr(), scale.data_ptr(), w.data_ptr(), n, k, st, err, errlen));
    py::object lin = py::module_::import("barlink_sm86_b200").attr("load_extension")().attr("linear");
    // `w` was written by the kernel just launched: the GEMM must not fetch weight tiles ahead of
    // that kernel's completion (its producer otherwise requests them before griddepcontrol.wait)
    using namespace pybind11::literals;
    return lin(x, w, bias ? py::cast(*bias) : py::none(), py::none(), silu_mul, "dynamic_weights"_a = true)
        .cast<at::Tensor>();
  }
  W8Scratch& s = w8_scratch(dev);
  blW8A16Args a;
  memset(&a, 0, sizeof(a));
  a.x = x.data_ptr();
  a.m = m;
  a.ldx = int(x.stride(0));
  a.wq = wq.data_ptr();
  a.n = n;
  a.k = k;
  a.scale = scale.data_ptr();
  if (group_rel) {
    a.group_rel = group_rel->data_ptr();
    a.group_k = k / int(group_rel->size(1));
  }
  if (bias) {
    check_bf16x(*bias, "bias");
    TORCH_CHECK(bias->numel() == n, "barlink: bias must have n entries");
    a.bias = bias->data_ptr();
  }
  a.out = out.data_ptr();
  a.ldo = silu_mul ? n / 2 : n;
  a.silu_mul = silu_mul ? 1 : 0;
  a.splits = splits;
  a.ws = s.ws.data_ptr();
  a.ws_bytes = size_t(s.ws.nbytes());
  a.counters = s.counters.data_ptr();
  a.n_counters = int(s.counters.numel());
  a.err_flag = s.err_flag.data_ptr();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_w8a16_linear(&a, st, err, errlen));
  }
  return out;
}

int w8_error_flag(int dev) { return w8_scratch(dev).err_flag.cpu()[0].item<int>(); }

// the reference's pair (binding.cpp:434-490 there)
std::vector<at::Tensor> w8a16_quant_act(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == at::kBFloat16,
              "barlink w8a16_quant_act: x must be a contiguous 2-D bfloat16 CUDA tensor");
  const int m = int(x.size(0)), k = int(x.size(1));
  TORCH_CHECK(k % 8 == 0, "barlink w8a16_quant_act: K % 8 must be 0");
  at::Tensor xq = at::empty({m, k}, x.options().dtype(at::kChar));
  at::Tensor xs = at::empty({m}, x.options().dtype(at::kFloat));
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(x.device().index()).stream();
  if (m > 0) BL_CHECK(bl_w8a16_quant_act(x.data_ptr(), m, k, xq.data_ptr(), xs.data_ptr(), st, err, errlen));
  return {xq, xs};
}

at::Tensor w8a16_gemm(const at::Tensor& xq, const at::Tensor& xs, const at::Tensor& wq_t,
                      const at::Tensor& sw_t, int64_t N, int64_t K, int64_t S) {
  TORCH_CHECK(xq.is_cuda() && xq.is_contiguous() && xq.dim() == 2 && xq.scalar_type() == at::kChar,
              "barlink w8a16_gemm: xq must be contiguous int8 [M, K]");
  const int m = int(xq.size(0));
  TORCH_CHECK(xq.size(1) == K && K % 128 == 0, "barlink w8a16_gemm: K must match xq and be a multiple of 128");
  TORCH_CHECK(wq_t.is_contiguous() && wq_t.scalar_type() == at::kChar && wq_t.numel() == N * K &&
                  sw_t.is_contiguous() && sw_t.scalar_type() == at::kFloat && sw_t.numel() == (K / 128) * N,
              "barlink w8a16_gemm: wq_t int8 [K/16, N, 16] and sw_t float32 [K/128, N], contiguous");
  TORCH_CHECK(xs.is_contiguous() && xs.scalar_type() == at::kFloat && xs.numel() == m,
              "barlink w8a16_gemm: xs must be float32 [M]");
  TORCH_CHECK(m <= 16, "barlink w8a16_gemm: M > 16 is not supported by this decode kernel (use w8a16_linear)");
  at::Tensor out = at::empty({m, N}, xq.options().dtype(at::kBFloat16));
  at::Tensor ws;
  void* wsp = nullptr;
  if (S > 1) {
    ws = at::empty({S, m, N}, xq.options().dtype(at::kFloat));
    wsp = ws.data_ptr();
  }
  c10::cuda::CUDAGuard guard(xq.device());
  void* st = at::cuda::getCurrentCUDAStream(xq.device().index()).stream();
  if (m > 0)
    BL_CHECK(bl_w8a16_gemm(xq.data_ptr(), xs.data_ptr(), wq_t.data_ptr(), sw_t.data_ptr(), out.data_ptr(),
                           m, int(N), int(K), int(S), wsp, st, err, errlen));
  return out;
}

// GPTQ-v1 int4 linear: 1..16 rows use the GEMV; more rows widen the weight and use the bf16 GEMM
at::Tensor w4a16_linear(const at::Tensor& x, const at::Tensor& qweight, const at::Tensor& scales,
                        const at::Tensor& qzeros, int group, int splits) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(),
              "barlink: x must be a contiguous 2-D bfloat16 CUDA tensor");
  TORCH_CHECK(qweight.is_cuda() && qweight.is_contiguous() && qweight.scalar_type() == at::kInt &&
                  qweight.dim() == 2 && qweight.size(0) * 8 == x.size(1),
              "barlink: qweight must be a contiguous int32 [K/8, N] CUDA tensor with K = x.shape[1]");
  const int m = int(x.size(0)), k = int(x.size(1)), n = int(qweight.size(1));
  TORCH_CHECK(group > 0 && k % group == 0, "barlink: K must be a multiple of the group size");
  TORCH_CHECK(scales.is_cuda() && scales.is_contiguous() && scales.scalar_type() == at::kHalf &&
                  scales.dim() == 2 && scales.size(0) == k / group && scales.size(1) == n,
              "barlink: scales must be a contiguous float16 [K/group, N] CUDA tensor");
  TORCH_CHECK(qzeros.is_cuda() && qzeros.is_contiguous() && qzeros.scalar_type() == at::kInt &&
                  qzeros.dim() == 2 && qzeros.size(0) == k / group && qzeros.size(1) * 8 == n,
              "barlink: qzeros must be a contiguous int32 [K/group, N/8] CUDA tensor");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  if (m == 0) return at::empty({0, n}, x.options());
  if (m > 16) {
    at::Tensor w = at::empty({n, k}, x.options());
    BL_CHECK(bl_w4_dequant(qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), w.data_ptr(), n, k, group,
                           st, err, errlen));
    return at::matmul(x, w.t());  // prefill path, not the decode hot path
  }
  W8Scratch& s = w8_scratch(dev);
  at::Tensor out = at::empty({m, n}, x.options());
  BL_CHECK(bl_w4a16_gemv(x.data_ptr(), qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), out.data_ptr(),
                         m, n, k, group, splits, s.ws.data_ptr(), size_t(s.ws.nbytes()), st, err, errlen));
  return out;
}

at::Tensor w4_dequant(const at::Tensor& qweight, const at::Tensor& scales, const at::Tensor& qzeros, int group) {
  TORCH_CHECK(qweight.is_cuda() && qweight.is_contiguous() && qweight.scalar_type() == at::kInt &&
                  scales.is_cuda() && scales.is_contiguous() && scales.scalar_type() == at::kHalf &&
                  qzeros.is_cuda() && qzeros.is_contiguous() && qzeros.scalar_type() == at::kInt,
              "barlink: w4_dequant needs contiguous CUDA qweight (int32), scales (float16), qzeros (int32)");
  const int k = int(qweight.size(0)) * 8, n = int(qweight.size(1));
  c10::cuda::CUDAGuard guard(qweight.device());
  at::Tensor w = at::empty({n, k}, scales.options().dtype(at::kBFloat16));
  BL_CHECK(bl_w4_dequant(qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), w.data_ptr(), n, k, group,
                         at::cuda::getCurrentCUDAStream(qweight.device().index()).stream(), err, errlen));
  return w;
}

void qknorm_rope(const at::Tensor& qkv, const c10::optional<at::Tensor>& gq,
                 const c10::optional<at::Tensor>& gk, const at::Tensor& positions, int heads, double eps,
                 double theta, int axes) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1 &&
                  qkv.size(1) >= int64_t(2 * heads) * 128,
              "barlink: qknorm_rope needs a 2-D bfloat16 CUDA tensor whose rows start with the q and k heads");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.is_contiguous() &&
                  positions.numel() == qkv.size(0) * axes,
              "barlink: positions must be int32 [rows, axes]");
  if (gq) check_bf16x(*gq, "gq");
  if (gk) check_bf16x(*gk, "gk");
  c10::cuda::CUDAGuard guard(qkv.device());
  void* st = at::cuda::getCurrentCUDAStream(qkv.device().index()).stream();
  if (qkv.size(0) > 0)
    BL_CHECK(bl_qknorm_rope(qkv.data_ptr(), gq ? gq->data_ptr() : nullptr, gk ? gk->data_ptr() : nullptr,
                            positions.data_ptr<int>(), int(qkv.size(0)), heads, 128, int(qkv.stride(0)),
                            float(eps), float(theta), axes, st, err, errlen));
}

at::Tensor layernorm_modulate(const at::Tensor& x, const at::Tensor& shift, const at::Tensor& scale,
                              int rows_per_batch, double eps) {
  check_bf16x(x, "x");
  TORCH_CHECK(shift.is_cuda() && scale.is_cuda() && shift.scalar_type() == at::kBFloat16 &&
                  scale.scalar_type() == at::kBFloat16 && shift.dim() == 2 && scale.dim() == 2 &&
                  shift.stride(1) == 1 && scale.stride(1) == 1 && shift.stride(0) == scale.stride(0),
              "barlink: shift/scale must be bfloat16 [batch, hidden] views with the same pitch");
  const int hidden = int(x.size(-1));
  const int rows = int(x.numel() / hidden);
  at::Tensor out = at::empty_like(x);
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(x.device().index()).stream();
  if (rows > 0)
    BL_CHECK(bl_layernorm_modulate(x.data_ptr(), shift.data_ptr(), scale.data_ptr(), out.data_ptr(), rows,
                                   hidden, rows_per_batch, int(shift.stride(0)), float(eps), st, err, errlen));
  return out;
}

void gate_residual(const at::Tensor& x, const at::Tensor& y, const at::Tensor& gate, int rows_per_batch) {
  check_bf16x(x, "x");
  check_bf16x(y, "y");
  TORCH_CHECK(gate.is_cuda() && gate.scalar_type() == at::kBFloat16 && gate.dim() == 2 && gate.stride(1) == 1 &&
                  x.sizes() == y.sizes(),
              "barlink: gate must be a bfloat16 [batch, hidden] view and y must match x");
  const int hidden = int(x.size(-1));
  const int rows = int(x.numel() / hidden);
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(x.device().index()).stream();
  if (rows > 0)
    BL_CHECK(bl_gate_residual(x.data_ptr(), y.data_ptr(), gate.data_ptr(), rows, hidden, rows_per_batch,
                              int(gate.stride(0)), st, err, errlen));
}

// ---- host-only internals, exposed so that they can be unit-tested without a GPU ----

// ---- decode linears with the collective folded in (dlin_kernels.cu) ----------------------
struct DlinScratch {
  at::Tensor sync, err_flag;
};
DlinScratch& dlin_scratch(int dev) {
  static std::map<int, DlinScratch> m;
  auto it = m.find(dev);
  if (it != m.end()) return it->second;
  auto o = at::TensorOptions().device(at::kCUDA, dev).dtype(at::kInt);
  DlinScratch s;
  s.sync = at::zeros({16 + 64 * 8}, o);  // counters, then the segment sums of the gather prologue
  s.err_flag = at::zeros({4}, o);
  return m.emplace(dev, s).first->second;
}
int dlin_error_flag(int dev) { return dlin_scratch(dev).err_flag.cpu()[0].item<int>(); }

// a one-rank stand-in for the link in ordinary device memory (single-GPU runs of the same kernels)
at::Tensor dlin_local_link(int tokens, int hidden, int dev) {
  c10::cuda::CUDAGuard guard(c10::Device(at::kCUDA, dev));
  at::Tensor buf = at::empty({int64_t(bl_dlin_local_link_bytes(tokens, hidden))},
                             at::TensorOptions().device(at::kCUDA, dev).dtype(at::kByte));
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  BL_CHECK(bl_dlin_local_link_init(buf.data_ptr(), tokens, hidden, st, err, errlen));
  return buf;
}

void dlin_fill_common(blDlinArgs& a, const at::Tensor& x, int hidden, const c10::optional<at::Tensor>& link,
                      int dev) {
  a.x = x.data_ptr();
  a.tokens = int(x.size(0));
  a.ldx = int(x.stride(0));
  a.hidden = hidden;
  if (link) {
    TORCH_CHECK(link->is_cuda() && link->is_contiguous() &&
                    size_t(link->nbytes()) >= bl_dlin_local_link_bytes(a.tokens, hidden),
                "barlink: the local link buffer is too small for ", a.tokens, " x ", hidden);
    a.local_link = link->data_ptr();
  }
  a.err_flag = dlin_scratch(dev).err_flag.data_ptr();
}

// pro: "none" | "gather_norm";  epi: "store" | "silu_mul" | "push"
// gather_norm: x is written first (RMSNorm(residual + all-reduced rows) * gamma), residual is
// updated in place.  push: returns nothing useful (the rows are in every rank's inbox).
at::Tensor dlin(const at::Tensor& x, const at::Tensor& w, const std::string& pro, const std::string& epi,
                const c10::optional<at::Tensor>& out_opt, const c10::optional<at::Tensor>& bias,
                const c10::optional<at::Tensor>& residual, const c10::optional<at::Tensor>& gamma, double eps,
                int hidden, const c10::optional<at::Tensor>& link, int cluster, bool first,
                const c10::optional<at::Tensor>& trace) {
  check_bf16x(w, "weight");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 &&
                  w.dim() == 2 && w.stride(1) == 1 && w.size(1) == x.size(1),
              "barlink: dlin needs bf16 x [tokens, k] and w [n, k] with unit inner strides");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  blDlinArgs a;
  memset(&a, 0, sizeof(a));
  a.w = w.data_ptr();
  a.n = int(w.size(0));
  a.k = int(w.size(1));
  a.ldw = int(w.stride(0));
  a.pro = pro == "gather_norm" ? 1 : 0;
  TORCH_CHECK(a.pro == 1 || pro == "none", "barlink: dlin prologue must be none or gather_norm");
  a.epi = epi == "store" ? 0 : epi == "silu_mul" ? 1 : epi == "push" ? 2 : -1;
  TORCH_CHECK(a.epi >= 0, "barlink: dlin epilogue must be store, silu_mul or push");
  dlin_fill_common(a, x, hidden > 0 ? hidden : a.k, link, dev);
  if (a.pro == 1) {
    TORCH_CHECK(residual && gamma, "barlink: gather_norm needs residual and gamma");
    check_bf16x(*residual, "residual");
    check_bf16x(*gamma, "gamma");
    TORCH_CHECK(residual->numel() == x.numel() && x.is_contiguous() && gamma->numel() == a.k,
                "barlink: residual must match x, gamma must have k entries");
    a.residual_in = first ? nullptr : residual->data_ptr();
    a.residual_out = residual->data_ptr();
    a.gamma = gamma->data_ptr();
    a.eps = float(eps);
    a.sync = dlin_scratch(dev).sync.data_ptr();
  }
  at::Tensor out;
  if (a.epi != 2) {
    const int64_t cols = a.epi == 1 ? a.n / 2 : a.n;
    out = out_opt ? *out_opt : at::empty({x.size(0), cols}, x.options());
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == x.size(0) &&
                    out.size(1) == cols && out.stride(1) == 1,
                "barlink: dlin out must be bf16 [tokens, ", cols, "]");
    a.out = out.data_ptr();
    a.ldo = int(out.stride(0));
    if (bias) {
      check_bf16x(*bias, "bias");
      TORCH_CHECK(bias->numel() == a.n, "barlink: bias must have n entries");
      a.bias = bias->data_ptr();
    }
  }
  a.cluster = cluster;
  if (trace) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() &&
                    trace->numel() >= 12 * 8 * ((a.n + 127) / 128),
                "barlink: trace must be a contiguous int64 CUDA tensor of 12 words per CTA");
    a.trace = trace->data_ptr();
  }
  blCtx* c = link ? nullptr : blpg::global_ctx();
  {
    py::gil_scoped_release nogil;
    BL_CHECK(bl_dlin(c, &a, st, err, errlen));
  }
  return a.epi == 2 ? x : out;
}

// x = RMSNorm(residual + all-reduced inbox rows) * gamma, residual updated in place
void gather_norm(const at::Tensor& x, const at::Tensor& residual, const at::Tensor& gamma, double eps,
                 const c10::optional<at::Tensor>& link, bool first) {
  check_bf16x(residual, "residual");
  check_bf16x(gamma, "gamma");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous() &&
                  residual.numel() == x.numel() && gamma.numel() == x.size(1),
              "barlink: gather_norm needs contiguous bf16 x [tokens, hidden], residual of that shape, gamma [hidden]");
  const int dev = x.device().index();
  c10::cuda::CUDAGuard guard(x.device());
  void* st = at::cuda::getCurrentCUDAStream(dev).stream();
  blDlinArgs a;
  memset(&a, 0, sizeof(a));
  dlin_fill_common(a, x, int(x.size(1)), link, dev);
  a.residual_in = first ? nullptr : residual.data_ptr();
  a.residual_out = residual.data_ptr();
  a.gamma = gamma.data_ptr();
  a.eps = float(eps);
  blCtx* c = link ? nullptr : blpg::global_ctx();
  py::gil_scoped_release nogil;
  BL_CHECK(bl_gather_norm(c, &a, st, err, errlen));
}

py::dict layout_of(size_t pool_bytes, int world) {
  const bl::Layout L = bl::compute_layout(pool_bytes, world);
  py::dict d;
  d["pool_bytes"] = L.pool_bytes;
  d["user_bytes"] = L.user_bytes;
  d["stage_off"] = L.stage_off;
  d["stage_slice"] = L.stage_slice;
  d["lamport_off"] = L.lamport_off;
  d["lamport_slice"] = L.lamport_slice;
  d["p2p_off"] = L.p2p_off;
  d["p2p_slice"] = L.p2p_slice;
  d["sig_off"] = L.sig_off;
  return d;
}

// ops: ("alloc", bytes) -> offset or -1; ("free", offset, bytes) -> 1 / 0
std::vector<int64_t> arena_replay(size_t user_bytes, const std::vector<py::tuple>& ops) {
  bl::Arena a;
  std::vector<int64_t> out;
  for (const auto& op : ops) {
    const std::string kind = op[0].cast<std::string>();
    if (kind == "alloc") out.push_back(bl::arena_alloc(a, user_bytes, op[1].cast<size_t>()));
    else out.push_back(bl::arena_free(a, op[1].cast<size_t>(), op[2].cast<size_t>()) ? 1 : 0);
  }
  return out;
}

}  // namespace

void bind_extra(py::module_& m) {
  m.def("layout_of", &layout_of, py::arg("pool_bytes"), py::arg("world"));
  m.def("arena_replay", &arena_replay, py::arg("user_bytes"), py::arg("ops"));
  m.def("algo_for", [](size_t bytes, int world, const std::string& dtype, bool multicast, size_t pool_bytes,
                       const std::string& algo) {
    const int dt = dtype == "bf16" ? BL_DTYPE_BF16 : dtype == "fp16" ? BL_DTYPE_FP16 : dtype == "fp32" ? BL_DTYPE_FP32
                 : dtype == "fp64" ? BL_DTYPE_FP64 : BL_DTYPE_U8;
    const int al = algo == "oneshot" ? BL_ALGO_ONESHOT : algo == "twoshot" ? BL_ALGO_TWOSHOT
                 : algo == "nvls" ? BL_ALGO_NVLS : BL_ALGO_AUTO;
    static const char* names[] = {"auto", "oneshot", "twoshot", "nvls"};
    return std::string(names[bl_algo_for(bytes, world, dt, multicast ? 1 : 0, pool_bytes, al)]);
  }, py::arg("bytes"), py::arg("world"), py::arg("dtype") = "bf16", py::arg("multicast") = false,
        py::arg("pool_bytes") = size_t(1) << 30, py::arg("algo") = "auto");
  m.def("pick_splits", [](int tiles, int kblocks, int sms, int want) { return bl::pick_splits(tiles, kblocks, sms, want); },
        py::arg("tiles"), py::arg("kblocks"), py::arg("sms") = 148, py::arg("want") = 0);
  m.def("w4a16_linear", &w4a16_linear, py::arg("x"), py::arg("qweight"), py::arg("scales"), py::arg("qzeros"),
        py::arg("group") = 128, py::arg("splits") = 0);
  m.def("w4_dequant", &w4_dequant, py::arg("qweight"), py::arg("scales"), py::arg("qzeros"), py::arg("group") = 128);
  m.def("qknorm_rope", &qknorm_rope, py::arg("qkv"), py::arg("gq"), py::arg("gk"), py::arg("positions"),
        py::arg("heads"), py::arg("eps") = 1e-6, py::arg("theta") = 1e4, py::arg("axes") = 2);
  m.def("layernorm_modulate", &layernorm_modulate, py::arg("x"), py::arg("shift"), py::arg("scale"),
        py::arg("rows_per_batch"), py::arg("eps") = 1e-6);
  m.def("gate_residual", &gate_residual, py::arg("x"), py::arg("y"), py::arg("gate"),
        py::arg("rows_per_batch"));
  m.def("w8a16_linear", &w8a16_linear, py::arg("x"), py::arg("wq"), py::arg("scale"),
        py::arg("bias") = py::none(), py::arg("silu_mul") = false, py::arg("splits") = 0,
        py::arg("group_rel") = py::none(), py::arg("act_int8") = false, py::arg("group_scale") = py::none());
  m.def("w8_group_scales", &w8_group_scales, py::arg("scales"));
  m.def("w8_error_flag", &w8_error_flag, py::arg("device") = 0);
  m.def("dlin", &dlin, py::arg("x"), py::arg("weight"), py::arg("pro") = "none", py::arg("epi") = "store",
        py::arg("out") = py::none(), py::arg("bias") = py::none(), py::arg("residual") = py::none(),
        py::arg("gamma") = py::none(), py::arg("eps") = 1e-6, py::arg("hidden") = 0, py::arg("link") = py::none(),
        py::arg("cluster") = 0, py::arg("first") = false, py::arg("trace") = py::none());
  m.def("gather_norm", &gather_norm, py::arg("x"), py::arg("residual"), py::arg("gamma"), py::arg("eps") = 1e-6,
        py::arg("link") = py::none(), py::arg("first") = false);
  m.def("dlin_local_link", &dlin_local_link, py::arg("tokens"), py::arg("hidden"), py::arg("device") = 0);
  m.def("dlin_error_flag", &dlin_error_flag, py::arg("device") = 0);
  m.def("dlin_cluster", [](int n, int k, int tokens, int want) { return bl_dlin_cluster(n, k, tokens, want); },
        py::arg("n"), py::arg("k"), py::arg("tokens") = 64, py::arg("want") = 0);
  m.def("w8a16_quant_act", &w8a16_quant_act);
  m.def("w8a16_gemm", &w8a16_gemm, py::arg("xq"), py::arg("xs"), py::arg("wq_t"), py::arg("sw_t"),
        py::arg("N"), py::arg("K"), py::arg("S"));
  m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("cu_q"),
        py::arg("cu_k"), py::arg("max_q"), py::arg("scale"), py::arg("causal"), py::arg("max_k") = 0);
  m.def("attn_error_flag", &attn_error_flag, py::arg("device") = 0);
  m.def("sp_collective", &sp_collective, py::arg("kind"), py::arg("ins") = std::vector<at::Tensor>{},
        py::arg("outs") = std::vector<at::Tensor>{}, py::arg("aux_in") = std::vector<at::Tensor>{},
        py::arg("aux_out") = std::vector<at::Tensor>{}, py::arg("gamma") = std::vector<at::Tensor>{},
        py::arg("algo") = "auto", py::arg("root") = 0, py::arg("eps") = 1e-6);
  m.def("sp_sendrecv", &sp_sendrecv, py::arg("src"), py::arg("dst"), py::arg("inp"), py::arg("out"));
}
