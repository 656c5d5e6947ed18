// Bindings of the mixture-of-experts routing / exchange kernels (moe.cu).  Exchange buffers are passed as one device
// address per rank (from torch.distributed._symmetric_memory handles; a single local address when world == 1).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "kernels.h"

int* package_status_ptr(const c10::Device& dev);  // gemm_bindings.cpp

namespace {

using torch::Tensor;

void check(const Tensor& t, at::ScalarType ty, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == ty, name, ": contiguous CUDA tensor of the expected dtype required");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must start on a 16-byte boundary");
}

int fill(const std::vector<int64_t>& in, void** out) {
  const int world = (int)in.size();
  TORCH_CHECK(world >= 1 && world <= seg::kMaxRanks, "need one buffer address per rank (at most ", seg::kMaxRanks, ")");
  for (int i = 0; i < world; ++i) {
    TORCH_CHECK((in[i] & 15) == 0, "exchange buffers must be 16-byte aligned");
    out[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(in[i]));
  }
  return world;
}

// -> probs [T,E] f32, idx [T,k] i32, w [T,k] f32, block_off [nblk,E] i32, totals [E] i32
std::vector<Tensor> moe_route(const Tensor& x, const Tensor& wr, int64_t k) {
  check(x, at::kBFloat16, "x");
  check(wr, at::kFloat, "router weight");
  TORCH_CHECK(x.dim() == 2 && wr.dim() == 2 && wr.size(1) == x.size(1), "x [T,d], router weight [E,d]");
  const int T = (int)x.size(0), d = (int)x.size(1), E = (int)wr.size(0);
  c10::cuda::CUDAGuard guard(x.device());
  const int nblk = (T + seg::kMoeTokensPerBlock - 1) / seg::kMoeTokensPerBlock;
  auto f32 = x.options().dtype(at::kFloat), i32 = x.options().dtype(at::kInt);
  Tensor probs = at::empty({T, E}, f32), idx = at::empty({T, k}, i32), w = at::empty({T, k}, f32);
  Tensor counts = at::empty({nblk, E}, i32), off = at::empty({nblk, E}, i32), totals = at::empty({E}, i32);
  const int rc = seg::moe_route(x.data_ptr(), wr.data_ptr<float>(), T, d, E, (int)k, probs.data_ptr<float>(), idx.data_ptr<int>(),
                                w.data_ptr<float>(), counts.data_ptr<int>(), off.data_ptr<int>(), totals.data_ptr<int>(),
                                at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "moe_route: need E <= ", seg::kMoeMaxExperts, ", k <= min(", seg::kMoeMaxTopK, ", E), d % 8 == 0");
  return {probs, idx, w, off, totals};
}

Tensor moe_slots(const Tensor& idx, const Tensor& block_off, int64_t cap) {
  check(idx, at::kInt, "idx");
  check(block_off, at::kInt, "block_off");
  const int T = (int)idx.size(0), k = (int)idx.size(1), E = (int)block_off.size(1);
  TORCH_CHECK(k <= seg::kMoeMaxTopK, "k too large");
  c10::cuda::CUDAGuard guard(idx.device());
  Tensor slot = at::empty_like(idx);
  seg::moe_slots(idx.data_ptr<int>(), block_off.data_ptr<int>(), T, E, k, (int)cap, slot.data_ptr<int>(),
                 at::cuda::getCurrentCUDAStream().stream());
  return slot;
}

// flag_ptrs (one per rank, or empty) + done_counter (zeroed uint32/int32 CUDA scalar) + seq: completion signal for the
// consumer's per-region waits.
void moe_push(const Tensor& x, const Tensor& idx, const Tensor& slot, const std::optional<Tensor>& w, const Tensor& totals,
              std::vector<int64_t> dst, int64_t cap, int64_t rank, std::vector<int64_t> flag_ptrs,
              const std::optional<Tensor>& done_counter, int64_t seq) {
  check(x, at::kBFloat16, "x");
  check(idx, at::kInt, "idx");
  check(slot, at::kInt, "slot");
  check(totals, at::kInt, "totals");
  if (w.has_value()) check(*w, at::kFloat, "w");
  void* bufs[seg::kMaxRanks];
  const int world = fill(dst, bufs);
  const int T = (int)x.size(0), d = (int)x.size(1), k = (int)idx.size(1), E = (int)totals.size(0);
  TORCH_CHECK(d % 8 == 0 && E % world == 0 && idx.size(0) == T && slot.sizes() == idx.sizes(), "moe_push: shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  void* flags[seg::kMaxRanks];
  const bool signal = !flag_ptrs.empty();
  if (signal) {
    TORCH_CHECK((int)flag_ptrs.size() == world && done_counter.has_value(), "moe_push: flags need one array per rank and a counter");
    check(*done_counter, at::kInt, "done_counter");
    for (int i = 0; i < world; ++i) flags[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(flag_ptrs[i]));
  }
  seg::moe_push(x.data_ptr(), idx.data_ptr<int>(), slot.data_ptr<int>(), w.has_value() ? w->data_ptr<float>() : nullptr,
                totals.data_ptr<int>(), bufs, T, d, E, k, (int)cap, world, (int)rank, at::cuda::getCurrentCUDAStream().stream(),
                signal ? reinterpret_cast<uint32_t* const*>(flags) : nullptr,
                signal ? reinterpret_cast<uint32_t*>(done_counter->data_ptr<int>()) : nullptr, (uint32_t)seq, package_status_ptr(x.device()));
}

// returns (out [T,d], dots [T,k] or empty)
std::vector<Tensor> moe_pull(std::vector<int64_t> src, std::vector<int64_t> src2, const Tensor& idx, const Tensor& slot,
                             const std::optional<Tensor>& w, const std::optional<Tensor>& g, int64_t d, int64_t n_experts,
                             int64_t cap, int64_t rank, bool out_f32) {
  check(idx, at::kInt, "idx");
  check(slot, at::kInt, "slot");
  if (w.has_value()) check(*w, at::kFloat, "w");
  void* a[seg::kMaxRanks];
  void* b[seg::kMaxRanks];
  const int world = fill(src, a);
  const bool want_dots = !src2.empty();
  if (want_dots) {
    TORCH_CHECK((int)src2.size() == world && g.has_value(), "moe_pull: dots need a second buffer per rank and g");
    fill(src2, b);
    check(*g, at::kBFloat16, "g");
  }
  const int T = (int)idx.size(0), k = (int)idx.size(1);
  TORCH_CHECK(d % 8 == 0 && n_experts % world == 0, "moe_pull: shape mismatch");
  c10::cuda::CUDAGuard guard(idx.device());
  Tensor out = at::empty({T, d}, idx.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  Tensor dots = want_dots ? at::empty({T, k}, idx.options().dtype(at::kFloat)) : Tensor();
  seg::moe_pull(a, want_dots ? b : nullptr, idx.data_ptr<int>(), slot.data_ptr<int>(), w.has_value() ? w->data_ptr<float>() : nullptr,
                want_dots ? g->data_ptr() : nullptr, out.data_ptr(), out_f32, want_dots ? dots.data_ptr<float>() : nullptr, T, (int)d,
                (int)n_experts, k, (int)cap, world, (int)rank, at::cuda::getCurrentCUDAStream().stream());
  if (want_dots) return {out, dots};
  return {out};
}

Tensor moe_route_bwd(const Tensor& probs, const Tensor& idx, const Tensor& dw, const Tensor& aux_vec) {
  check(probs, at::kFloat, "probs");
  check(idx, at::kInt, "idx");
  check(dw, at::kFloat, "dw");
  check(aux_vec, at::kFloat, "aux_vec");
  const int T = (int)probs.size(0), E = (int)probs.size(1), k = (int)idx.size(1);
  TORCH_CHECK(E <= seg::kMoeMaxExperts && k <= seg::kMoeMaxTopK && aux_vec.numel() == E && dw.sizes() == idx.sizes(), "moe_route_bwd: shapes");
  c10::cuda::CUDAGuard guard(probs.device());
  Tensor dlogits = at::empty_like(probs);
  seg::moe_route_bwd(probs.data_ptr<float>(), idx.data_ptr<int>(), dw.data_ptr<float>(), aux_vec.data_ptr<float>(), T, E, k,
                     dlogits.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream());
  return dlogits;
}

}  // namespace

void register_moe(pybind11::module_& m) {
  m.def("moe_route", &moe_route);
  m.def("moe_slots", &moe_slots);
  m.def("moe_push", &moe_push, pybind11::arg("x"), pybind11::arg("idx"), pybind11::arg("slot"), pybind11::arg("w"),
        pybind11::arg("totals"), pybind11::arg("dst"), pybind11::arg("cap"), pybind11::arg("rank"),
        pybind11::arg("flag_ptrs") = std::vector<int64_t>{}, pybind11::arg("done_counter") = std::nullopt, pybind11::arg("seq") = 0);
  m.def("moe_pull", &moe_pull);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.attr("MOE_MAX_EXPERTS") = seg::kMoeMaxExperts;
  m.attr("MOE_MAX_TOPK") = seg::kMoeMaxTopK;
}
