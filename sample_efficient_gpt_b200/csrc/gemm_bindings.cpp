// Bindings of the tcgen05 GEMM (gemm.cu).  Operands may be 2-D or batched 3-D bf16 tensors whose last dimension is
// contiguous; the bindings derive leading dimensions and batch strides and check the 16-byte alignment TMA needs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <optional>
#include <vector>

#include "kernels.h"

namespace {

using torch::Tensor;

struct PairWorkspace {
  Tensor slots, flags;  // parts of tiles cut along the contraction and their ready flags; launches on one stream share them
};

struct DeviceState {
  Tensor status;  // int32[1], stays 0 unless a bounded wait gave up
  int sm_count = 0;
  std::map<cudaStream_t, PairWorkspace> workspaces;
};

PairWorkspace& pair_workspace(DeviceState& st, const c10::Device& dev, cudaStream_t stream) {
  auto it = st.workspaces.find(stream);
  if (it == st.workspaces.end()) {
    PairWorkspace w;
    w.slots = torch::empty({(int64_t)seg::gemm_pair_workspace_bytes()}, torch::dtype(torch::kUInt8).device(dev));
    w.flags = torch::zeros({(int64_t)seg::gemm_pair_flag_words()}, torch::dtype(torch::kInt32).device(dev));
    it = st.workspaces.emplace(stream, std::move(w)).first;
  }
  return it->second;
}

DeviceState& device_state(const c10::Device& dev) {
  static std::map<int, DeviceState> states;
  auto it = states.find(dev.index());
  if (it == states.end()) {
    DeviceState st;
    st.status = torch::zeros({1}, torch::dtype(torch::kInt32).device(dev));
    st.sm_count = at::cuda::getDeviceProperties(dev.index())->multiProcessorCount;
    it = states.emplace(dev.index(), std::move(st)).first;
  }
  return it->second;
}

}  // namespace

// The per-device status word of the GEMM / attention kernels, for other binding files whose kernels report into it
// (index checks of the debug build).
int* package_status_ptr(const c10::Device& dev) { return device_state(dev).status.data_ptr<int>(); }

namespace {

void check_operand(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 2 || t.dim() == 3, name, " must be 2-D or 3-D");
  TORCH_CHECK(t.stride(-1) == 1, name, ": last dimension must be contiguous");
  TORCH_CHECK(t.stride(-2) % 8 == 0, name, ": row stride must be a multiple of 8 elements (16 bytes)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, ": base must be 16-byte aligned");
  if (t.dim() == 3) TORCH_CHECK(t.stride(0) % 8 == 0, name, ": batch stride must be a multiple of 8 elements");
}

// D = alpha * A op(B) + beta * C
Tensor gemm(const Tensor& a, const Tensor& b, const std::optional<Tensor>& c, std::optional<Tensor> out, bool out_f32, bool a_mn,
            bool b_mn, double alpha, double beta, bool symmetric, std::vector<int64_t> extra_dst,
            const std::optional<Tensor>& wait_flags, int64_t wait_seq, int64_t region_rows, std::vector<int64_t> route_ptrs,
            int64_t route_rows, int64_t route_batch_stride, int64_t route_base, int64_t route_ld, int64_t impl, bool split_k,
            int64_t wait_limit) {
  check_operand(a, "a");
  check_operand(b, "b");
  TORCH_CHECK(a.dim() == b.dim(), "a and b must have the same rank");
  const int batch = a.dim() == 3 ? (int)a.size(0) : 1;
  if (a.dim() == 3) TORCH_CHECK(b.size(0) == batch, "batch mismatch");
  const int M = (int)(a_mn ? a.size(-1) : a.size(-2));
  const int K = (int)(a_mn ? a.size(-2) : a.size(-1));
  const int N = (int)(b_mn ? b.size(-1) : b.size(-2));
  const int Kb = (int)(b_mn ? b.size(-2) : b.size(-1));
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  if (symmetric) TORCH_CHECK(M == N, "symmetric output must be square");
  c10::cuda::CUDAGuard guard(a.device());
  auto opts = a.options().dtype(out_f32 ? at::kFloat : at::kBFloat16);
  Tensor d;
  const bool routed = !route_ptrs.empty();
  if (routed) {
    TORCH_CHECK(!out.has_value() && !c.has_value() && route_ld > 0, "routed output: no out / c tensors, and the destination row stride is required");
    d = torch::empty({0}, opts);  // nothing is stored locally
  } else if (out.has_value()) {
    d = *out;
    TORCH_CHECK(d.is_cuda() && d.scalar_type() == (out_f32 ? at::kFloat : at::kBFloat16), "out has the wrong dtype");
    TORCH_CHECK(d.stride(-1) == 1 && d.size(-2) == M && d.size(-1) == N, "out has the wrong shape");
  } else {
    d = a.dim() == 3 ? torch::empty({batch, M, N}, opts) : torch::empty({M, N}, opts);
  }
  const void* cptr = nullptr;
  if (c.has_value()) {
    TORCH_CHECK(c->scalar_type() == d.scalar_type() && c->sizes() == d.sizes() && c->strides() == d.strides(),
                "c must match the output's dtype, shape and strides");
    cptr = c->data_ptr();
  }
  auto& st = device_state(a.device());
  const int64_t bsa = a.dim() == 3 ? a.stride(0) : 0, bsb = b.dim() == 3 ? b.stride(0) : 0, bsd = (!routed && d.dim() == 3) ? d.stride(0) : 0;
  void* routes[8] = {nullptr};
  TORCH_CHECK(route_ptrs.size() <= 8, "at most 8 routed destinations");
  for (size_t i = 0; i < route_ptrs.size(); ++i) routes[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(route_ptrs[i]));
  TORCH_CHECK(extra_dst.size() <= 7, "at most 7 extra destinations");
  const uint32_t* wf = nullptr;
  if (wait_flags.has_value()) {
    TORCH_CHECK(wait_flags->is_cuda() && wait_flags->scalar_type() == at::kInt && wait_flags->is_contiguous() && !a_mn && region_rows > 0,
                "wait_flags: contiguous CUDA int32 tensor, row-major A and region_rows > 0 required");
    TORCH_CHECK(wait_flags->numel() * region_rows >= M, "wait_flags: one flag per region of rows");
    wf = reinterpret_cast<const uint32_t*>(wait_flags->data_ptr<int>());
  }
  void* extras[7] = {nullptr};
  for (size_t i = 0; i < extra_dst.size(); ++i) extras[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(extra_dst[i]));
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  void* ws = nullptr;
  uint32_t* ws_flags = nullptr;
  if (impl != 0 && split_k) {
    auto& w = pair_workspace(st, a.device(), stream);
    ws = w.slots.data_ptr();
    ws_flags = reinterpret_cast<uint32_t*>(w.flags.data_ptr<int>());
  }
  const int rc = seg::gemm_bf16(a.data_ptr(), b.data_ptr(), cptr, routed ? nullptr : d.data_ptr(), M, N, K, batch, a.stride(-2), b.stride(-2),
                                routed ? route_ld : d.stride(-2), bsa, bsb, bsd, a_mn, b_mn, out_f32, (float)alpha, (float)beta, symmetric, extras,
                                (int)extra_dst.size(), st.status.data_ptr<int>(), st.sm_count, stream, wf, (uint32_t)wait_seq,
                                (int)region_rows, routes,
                                (int)route_ptrs.size(), (int)route_rows, route_batch_stride, route_base, (long long)wait_limit, (int)impl, ws,
                                ws_flags, split_k ? 1 : 0);
  TORCH_CHECK(rc == 0, "gemm_bf16 launch failed with code ", rc);
  return d;
}

// (u, f) = (x w^T, silu(u[:, :F]) * u[:, F:]) in one launch; w = [F gate rows | F up rows].
std::tuple<Tensor, Tensor> gemm_swiglu(const Tensor& x, const Tensor& w) {
  check_operand(x, "x");
  check_operand(w, "w");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1) && w.size(0) % 256 == 0, "x [M, K], w [2F, K] with F a multiple of 128");
  const int M = (int)x.size(0), K = (int)x.size(1), F = (int)(w.size(0) / 2);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor u = torch::empty({M, 2 * F}, x.options()), f = torch::empty({M, F}, x.options());
  auto& st = device_state(x.device());
  const int rc = seg::gemm_swiglu_pair(x.data_ptr(), w.data_ptr(), u.data_ptr(), f.data_ptr(), M, F, K, x.stride(0), w.stride(0), u.stride(0),
                                       f.stride(0), st.status.data_ptr<int>(), st.sm_count, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "gemm_swiglu launch failed with code ", rc);
  return {u, f};
}

// du = gradient of u = (gate | up) given dy [M, K], the down projection's weight w [K, F] and u [M, 2F].
Tensor gemm_swiglu_bwd(const Tensor& dy, const Tensor& w, const Tensor& u) {
  check_operand(dy, "dy");
  check_operand(w, "w");
  check_operand(u, "u");
  TORCH_CHECK(dy.dim() == 2 && w.dim() == 2 && u.dim() == 2 && dy.size(1) == w.size(0) && u.size(0) == dy.size(0) && u.size(1) == 2 * w.size(1) &&
                  w.size(1) % 256 == 0, "dy [M, K], w [K, F], u [M, 2F] with F a multiple of 256");
  const int M = (int)dy.size(0), K = (int)dy.size(1), F = (int)w.size(1);
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor du = torch::empty({M, 2 * F}, dy.options());
  auto& st = device_state(dy.device());
  const int rc = seg::gemm_swiglu_bwd_pair(dy.data_ptr(), w.data_ptr(), u.data_ptr(), du.data_ptr(), M, F, K, dy.stride(0), w.stride(0), u.stride(0),
                                           du.stride(0), st.status.data_ptr<int>(), st.sm_count, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "gemm_swiglu_bwd launch failed with code ", rc);
  return du;
}

// Host read of the status word (synchronises): 0 = every wait completed.
int64_t gemm_status(int64_t device_index) {
  auto& st = device_state(c10::Device(c10::kCUDA, (c10::DeviceIndex)device_index));
  return st.status.item<int>();
}

void gemm_reset_status(int64_t device_index) {
  // raw memsets: the tensors may have been created under inference mode, where in-place tensor ops are refused later
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_index);
  auto& st = device_state(c10::Device(c10::kCUDA, (c10::DeviceIndex)device_index));
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  cudaMemsetAsync(st.status.data_ptr(), 0, sizeof(int), stream);
  for (auto& kv : st.workspaces)  // a kernel that gave up may have left parts announced
    cudaMemsetAsync(kv.second.flags.data_ptr(), 0, (size_t)kv.second.flags.numel() * sizeof(int), stream);
}

// Causal GQA flash attention forward on the tcgen05 kernel: returns (o, lse).
static long long* prof_ptr(const std::optional<Tensor>& prof) {
  if (!prof.has_value()) return nullptr;
  TORCH_CHECK(prof->is_cuda() && prof->scalar_type() == at::kLong && prof->is_contiguous() && prof->numel() >= 16, "prof must be a CUDA int64 tensor of at least 16 elements");
  return reinterpret_cast<long long*>(prof->data_ptr<int64_t>());
}

std::tuple<Tensor, Tensor> fa_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, const std::optional<Tensor>& prof) {
  TORCH_CHECK(causal, "only causal attention is implemented");
  for (const Tensor* t : {&q, &k, &v}) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->is_contiguous() && t->dim() == 4, "q/k/v must be contiguous CUDA bf16 [B,S,H,hd]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "q/k/v must be 16-byte aligned");
  }
  const int B = q.size(0), S = q.size(1), H = q.size(2), hd = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(k.size(0) == B && k.size(1) == S && k.size(3) == hd && v.sizes() == k.sizes(), "k/v shape mismatch");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor o = torch::empty_like(q);
  Tensor lse = torch::empty({B, H, S}, q.options().dtype(at::kFloat));
  auto& st = device_state(q.device());
  const int rc = seg::attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B, S, H, Hkv, hd,
                               st.status.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream(), prof_ptr(prof));
  TORCH_CHECK(rc == 0, "attn_fwd: unsupported shape or launch failure (code ", rc, ")");
  return {o, lse};
}

// Backward of fa_fwd on the tcgen05 kernel: returns (dq, dk, dv).
std::tuple<Tensor, Tensor, Tensor> fa_bwd(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                          const Tensor& lse, bool causal, const std::optional<Tensor>& prof) {
  TORCH_CHECK(causal, "only causal attention is implemented");
  for (const Tensor* t : {&d_o, &q, &k, &v, &o}) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->is_contiguous() && t->dim() == 4, "dO/q/k/v/o must be contiguous CUDA bf16 [B,S,H,hd]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "dO/q/k/v/o must be 16-byte aligned");
  }
  const int B = q.size(0), S = q.size(1), H = q.size(2), hd = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(k.size(0) == B && k.size(1) == S && k.size(3) == hd && v.sizes() == k.sizes() && o.sizes() == q.sizes() && d_o.sizes() == q.sizes(),
              "shape mismatch");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.dim() == 3 && lse.size(0) == B && lse.size(1) == H &&
                  lse.size(2) == S, "lse must be contiguous fp32 [B,H,S]");
  c10::cuda::CUDAGuard guard(q.device());
  if (S % 128 != 0) {
    // The kernel walks whole 128-row tiles.  A ragged sequence is extended with zero rows: causality hides the added keys
    // from every real query, and an added query (q = 0, dO = 0, O = 0, lse = 0) has P = 1, dP = 0 and row sum 0, hence
    // dS = 0 and P^T dO = 0: it adds nothing to dK or dV.
    const int64_t pad = 128 - S % 128;
    auto rows = [&](const Tensor& t) { return at::constant_pad_nd(t, {0, 0, 0, 0, 0, pad}, 0).contiguous(); };
    auto [dq_p, dk_p, dv_p] = fa_bwd(rows(d_o), rows(q), rows(k), rows(v), rows(o), at::constant_pad_nd(lse, {0, pad}, 0).contiguous(), causal, prof);
    return {dq_p.narrow(1, 0, S).contiguous(), dk_p.narrow(1, 0, S).contiguous(), dv_p.narrow(1, 0, S).contiguous()};
  }
  Tensor dq = torch::empty_like(q), dk = torch::empty_like(k), dv = torch::empty_like(v);
  Tensor acc = torch::empty(q.sizes(), q.options().dtype(at::kFloat));
  Tensor dsum = torch::empty_like(lse), lse2 = torch::empty_like(lse);
  auto& st = device_state(q.device());
  const int rc = seg::attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(), dq.data_ptr(),
                               dk.data_ptr(), dv.data_ptr(), acc.data_ptr<float>(), dsum.data_ptr<float>(), lse2.data_ptr<float>(), B, S, H,
                               Hkv, hd, st.status.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream(), prof_ptr(prof));
  TORCH_CHECK(rc == 0, "attn_bwd: unsupported shape or launch failure (code ", rc, ")");
  return {dq, dk, dv};
}

}  // namespace

void register_gemm(pybind11::module_& m) {
  m.def("gemm", &gemm, pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("c") = std::nullopt, pybind11::arg("out") = std::nullopt,
        pybind11::arg("out_f32") = false, pybind11::arg("a_mn") = false, pybind11::arg("b_mn") = false, pybind11::arg("alpha") = 1.0,
        pybind11::arg("beta") = 0.0, pybind11::arg("symmetric") = false,
        pybind11::arg("extra_dst") = std::vector<int64_t>(), pybind11::arg("wait_flags") = std::nullopt, pybind11::arg("wait_seq") = 0,
        pybind11::arg("region_rows") = 0, pybind11::arg("route_ptrs") = std::vector<int64_t>(), pybind11::arg("route_rows") = 0,
        pybind11::arg("route_batch_stride") = 0, pybind11::arg("route_base") = 0, pybind11::arg("route_ld") = 0,
        pybind11::arg("impl") = 1, pybind11::arg("split_k") = true, pybind11::arg("wait_limit") = 0);
  m.def("gemm_swiglu", &gemm_swiglu, pybind11::arg("x"), pybind11::arg("w"));
  m.def("gemm_swiglu_bwd", &gemm_swiglu_bwd, pybind11::arg("dy"), pybind11::arg("w"), pybind11::arg("u"));
  m.def("fa_fwd", &fa_fwd, pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("causal"), pybind11::arg("prof") = std::nullopt);
  m.def("fa_bwd", &fa_bwd, pybind11::arg("d_o"), pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("o"), pybind11::arg("lse"),
        pybind11::arg("causal"), pybind11::arg("prof") = std::nullopt);
  m.def("gemm_status", &gemm_status);
  m.def("gemm_debug_extent_cap", [](int64_t n) { seg::gemm_debug_extent_cap(n); });
#ifdef SEG_DEBUG_BOUNDS
  m.attr("DEBUG_BOUNDS") = true;
#else
  m.attr("DEBUG_BOUNDS") = false;
#endif
  m.def("gemm_reset_status", &gemm_reset_status);
}
