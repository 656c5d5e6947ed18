// Python bindings (pybind11 via torch/extension.h) for the sm_100a kernels.  Tensors are checked here
// (device, dtype, contiguity, alignment-relevant sizes) and handed to the launchers as raw pointers on
// the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <optional>
#include <vector>

#include "kernels.h"

int* package_status_ptr(const c10::Device& dev);  // gemm_bindings.cpp

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// The kernels use 16-byte vector accesses: a tensor that starts off such a boundary (a view at an odd offset)
// is rejected here instead of faulting on the device.
void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.numel() == 0 || reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must start on a 16-byte boundary");
}
void check_lp(const Tensor& t, bool bf16, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == (bf16 ? at::kBFloat16 : at::kFloat), name, " has the wrong dtype");
}
// [rows, cols] activations that may be a column slice of a wider buffer: unit column stride, 16-byte aligned rows.
void check_rows(const Tensor& t, bool bf16, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.stride(1) == 1, name, " must be a CUDA matrix with unit column stride");
  TORCH_CHECK(t.scalar_type() == (bf16 ? at::kBFloat16 : at::kFloat), name, " has the wrong dtype");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && (t.stride(0) * t.element_size()) % 16 == 0, name,
              " rows must start on 16-byte boundaries");
}
void check_f32(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
}
const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// ------------------------------------------------------------------------------------------------ norm
std::tuple<Tensor, Tensor, Tensor, OptTensor> add_rmsnorm_fwd(const Tensor& res, const OptTensor& delta, const Tensor& gain,
                                                              double scale, double eps, bool bf16, bool want_kurt) {
  check_f32(res, "res");
  check_f32(gain, "gain");
  TORCH_CHECK(res.dim() == 2, "res must be [T, d]");
  const int T = res.size(0), d = res.size(1);
  TORCH_CHECK(d % 4 == 0, "d must be a multiple of 4");
  c10::cuda::CUDAGuard guard(res.device());
  if (delta.has_value()) check_lp(*delta, bf16, "delta");
  auto lp = res.options().dtype(bf16 ? at::kBFloat16 : at::kFloat);
  Tensor x = delta.has_value() ? torch::empty_like(res) : res;
  Tensor y = torch::empty({T, d}, lp);
  Tensor rstd = torch::empty({T}, res.options());
  OptTensor kurt;
  if (want_kurt) kurt = torch::zeros({}, res.options());
  seg::add_rmsnorm_fwd(res.data_ptr<float>(), opt_ptr(delta), gain.data_ptr<float>(),
                       delta.has_value() ? x.data_ptr<float>() : nullptr, y.data_ptr(), rstd.data_ptr<float>(),
                       want_kurt ? kurt->data_ptr<float>() : nullptr, T, d, (float)scale, (float)eps, bf16, cur_stream());
  return {x, y, rstd, kurt};
}

std::tuple<Tensor, Tensor, Tensor> add_rmsnorm_bwd(const Tensor& dy, const OptTensor& dres_in, const Tensor& x, const Tensor& gain,
                                                   const Tensor& rstd, double scale, bool bf16) {
  check_lp(dy, bf16, "dy");
  check_f32(x, "x");
  check_f32(gain, "gain");
  check_f32(rstd, "rstd");
  if (dres_in.has_value()) check_f32(*dres_in, "dres_in");
  const int T = x.size(0), d = x.size(1);
  TORCH_CHECK(d % 4 == 0, "d must be a multiple of 4");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dres = torch::empty_like(x);
  Tensor dres_lp = torch::empty_like(dy);
  Tensor dgain = torch::empty({d}, x.options());
  Tensor scratch = torch::empty({seg::add_rmsnorm_bwd_grid(T), d}, x.options());
  seg::add_rmsnorm_bwd(dy.data_ptr(), dres_in.has_value() ? dres_in->data_ptr<float>() : nullptr, x.data_ptr<float>(),
                       gain.data_ptr<float>(), rstd.data_ptr<float>(), dres.data_ptr<float>(), dres_lp.data_ptr(),
                       dgain.data_ptr<float>(), scratch.data_ptr<float>(), T, d, (float)scale, bf16, cur_stream());
  return {dres, dres_lp, dgain};
}

// ------------------------------------------------------------------------------------------------ elementwise
Tensor swiglu_fwd(const Tensor& u) {
  check_cuda(u, "u");
  const bool bf16 = u.scalar_type() == at::kBFloat16;
  check_lp(u, bf16, "u");
  const int64_t T = u.size(0);
  const int F = u.size(1) / 2;
  TORCH_CHECK(F % 4 == 0, "ffn width must be a multiple of 4");
  c10::cuda::CUDAGuard guard(u.device());
  Tensor f = torch::empty({T, F}, u.options());
  seg::swiglu_fwd(u.data_ptr(), f.data_ptr(), T, F, bf16, cur_stream());
  return f;
}

Tensor swiglu_bwd(const Tensor& df, const Tensor& u) {
  const bool bf16 = u.scalar_type() == at::kBFloat16;
  check_lp(u, bf16, "u");
  check_lp(df, bf16, "df");
  const int64_t T = u.size(0);
  const int F = u.size(1) / 2;
  c10::cuda::CUDAGuard guard(u.device());
  Tensor du = torch::empty_like(u);
  seg::swiglu_bwd(df.data_ptr(), u.data_ptr(), du.data_ptr(), T, F, bf16, cur_stream());
  return du;
}

void check_hd(int hd) { TORCH_CHECK(hd == 32 || hd == 64 || hd == 128, "head_dim must be 32, 64 or 128"); }

// z: [T, H] gate logits, possibly a column slice of a wider tensor (row stride >= H, unit column stride)
void check_gate_logits(const Tensor& z, bool bf16, int64_t T, int H, const char* name) {
  TORCH_CHECK(z.is_cuda() && z.scalar_type() == (bf16 ? at::kBFloat16 : at::kFloat), name, " has the wrong device or dtype");
  TORCH_CHECK(z.dim() == 2 && z.size(0) == T && z.size(1) == H && z.stride(1) == 1 && z.stride(0) >= H, name, " must be [T, H] with unit column stride");
}

Tensor gate_fwd(const Tensor& o, const Tensor& z) {
  const bool bf16 = o.scalar_type() == at::kBFloat16;
  check_lp(o, bf16, "o");
  TORCH_CHECK(o.dim() == 3, "o must be [T, H, hd]");
  const int64_t T = o.size(0);
  const int H = o.size(1), hd = o.size(2);
  check_hd(hd);
  check_gate_logits(z, bf16, T, H, "z");
  c10::cuda::CUDAGuard guard(o.device());
  Tensor g = torch::empty({T, (int64_t)H * hd}, o.options());
  seg::gate_fwd(o.data_ptr(), z.data_ptr(), g.data_ptr(), T, H, hd, bf16, cur_stream(), z.stride(0));
  return g;
}

// dz_out (optional): [T, H] destination of the gate-logit gradient, e.g. columns of the fused projection's gradient buffer
std::tuple<Tensor, Tensor> gate_bwd(const Tensor& dg, const Tensor& o, const Tensor& z, const OptTensor& dz_out) {
  const bool bf16 = o.scalar_type() == at::kBFloat16;
  check_lp(o, bf16, "o");
  check_lp(dg, bf16, "dg");
  const int64_t T = o.size(0);
  const int H = o.size(1), hd = o.size(2);
  check_hd(hd);
  check_gate_logits(z, bf16, T, H, "z");
  c10::cuda::CUDAGuard guard(o.device());
  Tensor dout = torch::empty_like(o);
  Tensor dz;
  if (dz_out.has_value()) {
    dz = *dz_out;
    check_gate_logits(dz, bf16, T, H, "dz_out");
  } else {
    dz = torch::empty({T, (int64_t)H}, o.options());
  }
  seg::gate_bwd(dg.data_ptr(), o.data_ptr(), z.data_ptr(), dout.data_ptr(), dz.data_ptr(), T, H, hd, bf16, cur_stream(), z.stride(0), dz.stride(0));
  return {dout, dz};
}

// ------------------------------------------------------------------------------------------------ qkv post
seg::QkvPostParams make_post(const Tensor& cos, const Tensor& sin, const Tensor& qgain, const Tensor& a1, const Tensor& a2,
                             const Tensor& vs, int B, int S, int H, int Hkv, int hd, bool qknorm) {
  check_f32(cos, "cos");
  check_f32(sin, "sin");
  check_f32(qgain, "qgain");
  check_f32(a1, "alpha1");
  check_f32(a2, "alpha2");
  check_f32(vs, "vscale");
  check_hd(hd);
  TORCH_CHECK(cos.size(0) >= S && cos.size(1) == hd / 2, "rope table too small for this sequence / head_dim");
  seg::QkvPostParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.hd = hd; p.qknorm = qknorm;
  p.cos = cos.data_ptr<float>(); p.sin = sin.data_ptr<float>(); p.qgain = qgain.data_ptr<float>();
  p.alpha1 = a1.data_ptr<float>(); p.alpha2 = a2.data_ptr<float>(); p.vscale = vs.data_ptr<float>();
  p.qkv_stride = 0;
  p.pos = nullptr;
  return p;
}

std::tuple<Tensor, Tensor, Tensor> qkv_post_fwd(const Tensor& qkv, const OptTensor& v1, const Tensor& cos, const Tensor& sin,
                                                const Tensor& qgain, const Tensor& a1, const Tensor& a2, const Tensor& vs, int B,
                                                int S, int H, int Hkv, int hd, bool qknorm, const OptTensor& pos) {
  const bool bf16 = qkv.scalar_type() == at::kBFloat16;
  check_rows(qkv, bf16, "qkv");
  TORCH_CHECK(qkv.size(0) == (int64_t)B * S && qkv.size(1) == (int64_t)(H + 2 * Hkv) * hd, "qkv has the wrong shape");
  if (v1.has_value()) check_lp(*v1, bf16, "v1");
  c10::cuda::CUDAGuard guard(qkv.device());
  auto p = make_post(cos, sin, qgain, a1, a2, vs, B, S, H, Hkv, hd, qknorm);
  p.qkv_stride = qkv.stride(0);
  p.status = package_status_ptr(qkv.device());
  if (pos.has_value()) {
    TORCH_CHECK(pos->is_cuda() && pos->scalar_type() == at::kInt && pos->numel() == 1, "pos must be a CUDA int32 scalar");
    p.pos = pos->data_ptr<int>();
  }
  Tensor q = torch::empty({B, S, H, hd}, qkv.options());
  Tensor k = torch::empty({B, S, Hkv, hd}, qkv.options());
  Tensor v = torch::empty({B, S, Hkv, hd}, qkv.options());
  seg::qkv_post_fwd(qkv.data_ptr(), opt_ptr(v1), q.data_ptr(), k.data_ptr(), v.data_ptr(), p, bf16, cur_stream());
  return {q, k, v};
}

std::tuple<Tensor, OptTensor, Tensor, Tensor, Tensor, Tensor> qkv_post_bwd(
    const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& qkv, const OptTensor& v1, const Tensor& cos,
    const Tensor& sin, const Tensor& qgain, const Tensor& a1, const Tensor& a2, const Tensor& vs, int B, int S, int H, int Hkv,
    int hd, bool qknorm, const OptTensor& dqkv_out, const OptTensor& dv1_acc) {
  const bool bf16 = qkv.scalar_type() == at::kBFloat16;
  check_rows(qkv, bf16, "qkv");
  check_lp(dq, bf16, "dq");
  check_lp(dk, bf16, "dk");
  check_cuda(dv, "dv");
  const bool dv_f32 = dv.scalar_type() == at::kFloat;
  TORCH_CHECK(dv_f32 || dv.scalar_type() == qkv.scalar_type(), "dv must be float32 or the activation dtype");
  if (v1.has_value()) check_lp(*v1, bf16, "v1");
  c10::cuda::CUDAGuard guard(qkv.device());
  auto p = make_post(cos, sin, qgain, a1, a2, vs, B, S, H, Hkv, hd, qknorm);
  const int64_t T = (int64_t)B * S;
  auto f32 = qkv.options().dtype(at::kFloat);
  // dqkv shares qkv's row stride: either a fresh buffer of qkv's layout or the caller's wider one (same stride as qkv)
  Tensor dqkv;
  if (dqkv_out.has_value()) {
    dqkv = *dqkv_out;
    check_rows(dqkv, bf16, "dqkv_out");
    TORCH_CHECK(dqkv.size(0) == qkv.size(0) && dqkv.size(1) == qkv.size(1) && dqkv.stride(0) == qkv.stride(0),
                "dqkv_out must have qkv's shape and row stride");
  } else {
    dqkv = torch::empty_strided(qkv.sizes(), qkv.strides(), qkv.options());
  }
  p.qkv_stride = qkv.stride(0);
  p.status = package_status_ptr(qkv.device());
  OptTensor dv1;
  if (v1.has_value()) {
    if (dv1_acc.has_value()) {  // running sum over blocks, updated in place
      check_f32(*dv1_acc, "dv1_acc");
      TORCH_CHECK(dv1_acc->numel() == T * Hkv * hd, "dv1_acc must hold [B, S, Hkv, hd]");
      dv1 = *dv1_acc;
      p.dv1_accumulate = true;
    } else {
      dv1 = torch::empty({B, S, Hkv, hd}, f32);
    }
  }
  Tensor scalars = torch::empty({4}, f32);
  Tensor partial = torch::empty({seg::qkv_post_bwd_grid(T, H + 2 * Hkv, hd), 4}, f32);
  seg::qkv_post_bwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dv_f32, qkv.data_ptr(), opt_ptr(v1), dqkv.data_ptr(),
                    dv1.has_value() ? dv1->data_ptr<float>() : nullptr, scalars.data_ptr<float>(), partial.data_ptr<float>(), p,
                    bf16, cur_stream());
  return {dqkv, dv1, scalars.slice(0, 0, 1), scalars.slice(0, 1, 2), scalars.slice(0, 2, 3), scalars.slice(0, 3, 4)};
}

// ------------------------------------------------------------------------------------------------ cross entropy
void ce_chunk_fwd_bwd(Tensor logits, const Tensor& targets, Tensor loss, Tensor z, Tensor lse, double lse_square_scale,
                      int64_t ignore_index, double grad_scale, double logit_scale, bool write_grad) {
  check_lp(logits, true, "logits");
  check_cuda(targets, "targets");
  TORCH_CHECK(targets.scalar_type() == at::kLong, "targets must be int64");
  check_f32(loss, "loss");
  check_f32(z, "z");
  check_f32(lse, "lse");
  const int rows = logits.size(0), V = logits.size(1);
  TORCH_CHECK(V % 8 == 0 && V <= 65536, "vocabulary must be a multiple of 8 and at most 65536");
  TORCH_CHECK(loss.numel() == rows && z.numel() == rows && lse.numel() == rows && targets.numel() == rows, "row count mismatch");
  c10::cuda::CUDAGuard guard(logits.device());
  seg::ce_chunk_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), z.data_ptr<float>(),
                        lse.data_ptr<float>(), rows, V, (float)lse_square_scale, ignore_index, (float)grad_scale,
                        (float)logit_scale, write_grad, cur_stream());
}

// ------------------------------------------------------------------------------------------------ multi-tensor
constexpr int kChunkElems = 64 * 1024;

struct TensorTable {
  Tensor ptrs;      // int64 [n_lists, n_tensors] device
  Tensor sizes;     // int64 [n_tensors]
  Tensor chunk_t;   // int32 [n_chunks]
  Tensor chunk_off; // int64 [n_chunks]
  int n_chunks = 0;
  int n_tensors = 0;
};

// Tables are cached by the pointer values they hold: a training run builds each one once.
const TensorTable& get_table(const std::vector<std::vector<Tensor>>& lists) {
  static std::map<std::vector<int64_t>, TensorTable> cache;
  const size_t n = lists[0].size();
  std::vector<int64_t> key;
  key.reserve(lists.size() * n + 1);
  key.push_back((int64_t)lists.size());
  for (const auto& l : lists) {
    TORCH_CHECK(l.size() == n, "tensor lists must have equal length");
    for (const auto& t : l) key.push_back(t.numel() ? (int64_t)(uintptr_t)t.data_ptr() : 0);
  }
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 64) cache.clear();
  TensorTable tb;
  tb.n_tensors = (int)n;
  auto dev = lists[0][0].device();
  Tensor ptrs = torch::empty({(int64_t)lists.size(), (int64_t)n}, torch::dtype(torch::kInt64).pinned_memory(true));
  Tensor sizes = torch::empty({(int64_t)n}, torch::dtype(torch::kInt64).pinned_memory(true));
  std::vector<int32_t> ct;
  std::vector<int64_t> co;
  for (size_t i = 0; i < n; ++i) {
    const int64_t ne = lists[0][i].numel();
    sizes.data_ptr<int64_t>()[i] = ne;
    for (size_t l = 0; l < lists.size(); ++l) ptrs.data_ptr<int64_t>()[l * n + i] = key[1 + l * n + i];
    for (int64_t o = 0; o < ne; o += kChunkElems) {
      ct.push_back((int32_t)i);
      co.push_back(o);
    }
  }
  tb.n_chunks = (int)ct.size();
  Tensor cth = torch::empty({(int64_t)ct.size()}, torch::dtype(torch::kInt32).pinned_memory(true));
  Tensor coh = torch::empty({(int64_t)co.size()}, torch::dtype(torch::kInt64).pinned_memory(true));
  std::memcpy(cth.data_ptr(), ct.data(), ct.size() * sizeof(int32_t));
  std::memcpy(coh.data_ptr(), co.data(), co.size() * sizeof(int64_t));
  tb.ptrs = ptrs.to(dev);
  tb.sizes = sizes.to(dev);
  tb.chunk_t = cth.to(dev);
  tb.chunk_off = coh.to(dev);
  return cache.emplace(std::move(key), std::move(tb)).first->second;
}

void check_list(const std::vector<Tensor>& l, at::ScalarType st, const char* name, const std::vector<Tensor>* like = nullptr,
                bool need_aligned = false) {
  for (size_t i = 0; i < l.size(); ++i) {
    if (l[i].numel() == 0) continue;
    TORCH_CHECK(l[i].is_cuda() && l[i].is_contiguous(), name, " must be contiguous CUDA tensors");
    if (need_aligned)
      TORCH_CHECK(reinterpret_cast<uintptr_t>(l[i].data_ptr()) % 16 == 0, name, " must start on 16-byte boundaries");
    TORCH_CHECK(l[i].scalar_type() == st, name, " has the wrong dtype");
    if (like) TORCH_CHECK(l[i].numel() == (*like)[i].numel(), name, " size mismatch");
  }
}

void adamw(std::vector<Tensor> ps, std::vector<Tensor> gs, std::vector<Tensor> ms, std::vector<Tensor> vs,
           std::vector<Tensor> shadows, double lr, double wd, double b1, double b2, double eps, double step_size) {
  if (ps.empty()) return;
  check_list(ps, at::kFloat, "params");
  check_list(gs, at::kFloat, "grads", &ps);
  check_list(ms, at::kFloat, "m", &ps);
  check_list(vs, at::kFloat, "v", &ps);
  check_list(shadows, at::kBFloat16, "shadows", &ps);
  c10::cuda::CUDAGuard guard(ps[0].device());
  const auto& tb = get_table({ps, gs, ms, vs, shadows});
  int64_t* base = tb.ptrs.data_ptr<int64_t>();
  const int n = tb.n_tensors;
  seg::adamw_multi((float**)(base), (const float**)(base + n), (float**)(base + 2 * n), (float**)(base + 3 * n),
                   (void**)(base + 4 * n), tb.sizes.data_ptr<int64_t>(), tb.chunk_t.data_ptr<int32_t>(),
                   tb.chunk_off.data_ptr<int64_t>(), tb.n_chunks, kChunkElems, (float)lr, (float)wd, (float)b1, (float)b2,
                   (float)eps, (float)step_size, cur_stream());
}

void ema(std::vector<Tensor> shadow, std::vector<Tensor> srcs, double decay) {
  if (shadow.empty()) return;
  check_list(shadow, at::kFloat, "ema");
  check_list(srcs, at::kFloat, "src", &shadow);
  c10::cuda::CUDAGuard guard(shadow[0].device());
  const auto& tb = get_table({shadow, srcs});
  int64_t* base = tb.ptrs.data_ptr<int64_t>();
  const int n = tb.n_tensors;
  seg::ema_multi((float**)base, (const float**)(base + n), tb.sizes.data_ptr<int64_t>(), tb.chunk_t.data_ptr<int32_t>(),
                 tb.chunk_off.data_ptr<int64_t>(), tb.n_chunks, kChunkElems, (float)decay, cur_stream());
}

void cast_bf16(std::vector<Tensor> dsts, std::vector<Tensor> srcs) {
  if (dsts.empty()) return;
  check_list(dsts, at::kBFloat16, "dst");
  check_list(srcs, at::kFloat, "src", &dsts);
  c10::cuda::CUDAGuard guard(dsts[0].device());
  const auto& tb = get_table({dsts, srcs});
  int64_t* base = tb.ptrs.data_ptr<int64_t>();
  const int n = tb.n_tensors;
  seg::cast_multi((void**)base, (const float**)(base + n), tb.sizes.data_ptr<int64_t>(), tb.chunk_t.data_ptr<int32_t>(),
                  tb.chunk_off.data_ptr<int64_t>(), tb.n_chunks, kChunkElems, cur_stream());
}

// ------------------------------------------------------------------------------------------------ muon
// grads: the owned matrices' fp32 gradients; slot_of: int32 device tensor with their slots in the stacked buffers.
void muon_momentum(std::vector<Tensor> grads, const Tensor& slot_of, Tensor momentum, Tensor xout, double mu, double eps) {
  if (grads.empty()) return;
  check_list(grads, at::kFloat, "grads", nullptr, true);
  check_f32(momentum, "momentum");
  check_lp(xout, true, "xout");
  TORCH_CHECK(slot_of.is_cuda() && slot_of.scalar_type() == at::kInt && slot_of.numel() == (int64_t)grads.size(), "slot_of mismatch");
  const int64_t numel = grads[0].numel();
  TORCH_CHECK(numel % 8 == 0, "matrix size must be a multiple of 8");
  for (auto& g : grads) TORCH_CHECK(g.numel() == numel && g.is_contiguous(), "gradients of one group must share a shape");
  TORCH_CHECK(momentum.numel() % numel == 0 && xout.numel() == momentum.numel(), "stacked buffers have the wrong size");
  c10::cuda::CUDAGuard guard(momentum.device());
  const auto& tb = get_table({grads});
  const int n = (int)grads.size();
  Tensor partial = torch::empty({(int64_t)n * seg::muon_chunks_per_matrix(numel)}, momentum.options());
  seg::muon_momentum((const float* const*)tb.ptrs.data_ptr<int64_t>(), slot_of.data_ptr<int>(), momentum.data_ptr<float>(),
                     xout.data_ptr(), partial.data_ptr<float>(), n, numel, (float)mu, (float)eps, cur_stream());
}

void muon_tail(const Tensor& v, const Tensor& slot_of, Tensor second, std::vector<Tensor> params, std::vector<Tensor> shadows,
               Tensor sq_sum_out, int64_t R, int64_t C, double beta2, bool normalize, double lr_eff, double decay, int64_t mode) {
  if (params.empty()) return;
  check_lp(v, true, "v");
  check_list(params, at::kFloat, "params", nullptr, true);
  check_f32(sq_sum_out, "sq_sum_out");
  const int n = (int)params.size();
  TORCH_CHECK(slot_of.is_cuda() && slot_of.scalar_type() == at::kInt && slot_of.numel() == n, "slot_of mismatch");
  TORCH_CHECK(C % 8 == 0, "columns must be a multiple of 8");
  for (auto& p : params) TORCH_CHECK(p.numel() == R * C && p.is_contiguous(), "parameters of one group must share a shape");
  const bool with_shadows = !shadows.empty();
  if (with_shadows) {
    TORCH_CHECK((int)shadows.size() == n, "shadows mismatch");
    check_list(shadows, at::kBFloat16, "shadows", &params, true);
  }
  const int64_t len = R >= C ? R : C;
  if (normalize) {
    check_f32(second, "second");
    TORCH_CHECK(second.numel() == (int64_t)n * len, "second-moment buffer has the wrong size");
  }
  c10::cuda::CUDAGuard guard(v.device());
  const auto& tb = with_shadows ? get_table({params, shadows}) : get_table({params});
  int64_t* base = tb.ptrs.data_ptr<int64_t>();
  auto f32 = v.options().dtype(at::kFloat);
  Tensor sq = torch::empty({(int64_t)n, len}, f32), mult = torch::empty({(int64_t)n, len}, f32);
  seg::muon_tail(v.data_ptr(), slot_of.data_ptr<int>(), normalize ? second.data_ptr<float>() : nullptr, sq.data_ptr<float>(),
                 mult.data_ptr<float>(), (float* const*)base, with_shadows ? (void* const*)(base + n) : nullptr,
                 sq_sum_out.data_ptr<float>(), n, (int)R, (int)C, (float)beta2, normalize ? 1 : 0, (float)lr_eff, (float)decay,
                 (int)mode, cur_stream());
}

}  // namespace

void register_gemm(pybind11::module_& m);  // gemm_bindings.cpp
void register_comm(pybind11::module_& m);  // comm_bindings.cpp
void register_moe(pybind11::module_& m);   // moe_bindings.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a kernels of sample_efficient_gpt_b200";
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("add_rmsnorm_bwd", &add_rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("gate_fwd", &gate_fwd);
  m.def("gate_bwd", &gate_bwd, pybind11::arg("dg"), pybind11::arg("o"), pybind11::arg("z"), pybind11::arg("dz_out") = std::nullopt);
  m.def("qkv_post_fwd", &qkv_post_fwd, pybind11::arg("qkv"), pybind11::arg("v1"), pybind11::arg("cos"), pybind11::arg("sin"),
        pybind11::arg("qgain"), pybind11::arg("a1"), pybind11::arg("a2"), pybind11::arg("vs"), pybind11::arg("B"), pybind11::arg("S"),
        pybind11::arg("H"), pybind11::arg("Hkv"), pybind11::arg("hd"), pybind11::arg("qknorm"), pybind11::arg("pos") = std::nullopt);
  m.def("qkv_post_bwd", &qkv_post_bwd, pybind11::arg("dq"), pybind11::arg("dk"), pybind11::arg("dv"), pybind11::arg("qkv"),
        pybind11::arg("v1"), pybind11::arg("cos"), pybind11::arg("sin"), pybind11::arg("qgain"), pybind11::arg("a1"), pybind11::arg("a2"),
        pybind11::arg("vs"), pybind11::arg("B"), pybind11::arg("S"), pybind11::arg("H"), pybind11::arg("Hkv"), pybind11::arg("hd"),
        pybind11::arg("qknorm"), pybind11::arg("dqkv_out") = std::nullopt, pybind11::arg("dv1_acc") = std::nullopt);
  m.def("ce_chunk_fwd_bwd", &ce_chunk_fwd_bwd);
  m.def("adamw", &adamw);
  m.def("ema", &ema);
  m.def("cast_bf16", &cast_bf16);
  m.def("muon_momentum", &muon_momentum);
  m.def("muon_tail", &muon_tail);
  register_gemm(m);
  register_comm(m);
  register_moe(m);
}
