// Element-wise parts of the (Nor)Muon step, fused.  All matrices of one shape [R, C] are handled by one launch;
// per-matrix tensors (gradients, parameters, bf16 shadows) come as device pointer arrays, stacked state
// (momentum, Newton-Schulz input/output, second moments) as [slots, R, C] buffers indexed through slot_of[i].
//
//   momentum : buf <- buf + (1-mu)(g-buf);  g~ = g + mu(buf-g);  X = bf16(g~);  partial sums of X^2 per chunk
//   fro_scale: X <- X / (bf16(||X||_F) + eps)                                  (Newton-Schulz input normalisation)
//   rowsq    : sq[i, j] = sum over the reduced axis of v^2  (j = row when R >= C, else column)
//   plan     : second <- lerp(second, sq/len, 1-beta2); step = rsqrt(max(second, 1e-10));
//              mult[j] = step[j] * ||v|| / max(sqrt(sum_j step[j]^2 sq[j]), 1e-10); also accumulates ||v||^2
//              (the renormalised norm follows from the per-row sums, so v is not read again)
//   apply    : v' = v * mult;  cautious decay p -= lr*wd*p*[sign v' == sign p] (or plain p *= 1 - lr*wd);
//              p -= lr_eff * v';  bf16 shadow of p refreshed
// Reference: training/optimizers/normuon_cwd.py:13-31,94-110 and muon_triton.py:352-357 (about 15 eager kernels
// per matrix there).
#include "common.cuh"
#include "kernels.h"

namespace seg {

__global__ void __launch_bounds__(256) muon_momentum_kernel(const float* const* __restrict__ grads, const int32_t* __restrict__ slot_of,
                                                          float* __restrict__ momentum, __nv_bfloat16* __restrict__ xout,
                                                          float* __restrict__ partial, int64_t numel, int chunks_per_mat,
                                                          int chunk_elems, float mu) {
  __shared__ float red[32];
  const int mat = blockIdx.x / chunks_per_mat;
  const int ch = blockIdx.x % chunks_per_mat;
  const int64_t off = (int64_t)ch * chunk_elems;
  const int64_t end = (off + chunk_elems < numel) ? off + chunk_elems : numel;
  const int64_t base = (int64_t)slot_of[mat] * numel;
  const float* g = grads[mat];
  float ss = 0.f;
  for (int64_t i = off + (int64_t)threadIdx.x * 4; i < end; i += (int64_t)blockDim.x * 4) {
    const float4 gv = *reinterpret_cast<const float4*>(g + i);
    float4 mv = *reinterpret_cast<const float4*>(momentum + base + i);
    mv.x += (1.f - mu) * (gv.x - mv.x);
    mv.y += (1.f - mu) * (gv.y - mv.y);
    mv.z += (1.f - mu) * (gv.z - mv.z);
    mv.w += (1.f - mu) * (gv.w - mv.w);
    *reinterpret_cast<float4*>(momentum + base + i) = mv;
    const float4 t = make_float4(gv.x + mu * (mv.x - gv.x), gv.y + mu * (mv.y - gv.y), gv.z + mu * (mv.z - gv.z),
                                 gv.w + mu * (mv.w - gv.w));
    __nv_bfloat162 lo = __floats2bfloat162_rn(t.x, t.y), hi = __floats2bfloat162_rn(t.z, t.w);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(xout + base + i) = u;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

__global__ void __launch_bounds__(256) muon_fro_scale_kernel(const int32_t* __restrict__ slot_of, __nv_bfloat16* __restrict__ x,
                                                           const float* __restrict__ partial, int64_t numel, int chunks_per_mat,
                                                           int chunk_elems, float eps) {
  __shared__ float red[32];
  const int mat = blockIdx.x / chunks_per_mat;
  const int ch = blockIdx.x % chunks_per_mat;
  float s = 0.f;
  for (int i = threadIdx.x; i < chunks_per_mat; i += blockDim.x) s += partial[mat * chunks_per_mat + i];
  s = block_sum(s, red);
  const float norm = __bfloat162float(__float2bfloat16_rn(sqrtf(s)));
  const float inv = 1.f / (norm + eps);
  const int64_t off = (int64_t)ch * chunk_elems;
  const int64_t end = (off + chunk_elems < numel) ? off + chunk_elems : numel;
  const int64_t base = (int64_t)slot_of[mat] * numel;
  for (int64_t i = off + (int64_t)threadIdx.x * 8; i < end; i += (int64_t)blockDim.x * 8) {
    float f[8];
    load8<__nv_bfloat16>(x + base + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= inv;
    store8<__nv_bfloat16>(x + base + i, f);
  }
}

// R >= C: one warp per row.  sq[mat, row] = sum_c v^2
__global__ void __launch_bounds__(256) muon_rowsq_kernel(const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ slot_of,
                                                       float* __restrict__ sq, int R, int C) {
  const int mat = blockIdx.y;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= R) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* p = v + ((int64_t)slot_of[mat] * R + row) * C;
  float s = 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    float f[8];
    load8<__nv_bfloat16>(p + c, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * f[j];
  }
  s = warp_sum(s);
  if (lane == 0) sq[(int64_t)mat * R + row] = s;
}

// R < C: one thread per column, rows walked in order.  sq[mat, col] = sum_r v^2
__global__ void __launch_bounds__(256) muon_colsq_kernel(const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ slot_of,
                                                       float* __restrict__ sq, int R, int C) {
  const int mat = blockIdx.y;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= C) return;
  const __nv_bfloat16* p = v + (int64_t)slot_of[mat] * R * C + col;
  float s = 0.f;
#pragma unroll 4
  for (int r = 0; r < R; ++r) {
    const float f = __bfloat162float(p[(int64_t)r * C]);
    s += f * f;
  }
  sq[(int64_t)mat * C + col] = s;
}

// One CTA per matrix.  len = number of entries of sq/second/mult per matrix, red_len = length of the reduced axis.
__global__ void __launch_bounds__(256) muon_plan_kernel(const float* __restrict__ sq, float* __restrict__ second,
                                                      float* __restrict__ mult, float* __restrict__ sq_sum_out, int len, int red_len,
                                                      float beta2, int normalize) {
  __shared__ float red[32];
  const int mat = blockIdx.x;
  const float* s = sq + (int64_t)mat * len;
  float tot = 0.f, tot_new = 0.f;
  for (int j = threadIdx.x; j < len; j += blockDim.x) {
    const float q = s[j];
    tot += q;
    if (normalize) {
      float sec = second[(int64_t)mat * len + j];
      sec += (1.f - beta2) * (q / red_len - sec);
      second[(int64_t)mat * len + j] = sec;
      const float step = rsqrtf(fmaxf(sec, 1e-10f));
      mult[(int64_t)mat * len + j] = step;
      tot_new += step * step * q;
    }
  }
  tot = block_sum(tot, red);
  if (normalize) {
    tot_new = block_sum(tot_new, red);
    const float f = sqrtf(tot) / fmaxf(sqrtf(tot_new), 1e-10f);
    for (int j = threadIdx.x; j < len; j += blockDim.x) mult[(int64_t)mat * len + j] *= f;
  } else {
    for (int j = threadIdx.x; j < len; j += blockDim.x) mult[(int64_t)mat * len + j] = 1.f;
  }
  if (threadIdx.x == 0) atomicAdd(sq_sum_out, tot);
}

// mode: 0 = no decay, 1 = plain decay (p *= 1 - decay), 2 = cautious decay (p -= decay * p where sign(v') == sign(p))
__global__ void __launch_bounds__(256) muon_apply_kernel(const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ slot_of,
                                                       const float* __restrict__ mult, float* const* __restrict__ params,
                                                       __nv_bfloat16* const* __restrict__ shadows, int R, int C, int per_row,
                                                       float lr_eff, float decay, int mode) {
  const int mat = blockIdx.y;
  const int64_t numel = (int64_t)R * C;
  const int len = per_row ? R : C;
  const __nv_bfloat16* vp = v + (int64_t)slot_of[mat] * numel;
  const float* mp = mult + (int64_t)mat * len;
  float* p = params[mat];
  __nv_bfloat16* sh = shadows ? shadows[mat] : nullptr;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < numel; i += (int64_t)gridDim.x * blockDim.x * 4) {
    const int row = numel <= 0x7fffffff ? (int)((uint32_t)i / (uint32_t)C) : (int)(i / C), col = (int)(i - (int64_t)row * C);
    const float4 vv = load4<__nv_bfloat16>(vp + i);
    float4 pv = *reinterpret_cast<float4*>(p + i);
    float m0, m1, m2, m3;
    if (per_row) {
      m0 = m1 = m2 = m3 = mp[row];
    } else {
      const float4 mm = *reinterpret_cast<const float4*>(mp + col);
      m0 = mm.x; m1 = mm.y; m2 = mm.z; m3 = mm.w;
    }
    const float u0 = vv.x * m0, u1 = vv.y * m1, u2 = vv.z * m2, u3 = vv.w * m3;
    if (mode == 1) {
      pv.x *= 1.f - decay; pv.y *= 1.f - decay; pv.z *= 1.f - decay; pv.w *= 1.f - decay;
    } else if (mode == 2) {
      if (signbit(u0) == signbit(pv.x)) pv.x -= decay * pv.x;
      if (signbit(u1) == signbit(pv.y)) pv.y -= decay * pv.y;
      if (signbit(u2) == signbit(pv.z)) pv.z -= decay * pv.z;
      if (signbit(u3) == signbit(pv.w)) pv.w -= decay * pv.w;
    }
    pv.x -= lr_eff * u0; pv.y -= lr_eff * u1; pv.z -= lr_eff * u2; pv.w -= lr_eff * u3;
    *reinterpret_cast<float4*>(p + i) = pv;
    if (sh != nullptr) store4<__nv_bfloat16>(sh + i, pv);
  }
}

constexpr int kMuonChunk = 32 * 1024;

int muon_chunks_per_matrix(int64_t numel) { return (int)((numel + kMuonChunk - 1) / kMuonChunk); }

void muon_momentum(const float* const* grads, const int32_t* slot_of, float* momentum, void* xout, float* partial, int n_mats,
                   int64_t numel, float mu, float eps, cudaStream_t st) {
  if (n_mats == 0) return;
  const int cpm = muon_chunks_per_matrix(numel);
  muon_momentum_kernel<<<n_mats * cpm, 256, 0, st>>>(grads, slot_of, momentum, (__nv_bfloat16*)xout, partial, numel, cpm, kMuonChunk, mu);
  muon_fro_scale_kernel<<<n_mats * cpm, 256, 0, st>>>(slot_of, (__nv_bfloat16*)xout, partial, numel, cpm, kMuonChunk, eps);
}

void muon_tail(const void* v, const int32_t* slot_of, float* second, float* sq, float* mult, float* const* params,
               void* const* shadows, float* sq_sum_out, int n_mats, int R, int C, float beta2, int normalize, float lr_eff,
               float decay, int mode, cudaStream_t st) {
  if (n_mats == 0) return;
  const bool per_row = R >= C;
  const __nv_bfloat16* vp = (const __nv_bfloat16*)v;
  if (per_row) {
    dim3 grid((R + 7) / 8, n_mats);
    muon_rowsq_kernel<<<grid, 256, 0, st>>>(vp, slot_of, sq, R, C);
  } else {
    dim3 grid((C + 255) / 256, n_mats);
    muon_colsq_kernel<<<grid, 256, 0, st>>>(vp, slot_of, sq, R, C);
  }
  const int len = per_row ? R : C;
  muon_plan_kernel<<<n_mats, 256, 0, st>>>(sq, second, mult, sq_sum_out, len, per_row ? C : R, beta2, normalize);
  const int64_t numel = (int64_t)R * C;
  int gx = (int)((numel / 4 + 255) / 256);
  if (gx > 512) gx = 512;
  dim3 grid(gx, n_mats);
  muon_apply_kernel<<<grid, 256, 0, st>>>(vp, slot_of, mult, params, (__nv_bfloat16* const*)shadows, R, C, per_row ? 1 : 0, lr_eff,
                                          decay, mode);
}

}  // namespace seg
