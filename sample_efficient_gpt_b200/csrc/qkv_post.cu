// Post-processing of the packed qkv projection, forward and backward:
//   split Q | K | V, rotary embedding (split-half, fp32) on q and k, per-token-and-head RMS normalisation of
//   q and k (eps 1e-6, q times a learnable scalar), value residual v' = s*c*(a1*v + a2*v1), c = rsqrt(a1^2+a2^2+1e-8).
// Reference math: transformer/rope.py:36-56, transformer/attention.py:51-63 and 222-228.
// Layouts: qkv [T, (H+2Hkv)*hd]; q [T,H,hd]; k, v, v1 [T,Hkv,hd] (token-major, what the attention kernel reads).
// One CTA per token, one warp per head slot; a lane owns the rotary pairs (l, l+hd/2) so the rotation needs no
// shuffles.  The backward recomputes the rotation and the norms from qkv (nothing extra is saved by the forward)
// and reduces the four scalar gradients deterministically: per-CTA partials, then a single-CTA finalize.
#include "common.cuh"
#include "kernels.h"

namespace seg {

constexpr float kQkEps = 1e-6f;
constexpr float kMixEps = 1e-8f;

template <typename T, int HD>
__global__ void __launch_bounds__(1024) qkv_post_fwd_kernel(const T* __restrict__ qkv, const T* __restrict__ v1, T* __restrict__ q,
                                                          T* __restrict__ k, T* __restrict__ v, QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int PP = (HALF + 31) / 32;  // rotary pairs per lane
  const int t = blockIdx.x;
  const int s = t % p.S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int nslots = p.H + 2 * p.Hkv;
  const int row_w = nslots * HD;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  for (int slot = warp; slot < nslots; slot += nwarps) {
    const T* src = qkv + (size_t)t * row_w + (size_t)slot * HD;
    float x1[PP], x2[PP];
    bool live[PP];
#pragma unroll
    for (int j = 0; j < PP; ++j) {
      const int i = lane + 32 * j;
      live[j] = i < HALF;
      x1[j] = live[j] ? to_f<T>(src[i]) : 0.f;
      x2[j] = live[j] ? to_f<T>(src[i + HALF]) : 0.f;
    }
    if (slot < p.H + p.Hkv) {  // q or k head: rotate, normalise
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        if (live[j]) {
          const float cs = p.cos[(size_t)s * HALF + i], sn = p.sin[(size_t)s * HALF + i];
          const float r1 = x1[j] * cs - x2[j] * sn, r2 = x1[j] * sn + x2[j] * cs;
          x1[j] = r1;
          x2[j] = r2;
          ss += r1 * r1 + r2 * r2;
        }
      }
      float mul = 1.f;
      if (p.qknorm) {
        ss = warp_sum(ss);
        mul = rsqrtf(ss / HD + kQkEps);
        if (slot < p.H) mul *= *p.qgain;
      }
      T* dst = (slot < p.H) ? q + ((size_t)t * p.H + slot) * HD : k + ((size_t)t * p.Hkv + (slot - p.H)) * HD;
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        if (live[j]) {
          dst[i] = from_f<T>(x1[j] * mul);
          dst[i + HALF] = from_f<T>(x2[j] * mul);
        }
      }
    } else {  // v head: value residual
      const int hv = slot - p.H - p.Hkv;
      const size_t off = ((size_t)t * p.Hkv + hv) * HD;
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        if (live[j]) {
          const float w1 = v1 ? to_f<T>(v1[off + i]) : x1[j];
          const float w2 = v1 ? to_f<T>(v1[off + i + HALF]) : x2[j];
          v[off + i] = from_f<T>(vs * c * (a1 * x1[j] + a2 * w1));
          v[off + i + HALF] = from_f<T>(vs * c * (a1 * x2[j] + a2 * w2));
        }
      }
    }
  }
}

template <typename T, typename DVT, int HD>
__global__ void __launch_bounds__(1024) qkv_post_bwd_kernel(const T* __restrict__ dq, const T* __restrict__ dk,
                                                          const DVT* __restrict__ dv, const T* __restrict__ qkv,
                                                          const T* __restrict__ v1, T* __restrict__ dqkv, float* __restrict__ dv1_out,
                                                          float* __restrict__ partial, QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int PP = (HALF + 31) / 32;
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int s = t % p.S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int nslots = p.H + 2 * p.Hkv;
  const int row_w = nslots * HD;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  const float qg = *p.qgain;
  float acc_qg = 0.f, acc_dvU = 0.f, acc_dvv = 0.f, acc_dvv1 = 0.f;  // per-thread partial sums
  for (int slot = warp; slot < nslots; slot += nwarps) {
    const T* src = qkv + (size_t)t * row_w + (size_t)slot * HD;
    T* dst = dqkv + (size_t)t * row_w + (size_t)slot * HD;
    float x1[PP], x2[PP];
    bool live[PP];
#pragma unroll
    for (int j = 0; j < PP; ++j) {
      const int i = lane + 32 * j;
      live[j] = i < HALF;
      x1[j] = live[j] ? to_f<T>(src[i]) : 0.f;
      x2[j] = live[j] ? to_f<T>(src[i + HALF]) : 0.f;
    }
    if (slot < p.H + p.Hkv) {
      const bool is_q = slot < p.H;
      const T* g = is_q ? dq + ((size_t)t * p.H + slot) * HD : dk + ((size_t)t * p.Hkv + (slot - p.H)) * HD;
      float g1[PP], g2[PP], cs[PP], sn[PP];
      float ss = 0.f, dot = 0.f;
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        cs[j] = sn[j] = g1[j] = g2[j] = 0.f;
        if (live[j]) {
          cs[j] = p.cos[(size_t)s * HALF + i];
          sn[j] = p.sin[(size_t)s * HALF + i];
          const float r1 = x1[j] * cs[j] - x2[j] * sn[j], r2 = x1[j] * sn[j] + x2[j] * cs[j];
          x1[j] = r1;
          x2[j] = r2;
          g1[j] = to_f<T>(g[i]);
          g2[j] = to_f<T>(g[i + HALF]);
          ss += r1 * r1 + r2 * r2;
          dot += r1 * g1[j] + r2 * g2[j];
        }
      }
      if (p.qknorm) {
        ss = warp_sum(ss);
        dot = warp_sum(dot);
        const float r = rsqrtf(ss / HD + kQkEps);
        const float gamma = is_q ? qg : 1.f;
        if (is_q && lane == 0) acc_qg += r * dot;
        const float ka = gamma * r, kb = gamma * r * r * r * dot / HD;
#pragma unroll
        for (int j = 0; j < PP; ++j) {
          g1[j] = ka * g1[j] - kb * x1[j];
          g2[j] = ka * g2[j] - kb * x2[j];
        }
      }
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        if (live[j]) {  // transpose rotation
          dst[i] = from_f<T>(g1[j] * cs[j] + g2[j] * sn[j]);
          dst[i + HALF] = from_f<T>(-g1[j] * sn[j] + g2[j] * cs[j]);
        }
      }
    } else {
      const int hv = slot - p.H - p.Hkv;
      const size_t off = ((size_t)t * p.Hkv + hv) * HD;
      const float kself = vs * c * (v1 ? a1 : (a1 + a2));
      const float kother = vs * c * a2;
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        const int i = lane + 32 * j;
        if (live[j]) {
          const float d1 = to_f<DVT>(dv[off + i]), d2 = to_f<DVT>(dv[off + i + HALF]);
          const float w1 = v1 ? to_f<T>(v1[off + i]) : x1[j];
          const float w2 = v1 ? to_f<T>(v1[off + i + HALF]) : x2[j];
          acc_dvU += d1 * (a1 * x1[j] + a2 * w1) + d2 * (a1 * x2[j] + a2 * w2);
          acc_dvv += d1 * x1[j] + d2 * x2[j];
          acc_dvv1 += d1 * w1 + d2 * w2;
          dst[i] = from_f<T>(kself * d1);
          dst[i + HALF] = from_f<T>(kself * d2);
          if (dv1_out != nullptr) {
            dv1_out[off + i] = kother * d1;
            dv1_out[off + i + HALF] = kother * d2;
          }
        }
      }
    }
  }
  const float s0 = block_sum(acc_qg, red);
  const float s1 = block_sum(acc_dvU, red);
  const float s2 = block_sum(acc_dvv, red);
  const float s3 = block_sum(acc_dvv1, red);
  if (threadIdx.x == 0) {
    float* o = partial + (size_t)blockIdx.x * 4;
    o[0] = s0; o[1] = s1; o[2] = s2; o[3] = s3;
  }
}

// scalars = {dqgain, dalpha1, dalpha2, dvscale} from the per-CTA partial sums {sum dq^.q_rot.r, sum dv.U, sum dv.v, sum dv.v1}
__global__ void __launch_bounds__(256) qkv_post_finalize(const float* __restrict__ partial, int n, float* __restrict__ scalars,
                                                       QkvPostParams p) {
  __shared__ float red[32];
  float a[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] += partial[(size_t)i * 4 + j];
  }
  float tot[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) tot[j] = block_sum(a[j], red);
  if (threadIdx.x == 0) {
    const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
    const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
    scalars[0] = tot[0];
    scalars[1] = vs * c * tot[2] - a1 * c * c * c * vs * tot[1];
    scalars[2] = vs * c * tot[3] - a2 * c * c * c * vs * tot[1];
    scalars[3] = c * tot[1];
  }
}

static int post_threads(const QkvPostParams& p) {
  int slots = p.H + 2 * p.Hkv;
  return 32 * (slots < 32 ? slots : 32);
}

void qkv_post_fwd(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  const int T = p.B * p.S, threads = post_threads(p);
#define SEG_POST(TY, HD) qkv_post_fwd_kernel<TY, HD><<<T, threads, 0, st>>>((const TY*)qkv, (const TY*)v1, (TY*)q, (TY*)k, (TY*)v, p)
  if (bf16) { if (p.hd == 64) SEG_POST(__nv_bfloat16, 64); else if (p.hd == 128) SEG_POST(__nv_bfloat16, 128); else SEG_POST(__nv_bfloat16, 32); }
  else { if (p.hd == 64) SEG_POST(float, 64); else if (p.hd == 128) SEG_POST(float, 128); else SEG_POST(float, 32); }
#undef SEG_POST
}

void qkv_post_bwd(const void* dq, const void* dk, const void* dv, bool dv_is_f32, const void* qkv, const void* v1, void* dqkv,
                  float* dv1_out, float* scalars, float* partial, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  const int T = p.B * p.S, threads = post_threads(p);
#define SEG_POSTB(TY, DV, HD)                                                                                                 \
  qkv_post_bwd_kernel<TY, DV, HD><<<T, threads, 0, st>>>((const TY*)dq, (const TY*)dk, (const DV*)dv, (const TY*)qkv, (const TY*)v1, \
                                                         (TY*)dqkv, dv1_out, partial, p)
#define SEG_POSTB_HD(TY, DV)                                                     \
  if (p.hd == 64) SEG_POSTB(TY, DV, 64); else if (p.hd == 128) SEG_POSTB(TY, DV, 128); else SEG_POSTB(TY, DV, 32)
  if (bf16) {
    if (dv_is_f32) { SEG_POSTB_HD(__nv_bfloat16, float); } else { SEG_POSTB_HD(__nv_bfloat16, __nv_bfloat16); }
  } else {
    SEG_POSTB_HD(float, float);
  }
#undef SEG_POSTB_HD
#undef SEG_POSTB
  qkv_post_finalize<<<1, 256, 0, st>>>(partial, T, scalars, p);
}

}  // namespace seg
