// Post-processing of the packed qkv projection, forward and backward:
//   split Q | K | V, rotary embedding (split-half, fp32) on q and k, per-token-and-head RMS normalisation of
//   q and k (eps 1e-6, q times a learnable scalar), value residual v' = s*c*(a1*v + a2*v1), c = rsqrt(a1^2+a2^2+1e-8).
// Reference math: transformer/rope.py:36-56, transformer/attention.py:51-63 and 222-228.
// Layouts: qkv [T, (H+2Hkv)*hd]; q [T,H,hd]; k, v, v1 [T,Hkv,hd] (token-major, what the attention kernel reads).
// Work item = 8 rotary pairs of one (token, head slot): a thread loads x[8j..8j+8) and x[hd/2+8j..] with 16-byte
// accesses, hd/16 neighbouring lanes share a head and combine their sums of squares with shuffles.  The backward
// recomputes rotation and norms from qkv (the forward saves nothing extra) and reduces the four scalar gradients
// deterministically: per-CTA partials, then a single-CTA finalize.
#include "common.cuh"
#include "kernels.h"

namespace seg {

constexpr float kQkEps = 1e-6f;
constexpr float kMixEps = 1e-8f;
constexpr int kPostThreads = 256;

// Sum over the LPH neighbouring lanes that share a head.  Only those lanes are named in the mask: lanes of one
// head always take the same branch, lanes of different heads in a warp may not (q/k heads vs v heads).
template <int LPH>
__device__ __forceinline__ float group_sum(float v) {
  const unsigned lane = threadIdx.x & 31u;
  const unsigned mask = (LPH == 32) ? 0xffffffffu : (((1u << LPH) - 1u) << (lane & ~(unsigned)(LPH - 1)));
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}

template <typename T, int HD>
__global__ void __launch_bounds__(kPostThreads, 4) qkv_post_fwd_kernel(const T* __restrict__ qkv, const T* __restrict__ v1,
                                                                  T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                                  QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int LPH = HALF / 8;  // lanes per head
  const int nslots = p.H + 2 * p.Hkv;
  const int64_t total = (int64_t)p.B * p.S * nslots * LPH;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (total + stride - 1) / stride;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  const float qg = *p.qgain;
  const int pos_off = p.pos != nullptr ? *p.pos : 0;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (int64_t it = 0; it < rounds; ++it, idx += stride) {
    const bool live = idx < total;
    int sub, slot, s;
    int64_t t;
    if (total <= 0x7fffffffLL) {  // 32-bit index arithmetic (uniform branch): 64-bit divisions by run-time values dominate otherwise
      const uint32_t i32 = live ? (uint32_t)idx : 0u;
      sub = (int)(i32 % LPH);
      const uint32_t sg = i32 / LPH;
      slot = (int)(sg % (uint32_t)nslots);
      const uint32_t t32 = sg / (uint32_t)nslots;
      s = (int)(t32 % (uint32_t)p.S) + pos_off;
      t = t32;
    } else {
      sub = (int)(idx % LPH);
      const int64_t sg = live ? idx / LPH : 0;
      slot = (int)(sg % nslots);
      t = sg / nslots;
      s = (int)(t % p.S) + pos_off;
    }
    float x1[8], x2[8];
    if (live) {
      const T* src = qkv + (size_t)t * p.qkv_stride + (size_t)slot * HD + sub * 8;
      load8<T>(src, x1);
      load8<T>(src + HALF, x2);
    }
    if (slot < p.H + p.Hkv) {
      float ss = 0.f;
      if (live) {
        float cs[8], sn[8];
        load8<float>(p.cos + (size_t)s * HALF + sub * 8, cs);
        load8<float>(p.sin + (size_t)s * HALF + sub * 8, sn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float r1 = x1[j] * cs[j] - x2[j] * sn[j], r2 = x1[j] * sn[j] + x2[j] * cs[j];
          x1[j] = r1;
          x2[j] = r2;
          ss += r1 * r1 + r2 * r2;
        }
      }
      float mul = 1.f;
      if (p.qknorm) {
        ss = group_sum<LPH>(ss);
        mul = rsqrtf(ss / HD + kQkEps);
        if (slot < p.H) mul *= qg;
      }
      if (live) {
        T* dst = (slot < p.H) ? q + ((size_t)t * p.H + slot) * HD : k + ((size_t)t * p.Hkv + (slot - p.H)) * HD;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          x1[j] *= mul;
          x2[j] *= mul;
        }
        store8<T>(dst + sub * 8, x1);
        store8<T>(dst + HALF + sub * 8, x2);
      }
    } else {
      if (live) {
        const size_t off = ((size_t)t * p.Hkv + (slot - p.H - p.Hkv)) * HD + sub * 8;
        float w1[8], w2[8];
        if (v1 != nullptr) {
          load8<T>(v1 + off, w1);
          load8<T>(v1 + off + HALF, w2);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float u1 = v1 ? w1[j] : x1[j], u2 = v1 ? w2[j] : x2[j];
          x1[j] = vs * c * (a1 * x1[j] + a2 * u1);
          x2[j] = vs * c * (a1 * x2[j] + a2 * u2);
        }
        store8<T>(v + off, x1);
        store8<T>(v + off + HALF, x2);
      }
    }
  }
}

template <typename T, typename DVT, int HD>
__global__ void __launch_bounds__(kPostThreads) qkv_post_bwd_kernel(const T* __restrict__ dq, const T* __restrict__ dk,
                                                                  const DVT* __restrict__ dv, const T* __restrict__ qkv,
                                                                  const T* __restrict__ v1, T* __restrict__ dqkv,
                                                                  float* __restrict__ dv1_out, float* __restrict__ partial,
                                                                  QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int LPH = HALF / 8;
  __shared__ float red[32];
  const int nslots = p.H + 2 * p.Hkv;
  const int64_t total = (int64_t)p.B * p.S * nslots * LPH;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (total + stride - 1) / stride;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  const float qg = *p.qgain;
  const int pos_off = p.pos != nullptr ? *p.pos : 0;
  float acc_qg = 0.f, acc_dvU = 0.f, acc_dvv = 0.f, acc_dvv1 = 0.f;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (int64_t it = 0; it < rounds; ++it, idx += stride) {
    const bool live = idx < total;
    int sub, slot, s;
    int64_t t;
    if (total <= 0x7fffffffLL) {  // 32-bit index arithmetic (uniform branch): 64-bit divisions by run-time values dominate otherwise
      const uint32_t i32 = live ? (uint32_t)idx : 0u;
      sub = (int)(i32 % LPH);
      const uint32_t sg = i32 / LPH;
      slot = (int)(sg % (uint32_t)nslots);
      const uint32_t t32 = sg / (uint32_t)nslots;
      s = (int)(t32 % (uint32_t)p.S) + pos_off;
      t = t32;
    } else {
      sub = (int)(idx % LPH);
      const int64_t sg = live ? idx / LPH : 0;
      slot = (int)(sg % nslots);
      t = sg / nslots;
      s = (int)(t % p.S) + pos_off;
    }
    const size_t row_off = (size_t)t * p.qkv_stride + (size_t)slot * HD + sub * 8;
    float x1[8], x2[8];
    if (live) {
      load8<T>(qkv + row_off, x1);
      load8<T>(qkv + row_off + HALF, x2);
    }
    if (slot < p.H + p.Hkv) {
      const bool is_q = slot < p.H;
      float g1[8], g2[8], cs[8], sn[8];
      float ss = 0.f, dot = 0.f;
      if (live) {
        const T* g = is_q ? dq + ((size_t)t * p.H + slot) * HD + sub * 8 : dk + ((size_t)t * p.Hkv + (slot - p.H)) * HD + sub * 8;
        load8<T>(g, g1);
        load8<T>(g + HALF, g2);
        load8<float>(p.cos + (size_t)s * HALF + sub * 8, cs);
        load8<float>(p.sin + (size_t)s * HALF + sub * 8, sn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float r1 = x1[j] * cs[j] - x2[j] * sn[j], r2 = x1[j] * sn[j] + x2[j] * cs[j];
          x1[j] = r1;
          x2[j] = r2;
          ss += r1 * r1 + r2 * r2;
          dot += r1 * g1[j] + r2 * g2[j];
        }
      }
      if (p.qknorm) {
        ss = group_sum<LPH>(ss);
        dot = group_sum<LPH>(dot);
        const float r = rsqrtf(ss / HD + kQkEps);
        const float gamma = is_q ? qg : 1.f;
        if (live && is_q && sub == 0) acc_qg += r * dot;
        const float ka = gamma * r, kb = gamma * r * r * r * dot / HD;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g1[j] = ka * g1[j] - kb * x1[j];
          g2[j] = ka * g2[j] - kb * x2[j];
        }
      }
      if (live) {
        float o1[8], o2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // transpose of the rotation
          o1[j] = g1[j] * cs[j] + g2[j] * sn[j];
          o2[j] = -g1[j] * sn[j] + g2[j] * cs[j];
        }
        store8<T>(dqkv + row_off, o1);
        store8<T>(dqkv + row_off + HALF, o2);
      }
    } else {
      if (live) {
        const size_t off = ((size_t)t * p.Hkv + (slot - p.H - p.Hkv)) * HD + sub * 8;
        const float kself = vs * c * (v1 ? a1 : (a1 + a2));
        const float kother = vs * c * a2;
        float d1[8], d2[8], w1[8], w2[8];
        load8<DVT>(dv + off, d1);
        load8<DVT>(dv + off + HALF, d2);
        if (v1 != nullptr) {
          load8<T>(v1 + off, w1);
          load8<T>(v1 + off + HALF, w2);
        }
        float o1[8], o2[8], e1[8], e2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float u1 = v1 ? w1[j] : x1[j], u2 = v1 ? w2[j] : x2[j];
          acc_dvU += d1[j] * (a1 * x1[j] + a2 * u1) + d2[j] * (a1 * x2[j] + a2 * u2);
          acc_dvv += d1[j] * x1[j] + d2[j] * x2[j];
          acc_dvv1 += d1[j] * u1 + d2[j] * u2;
          o1[j] = kself * d1[j];
          o2[j] = kself * d2[j];
          e1[j] = kother * d1[j];
          e2[j] = kother * d2[j];
        }
        store8<T>(dqkv + row_off, o1);
        store8<T>(dqkv + row_off + HALF, o2);
        if (dv1_out != nullptr) {
          if (p.dv1_accumulate) {  // the gradient of the first block's values gathers over all later blocks
            float b1[8], b2[8];
            load8<float>(dv1_out + off, b1);
            load8<float>(dv1_out + off + HALF, b2);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              e1[j] += b1[j];
              e2[j] += b2[j];
            }
          }
          store8<float>(dv1_out + off, e1);
          store8<float>(dv1_out + off + HALF, e2);
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

int qkv_post_bwd_grid(int64_t T, int nslots, int hd) {
  const int64_t items = T * nslots * (hd / 16);
  int64_t g = (items + kPostThreads - 1) / kPostThreads;
  return (int)(g < kQkvPostMaxGrid ? (g > 0 ? g : 1) : kQkvPostMaxGrid);
}

void qkv_post_fwd(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  const int grid = qkv_post_bwd_grid((int64_t)p.B * p.S, p.H + 2 * p.Hkv, p.hd);
#define SEG_POST(TY, HD) qkv_post_fwd_kernel<TY, HD><<<grid, kPostThreads, 0, st>>>((const TY*)qkv, (const TY*)v1, (TY*)q, (TY*)k, (TY*)v, p)
  if (bf16) { if (p.hd == 64) SEG_POST(__nv_bfloat16, 64); else if (p.hd == 128) SEG_POST(__nv_bfloat16, 128); else SEG_POST(__nv_bfloat16, 32); }
  else { if (p.hd == 64) SEG_POST(float, 64); else if (p.hd == 128) SEG_POST(float, 128); else SEG_POST(float, 32); }
#undef SEG_POST
}

void qkv_post_bwd(const void* dq, const void* dk, const void* dv, bool dv_is_f32, const void* qkv, const void* v1, void* dqkv,
                  float* dv1_out, float* scalars, float* partial, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  const int grid = qkv_post_bwd_grid((int64_t)p.B * p.S, p.H + 2 * p.Hkv, p.hd);
#define SEG_POSTB(TY, DV, HD)                                                                                                      \
  qkv_post_bwd_kernel<TY, DV, HD><<<grid, kPostThreads, 0, st>>>((const TY*)dq, (const TY*)dk, (const DV*)dv, (const TY*)qkv,       \
                                                                 (const TY*)v1, (TY*)dqkv, dv1_out, partial, p)
#define SEG_POSTB_HD(TY, DV)                                                     \
  if (p.hd == 64) SEG_POSTB(TY, DV, 64); else if (p.hd == 128) SEG_POSTB(TY, DV, 128); else SEG_POSTB(TY, DV, 32)
  if (bf16) {
    if (dv_is_f32) { SEG_POSTB_HD(__nv_bfloat16, float); } else { SEG_POSTB_HD(__nv_bfloat16, __nv_bfloat16); }
  } else {
    SEG_POSTB_HD(float, float);
  }
#undef SEG_POSTB_HD
#undef SEG_POSTB
  qkv_post_finalize<<<1, 256, 0, st>>>(partial, grid, scalars, p);
}

}  // namespace seg
