// Post-processing of the packed qkv projection, forward and backward:
//   split Q | K | V, rotary embedding (split-half, fp32) on q and k, per-token-and-head RMS normalisation of
//   q and k (eps 1e-6, q times a learnable scalar), value residual v' = s*c*(a1*v + a2*v1), c = rsqrt(a1^2+a2^2+1e-8).
// Reference math: transformer/rope.py:36-56, transformer/attention.py:51-63 and 222-228.
// Layouts: qkv [T, (H+2Hkv)*hd]; q [T,H,hd]; k, v, v1 [T,Hkv,hd] (token-major, what the attention kernel reads).
// Work item = 8 rotary pairs of up to six head slots of one token: a thread loads x[8j..8j+8) and x[hd/2+8j..] of each
// with 16-byte accesses, hd/16 neighbouring lanes share a head and combine their sums of squares with shuffles.  The backward
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

// Decomposition of a work-item index: item = ((token * ng) + group) * LPH + sub.  A thread serves head slots group,
// group + ng, group + 2 ng, ... of its token, so the rotation table row (64 bytes per thread) and the index arithmetic are
// paid once per kSlotsPerItem heads instead of once per head: that, not DRAM, bounded these kernels.
constexpr int kSlotsPerItem = 6;
constexpr int kSlotBatch = 3;     // forward: slots whose loads are issued together before any of them is used
constexpr int kSlotBatchBwd = 2;  // backward (twice the registers per slot)
__host__ __device__ inline int qkv_post_groups(int nslots) { return (nslots + kSlotsPerItem - 1) / kSlotsPerItem; }

struct PostItem {
  int sub, grp, s;
  int64_t t;
};
template <int LPH>
__device__ __forceinline__ PostItem post_item(int64_t idx, bool live, int64_t total, int ng, int S, int pos_off) {
  PostItem it;
  if (total <= 0x7fffffffLL) {  // 32-bit index arithmetic (uniform branch): 64-bit divisions by run-time values are slow
    const uint32_t i32 = live ? (uint32_t)idx : 0u;
    it.sub = (int)(i32 % LPH);
    const uint32_t sg = i32 / LPH;
    it.grp = (int)(sg % (uint32_t)ng);
    const uint32_t t32 = sg / (uint32_t)ng;
    it.s = (int)(t32 % (uint32_t)S) + pos_off;
    it.t = t32;
  } else {
    const int64_t i64 = live ? idx : 0;
    it.sub = (int)(i64 % LPH);
    const int64_t sg = i64 / LPH;
    it.grp = (int)(sg % ng);
    it.t = sg / ng;
    it.s = (int)(it.t % S) + pos_off;
  }
  return it;
}

template <typename T, int HD>
__global__ void __launch_bounds__(kPostThreads, 2) qkv_post_fwd_kernel(const T* __restrict__ qkv, const T* __restrict__ v1,
                                                                  T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                                  QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int LPH = HALF / 8;  // lanes per head
  const int nslots = p.H + 2 * p.Hkv, nrot = p.H + p.Hkv;
  const int ng = qkv_post_groups(nslots);
  const int iters = (nslots + ng - 1) / ng;
  const int64_t total = (int64_t)p.B * p.S * ng * LPH;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (total + stride - 1) / stride;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  const float qg = *p.qgain;
  const int pos_off = p.pos != nullptr ? *p.pos : 0;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (int64_t round = 0; round < rounds; ++round, idx += stride) {
    const bool live = idx < total;  // the LPH lanes of a head are live together (total and stride are multiples of LPH)
    if (!live) continue;
    const PostItem it = post_item<LPH>(idx, live, total, ng, p.S, pos_off);
    float cs[8], sn[8];
    load8<float>(p.cos + (size_t)it.s * HALF + it.sub * 8, cs);
    load8<float>(p.sin + (size_t)it.s * HALF + it.sub * 8, sn);
    const T* row = qkv + (size_t)it.t * p.qkv_stride + it.sub * 8;
    for (int i0 = 0; i0 < iters; i0 += kSlotBatch) {
      float x1[kSlotBatch][8], x2[kSlotBatch][8];
#pragma unroll
      for (int b = 0; b < kSlotBatch; ++b) {
        const int slot = it.grp + (i0 + b) * ng;
        if (i0 + b < iters && slot < nslots) {
          load8<T>(row + (size_t)slot * HD, x1[b]);
          load8<T>(row + (size_t)slot * HD + HALF, x2[b]);
        }
      }
#pragma unroll
      for (int b = 0; b < kSlotBatch; ++b) {
        const int slot = it.grp + (i0 + b) * ng;
        if (i0 + b >= iters || slot >= nslots) continue;
        if (slot < nrot) {
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float r1 = x1[b][j] * cs[j] - x2[b][j] * sn[j], r2 = x1[b][j] * sn[j] + x2[b][j] * cs[j];
            x1[b][j] = r1;
            x2[b][j] = r2;
            ss += r1 * r1 + r2 * r2;
          }
          float mul = 1.f;
          if (p.qknorm) {
            ss = group_sum<LPH>(ss);
            mul = rsqrtf(ss / HD + kQkEps);
            if (slot < p.H) mul *= qg;
          }
          T* dst = (slot < p.H) ? q + ((size_t)it.t * p.H + slot) * HD : k + ((size_t)it.t * p.Hkv + (slot - p.H)) * HD;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            x1[b][j] *= mul;
            x2[b][j] *= mul;
          }
          store8<T>(dst + it.sub * 8, x1[b]);
          store8<T>(dst + HALF + it.sub * 8, x2[b]);
        } else {
          const size_t off = ((size_t)it.t * p.Hkv + (slot - nrot)) * HD + it.sub * 8;
          float w1[8], w2[8];
          if (v1 != nullptr) {
            load8<T>(v1 + off, w1);
            load8<T>(v1 + off + HALF, w2);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float u1 = v1 ? w1[j] : x1[b][j], u2 = v1 ? w2[j] : x2[b][j];
            x1[b][j] = vs * c * (a1 * x1[b][j] + a2 * u1);
            x2[b][j] = vs * c * (a1 * x2[b][j] + a2 * u2);
          }
          store8<T>(v + off, x1[b]);
          store8<T>(v + off + HALF, x2[b]);
        }
      }
    }
  }
}

template <typename T, typename DVT, int HD>
__global__ void __launch_bounds__(kPostThreads, 2) qkv_post_bwd_kernel(const T* __restrict__ dq, const T* __restrict__ dk,
                                                                  const DVT* __restrict__ dv, const T* __restrict__ qkv,
                                                                  const T* __restrict__ v1, T* __restrict__ dqkv,
                                                                  float* __restrict__ dv1_out, float* __restrict__ partial,
                                                                  QkvPostParams p) {
  constexpr int HALF = HD / 2;
  constexpr int LPH = HALF / 8;
  __shared__ float red[32];
  const int nslots = p.H + 2 * p.Hkv, nrot = p.H + p.Hkv;
  const int ng = qkv_post_groups(nslots);
  const int iters = (nslots + ng - 1) / ng;
  const int64_t total = (int64_t)p.B * p.S * ng * LPH;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (total + stride - 1) / stride;
  const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
  const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
  const float qg = *p.qgain;
  const int pos_off = p.pos != nullptr ? *p.pos : 0;
  const float kself = vs * c * (v1 ? a1 : (a1 + a2));
  const float kother = vs * c * a2;
  float acc_qg = 0.f, acc_dvU = 0.f, acc_dvv = 0.f, acc_dvv1 = 0.f;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (int64_t round = 0; round < rounds; ++round, idx += stride) {
    const bool live = idx < total;
    if (!live) continue;
    const PostItem it = post_item<LPH>(idx, live, total, ng, p.S, pos_off);
    float cs[8], sn[8];
    load8<float>(p.cos + (size_t)it.s * HALF + it.sub * 8, cs);
    load8<float>(p.sin + (size_t)it.s * HALF + it.sub * 8, sn);
    const size_t row0 = (size_t)it.t * p.qkv_stride + it.sub * 8;
    for (int i0 = 0; i0 < iters; i0 += kSlotBatchBwd) {
      float x1[kSlotBatchBwd][8], x2[kSlotBatchBwd][8], g1[kSlotBatchBwd][8], g2[kSlotBatchBwd][8];
#pragma unroll
      for (int b = 0; b < kSlotBatchBwd; ++b) {
        const int slot = it.grp + (i0 + b) * ng;
        if (i0 + b < iters && slot < nslots) {
          load8<T>(qkv + row0 + (size_t)slot * HD, x1[b]);
          load8<T>(qkv + row0 + (size_t)slot * HD + HALF, x2[b]);
          if (slot < nrot) {
            const T* g = slot < p.H ? dq + ((size_t)it.t * p.H + slot) * HD + it.sub * 8
                                    : dk + ((size_t)it.t * p.Hkv + (slot - p.H)) * HD + it.sub * 8;
            load8<T>(g, g1[b]);
            load8<T>(g + HALF, g2[b]);
          } else {
            const size_t off = ((size_t)it.t * p.Hkv + (slot - nrot)) * HD + it.sub * 8;
            load8<DVT>(dv + off, g1[b]);
            load8<DVT>(dv + off + HALF, g2[b]);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < kSlotBatchBwd; ++b) {
        const int slot = it.grp + (i0 + b) * ng;
        if (i0 + b >= iters || slot >= nslots) continue;
        const size_t row_off = row0 + (size_t)slot * HD;
        if (slot < nrot) {
          const bool is_q = slot < p.H;
          float ss = 0.f, dot = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float r1 = x1[b][j] * cs[j] - x2[b][j] * sn[j], r2 = x1[b][j] * sn[j] + x2[b][j] * cs[j];
            x1[b][j] = r1;
            x2[b][j] = r2;
            ss += r1 * r1 + r2 * r2;
            dot += r1 * g1[b][j] + r2 * g2[b][j];
          }
          if (p.qknorm) {
            ss = group_sum<LPH>(ss);
            dot = group_sum<LPH>(dot);
            const float r = rsqrtf(ss / HD + kQkEps);
            const float gamma = is_q ? qg : 1.f;
            if (is_q && it.sub == 0) acc_qg += r * dot;
            const float ka = gamma * r, kb = gamma * r * r * r * dot / HD;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              g1[b][j] = ka * g1[b][j] - kb * x1[b][j];
              g2[b][j] = ka * g2[b][j] - kb * x2[b][j];
            }
          }
          float o1[8], o2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // transpose of the rotation
            o1[j] = g1[b][j] * cs[j] + g2[b][j] * sn[j];
            o2[j] = -g1[b][j] * sn[j] + g2[b][j] * cs[j];
          }
          store8<T>(dqkv + row_off, o1);
          store8<T>(dqkv + row_off + HALF, o2);
        } else {
          const size_t off = ((size_t)it.t * p.Hkv + (slot - nrot)) * HD + it.sub * 8;
          float w1[8], w2[8];
          if (v1 != nullptr) {
            load8<T>(v1 + off, w1);
            load8<T>(v1 + off + HALF, w2);
          }
          float o1[8], o2[8], e1[8], e2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d1 = g1[b][j], d2 = g2[b][j];
            const float u1 = v1 ? w1[j] : x1[b][j], u2 = v1 ? w2[j] : x2[b][j];
            acc_dvU += d1 * (a1 * x1[b][j] + a2 * u1) + d2 * (a1 * x2[b][j] + a2 * u2);
            acc_dvv += d1 * x1[b][j] + d2 * x2[b][j];
            acc_dvv1 += d1 * u1 + d2 * u2;
            o1[j] = kself * d1;
            o2[j] = kself * d2;
            e1[j] = kother * d1;
            e2[j] = kother * d2;
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
  const int64_t items = T * qkv_post_groups(nslots) * (hd / 16);
  int64_t g = (items + kPostThreads - 1) / kPostThreads;
  return (int)(g < kQkvPostMaxGrid ? (g > 0 ? g : 1) : kQkvPostMaxGrid);
}

void qkv_post_fwd(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  if (qkv_post_fwd_tile(qkv, v1, q, k, v, p, bf16, st)) return;
  const int grid = qkv_post_bwd_grid((int64_t)p.B * p.S, p.H + 2 * p.Hkv, p.hd);
#define SEG_POST(TY, HD) qkv_post_fwd_kernel<TY, HD><<<grid, kPostThreads, 0, st>>>((const TY*)qkv, (const TY*)v1, (TY*)q, (TY*)k, (TY*)v, p)
  if (bf16) { if (p.hd == 64) SEG_POST(__nv_bfloat16, 64); else if (p.hd == 128) SEG_POST(__nv_bfloat16, 128); else SEG_POST(__nv_bfloat16, 32); }
  else { if (p.hd == 64) SEG_POST(float, 64); else if (p.hd == 128) SEG_POST(float, 128); else SEG_POST(float, 32); }
#undef SEG_POST
}

void qkv_post_bwd(const void* dq, const void* dk, const void* dv, bool dv_is_f32, const void* qkv, const void* v1, void* dqkv,
                  float* dv1_out, float* scalars, float* partial, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  const int grid = qkv_post_bwd_grid((int64_t)p.B * p.S, p.H + 2 * p.Hkv, p.hd);
  if (!dv_is_f32) {
    const int rows = qkv_post_bwd_tile(dq, dk, dv, qkv, v1, dqkv, dv1_out, partial, grid, p, bf16, st);
    if (rows > 0) {
      qkv_post_finalize<<<1, 256, 0, st>>>(partial, rows, scalars, p);
      return;
    }
  }
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
