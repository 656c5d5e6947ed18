// Fused residual-add + RMSNorm (with LayerNorm-scaling and a kurtosis side output), forward and backward.
//
// forward : x = res + delta (fp32);  y = x * rsqrt(mean(x^2)+eps) * gain * scale  (bf16 or fp32);
//           rstd per row;  kurt += sum_rows mean(x^4)/max(mean(x^2),1e-8)^2   (optional)
// backward: m = dy*gain*scale;  dx = rstd*m - rstd^3 * x * mean(m*x);  dres = dres_in + dx (fp32 and a
//           low-precision copy for the following GEMMs);  dgain = sum_rows dy * x * rstd * scale.
// One warp owns a row and keeps it in registers (d/128 float4 per lane), so every tensor is read and
// written exactly once.  dgain is reduced in two stages: per-CTA partial rows into scratch
// [gridDim.x, d], then a column reduction kernel (deterministic: no atomics).
// Math source in the reference: transformer/core.py:61-72 (forward), transformer/transformer.py:58-61 (kurtosis).
#include "common.cuh"
#include "kernels.h"

namespace seg {

template <int VPL, typename OutT>
__global__ void __launch_bounds__(256) add_rmsnorm_fwd_kernel(const float* __restrict__ res, const OutT* __restrict__ delta,
                                                            const float* __restrict__ gain, float* __restrict__ x_out,
                                                            OutT* __restrict__ y, float* __restrict__ rstd_out,
                                                            float* __restrict__ kurt, int T, int d, float scale, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float kurt_local = 0.f;
  if (row < T) {
    const float4* r4 = reinterpret_cast<const float4*>(res + (size_t)row * d);
    float4 v[VPL];
    float ss = 0.f, s4 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c4 = lane + i * 32;  // float4 index within the row
      v[i] = r4[c4];
      if (delta != nullptr) {
        const float4 dl = load4<OutT>(delta + (size_t)row * d + c4 * 4);
        v[i].x += dl.x;
        v[i].y += dl.y;
        v[i].z += dl.z;
        v[i].w += dl.w;
      }
      const float a = v[i].x * v[i].x, b = v[i].y * v[i].y, c = v[i].z * v[i].z, e = v[i].w * v[i].w;
      ss += a + b + c + e;
      s4 += a * a + b * b + c * c + e * e;
    }
    ss = warp_sum(ss);
    const float ms = ss / d;
    const float rstd = rsqrtf(ms + eps);
    if (kurt != nullptr) {
      s4 = warp_sum(s4);
      const float m2 = fmaxf(ms, 1e-8f);
      kurt_local = (s4 / d) / (m2 * m2);
    }
    if (lane == 0) rstd_out[row] = rstd;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c4 = lane + i * 32;
      if (x_out != nullptr) reinterpret_cast<float4*>(x_out + (size_t)row * d)[c4] = v[i];
      const float4 g = g4[c4];
      const float k = rstd * scale;
      store4<OutT>(y + (size_t)row * d + c4 * 4, make_float4(v[i].x * k * g.x, v[i].y * k * g.y, v[i].z * k * g.z, v[i].w * k * g.w));
    }
  }
  if (kurt != nullptr) {
    __shared__ float red[32];
    float tot = (lane == 0) ? kurt_local : 0.f;
    tot = block_sum(tot, red);
    if (threadIdx.x == 0) atomicAdd(kurt, tot);
  }
}

// Generic width (d % 4 == 0 only): re-reads the row instead of holding it in registers.
template <typename OutT>
__global__ void __launch_bounds__(256) add_rmsnorm_fwd_generic(const float* __restrict__ res, const OutT* __restrict__ delta,
                                                             const float* __restrict__ gain, float* __restrict__ x_out,
                                                             OutT* __restrict__ y, float* __restrict__ rstd_out,
                                                             float* __restrict__ kurt, int T, int d, float scale, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float kurt_local = 0.f;
  if (row < T) {
    const float* r = res + (size_t)row * d;
    const OutT* dp = delta ? delta + (size_t)row * d : nullptr;
    float ss = 0.f, s4 = 0.f;
    for (int c = lane; c < d; c += 32) {
      float v = r[c] + (dp ? to_f<OutT>(dp[c]) : 0.f);
      ss += v * v;
      s4 += v * v * v * v;
    }
    ss = warp_sum(ss);
    s4 = warp_sum(s4);
    const float ms = ss / d, rstd = rsqrtf(ms + eps);
    const float m2 = fmaxf(ms, 1e-8f);
    kurt_local = (s4 / d) / (m2 * m2);
    if (lane == 0) rstd_out[row] = rstd;
    for (int c = lane; c < d; c += 32) {
      float v = r[c] + (dp ? to_f<OutT>(dp[c]) : 0.f);
      if (x_out) x_out[(size_t)row * d + c] = v;
      y[(size_t)row * d + c] = from_f<OutT>(v * rstd * scale * gain[c]);
    }
  }
  if (kurt != nullptr) {
    __shared__ float red[32];
    float tot = (lane == 0) ? kurt_local : 0.f;
    tot = block_sum(tot, red);
    if (threadIdx.x == 0) atomicAdd(kurt, tot);
  }
}

template <typename OutT>
static void launch_fwd(const float* res, const OutT* delta, const float* gain, float* x_out, OutT* y, float* rstd,
                       float* kurt, int T, int d, float scale, float eps, cudaStream_t st) {
  const int wpb = 8;
  dim3 grid((T + wpb - 1) / wpb), block(wpb * 32);
#define SEG_CASE(V)                                                                                              \
  case V:                                                                                                        \
    add_rmsnorm_fwd_kernel<V, OutT><<<grid, block, 0, st>>>(res, delta, gain, x_out, y, rstd, kurt, T, d, scale, eps); \
    return;
  if (d % 128 == 0) {
    switch (d / 128) {
      SEG_CASE(1) SEG_CASE(2) SEG_CASE(3) SEG_CASE(4) SEG_CASE(6) SEG_CASE(8) SEG_CASE(9) SEG_CASE(12) SEG_CASE(16)
      default: break;
    }
  }
#undef SEG_CASE
  add_rmsnorm_fwd_generic<OutT><<<grid, block, 0, st>>>(res, delta, gain, x_out, y, rstd, kurt, T, d, scale, eps);
}

void add_rmsnorm_fwd(const float* res, const void* delta, const float* gain, float* x_out, void* y, float* rstd, float* kurt,
                     int T, int d, float scale, float eps, bool bf16, cudaStream_t st) {
  if (bf16)
    launch_fwd<__nv_bfloat16>(res, (const __nv_bfloat16*)delta, gain, x_out, (__nv_bfloat16*)y, rstd, kurt, T, d, scale, eps, st);
  else
    launch_fwd<float>(res, (const float*)delta, gain, x_out, (float*)y, rstd, kurt, T, d, scale, eps, st);
}

// ---------------------------------------------------------------------------------------------- backward
// Grid-stride over rows by warp; lane keeps its dgain columns in registers across rows.
template <int VPL, typename InT>
__global__ void __launch_bounds__(256) add_rmsnorm_bwd_kernel(const InT* __restrict__ dy, const float* __restrict__ dres_in,
                                                            const float* __restrict__ x, const float* __restrict__ gain,
                                                            const float* __restrict__ rstd, float* __restrict__ dres,
                                                            InT* __restrict__ dres_lp, float* __restrict__ dgain_partial,
                                                            int T, int d, float scale) {
  extern __shared__ float smem[];  // [warps_per_block][d]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int warp_global = blockIdx.x * wpb + w, total_warps = gridDim.x * wpb;
  float4 dg[VPL];
  float4 g[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    dg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    g[i] = reinterpret_cast<const float4*>(gain)[lane + i * 32];
  }
  for (int row = warp_global; row < T; row += total_warps) {
    const float r = rstd[row];
    float4 xv[VPL], m[VPL], av[VPL];
    float dot = 0.f;
    // the incoming residual gradient is needed only after the row's reduction, but its loads are issued here with the
    // others: one memory latency per row instead of two
    if (dres_in != nullptr) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) av[i] = reinterpret_cast<const float4*>(dres_in + (size_t)row * d)[lane + i * 32];
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c4 = lane + i * 32;
      xv[i] = reinterpret_cast<const float4*>(x + (size_t)row * d)[c4];
      const float4 dv = load4<InT>(dy + (size_t)row * d + c4 * 4);
      const float d0 = dv.x, d1 = dv.y, d2 = dv.z, d3 = dv.w;
      dg[i].x += d0 * xv[i].x * r;
      dg[i].y += d1 * xv[i].y * r;
      dg[i].z += d2 * xv[i].z * r;
      dg[i].w += d3 * xv[i].w * r;
      m[i] = make_float4(d0 * g[i].x * scale, d1 * g[i].y * scale, d2 * g[i].z * scale, d3 * g[i].w * scale);
      dot += m[i].x * xv[i].x + m[i].y * xv[i].y + m[i].z * xv[i].z + m[i].w * xv[i].w;
    }
    dot = warp_sum(dot);
    const float k = r * r * r * dot / d;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c4 = lane + i * 32;
      float4 o = make_float4(r * m[i].x - k * xv[i].x, r * m[i].y - k * xv[i].y, r * m[i].z - k * xv[i].z, r * m[i].w - k * xv[i].w);
      if (dres_in != nullptr) {
        o.x += av[i].x; o.y += av[i].y; o.z += av[i].z; o.w += av[i].w;
      }
      reinterpret_cast<float4*>(dres + (size_t)row * d)[c4] = o;
      store4<InT>(dres_lp + (size_t)row * d + c4 * 4, o);
    }
  }
  // CTA reduction of dgain over its warps, then one partial row per CTA
#pragma unroll
  for (int i = 0; i < VPL; ++i) reinterpret_cast<float4*>(smem + (size_t)w * d)[lane + i * 32] = dg[i];
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float s = 0.f;
    for (int ww = 0; ww < wpb; ++ww) s += smem[(size_t)ww * d + c];
    dgain_partial[(size_t)blockIdx.x * d + c] = s * scale;
  }
}

template <typename InT>
__global__ void __launch_bounds__(256) add_rmsnorm_bwd_generic(const InT* __restrict__ dy, const float* __restrict__ dres_in,
                                                             const float* __restrict__ x, const float* __restrict__ gain,
                                                             const float* __restrict__ rstd, float* __restrict__ dres,
                                                             InT* __restrict__ dres_lp, float* __restrict__ dgain_partial,
                                                             int T, int d, float scale) {
  extern __shared__ float smem[];  // [d] accumulated with shared atomics
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int c = threadIdx.x; c < d; c += blockDim.x) smem[c] = 0.f;
  __syncthreads();
  for (int row = blockIdx.x * wpb + w; row < T; row += gridDim.x * wpb) {
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane; c < d; c += 32) dot += to_f<InT>(dy[(size_t)row * d + c]) * gain[c] * scale * x[(size_t)row * d + c];
    dot = warp_sum(dot);
    const float k = r * r * r * dot / d;
    for (int c = lane; c < d; c += 32) {
      const float dyv = to_f<InT>(dy[(size_t)row * d + c]), xv = x[(size_t)row * d + c];
      float o = r * dyv * gain[c] * scale - k * xv;
      if (dres_in) o += dres_in[(size_t)row * d + c];
      dres[(size_t)row * d + c] = o;
      dres_lp[(size_t)row * d + c] = from_f<InT>(o);
      atomicAdd(&smem[c], dyv * xv * r);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) dgain_partial[(size_t)blockIdx.x * d + c] = smem[c] * scale;
}

// out[c] = sum_r partial[r, c]; 32 columns per CTA, 8 row groups per column reduced through shared memory.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int d) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < d)
    for (int r = ty; r < rows; r += 8) s += partial[(size_t)r * d + c];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += red[j][tx];
    out[c] = t;
  }
}

int add_rmsnorm_bwd_grid(int T) {
  const int wpb = 8;
  int g = (T + wpb - 1) / wpb;
  return g < kNormBwdMaxGrid ? g : kNormBwdMaxGrid;
}

template <typename InT>
static void launch_bwd(const InT* dy, const float* dres_in, const float* x, const float* gain, const float* rstd, float* dres,
                       InT* dres_lp, float* dgain, float* scratch, int T, int d, float scale, cudaStream_t st) {
  const int wpb = 8;
  const int grid = add_rmsnorm_bwd_grid(T);
  dim3 block(wpb * 32);
  bool done = false;
#define SEG_CASE(V)                                                                                                   \
  case V:                                                                                                             \
    add_rmsnorm_bwd_kernel<V, InT><<<grid, block, (size_t)wpb * d * sizeof(float), st>>>(dy, dres_in, x, gain, rstd, dres, \
                                                                                           dres_lp, scratch, T, d, scale);  \
    done = true;                                                                                                      \
    break;
  if (d % 128 == 0 && (size_t)wpb * d * sizeof(float) <= 48 * 1024) {
    switch (d / 128) {
      SEG_CASE(1) SEG_CASE(2) SEG_CASE(3) SEG_CASE(4) SEG_CASE(6) SEG_CASE(8) SEG_CASE(9) SEG_CASE(12)
      default: break;
    }
  }
#undef SEG_CASE
  if (!done)
    add_rmsnorm_bwd_generic<InT><<<grid, block, (size_t)d * sizeof(float), st>>>(dy, dres_in, x, gain, rstd, dres, dres_lp,
                                                                                  scratch, T, d, scale);
  colsum_kernel<<<(d + 31) / 32, 256, 0, st>>>(scratch, dgain, grid, d);
}

void add_rmsnorm_bwd(const void* dy, const float* dres_in, const float* x, const float* gain, const float* rstd, float* dres,
                     void* dres_lp, float* dgain, float* scratch, int T, int d, float scale, bool bf16, cudaStream_t st) {
  if (bf16)
    launch_bwd<__nv_bfloat16>((const __nv_bfloat16*)dy, dres_in, x, gain, rstd, dres, (__nv_bfloat16*)dres_lp, dgain, scratch, T, d, scale, st);
  else
    launch_bwd<float>((const float*)dy, dres_in, x, gain, rstd, dres, (float*)dres_lp, dgain, scratch, T, d, scale, st);
}

}  // namespace seg
