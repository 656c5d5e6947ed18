// SwiGLU on the packed [gate | up] projection and the per-head output gate, forward and backward.
//   swiglu: f = silu(a) * b with a = u[:, :F], b = u[:, F:]          (transformer/core.py:86-89 of the reference)
//           da = df * b * (s + a s (1 - s)), db = df * a * s,  s = sigmoid(a)
//   gate  : g[t,h,:] = 2 sigmoid(z[t,h]) * o[t,h,:]                   (transformer/attention.py:249-255)
//           do = 2 s dg ;  dz = 2 s (1 - s) sum_d dg * o
// Pure streaming kernels: 4 elements per thread per access, every tensor touched once.  Index divisions run in 32 bits
// whenever the item count allows (a 64-bit division costs more instructions than the rest of an item).
#include "common.cuh"
#include "kernels.h"

namespace seg {

// VEC elements per thread and access: 8 (16-byte bf16 / 2 x 16-byte fp32 accesses) when F % 8 == 0, else 4.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ u, T* __restrict__ f, int64_t rows, int F) {
  const int fv = F / VEC;
  const int64_t total = rows * fv;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = total <= 0x7fffffff ? (int64_t)((uint32_t)i / (uint32_t)fv) : i / fv;
    const int c = (int)(i - r * fv) * VEC;
    float a[8], b[8], o[8];
    if (VEC == 8) {
      load8<T>(u + r * 2 * F + c, a);
      load8<T>(u + r * 2 * F + F + c, b);
    } else {
      const float4 a4 = load4<T>(u + r * 2 * F + c), b4 = load4<T>(u + r * 2 * F + F + c);
      a[0] = a4.x; a[1] = a4.y; a[2] = a4.z; a[3] = a4.w;
      b[0] = b4.x; b[1] = b4.y; b[2] = b4.z; b[3] = b4.w;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = a[j] * sigmoidf_(a[j]) * b[j];
    if (VEC == 8)
      store8<T>(f + r * F + c, o);
    else
      store4<T>(f + r * F + c, make_float4(o[0], o[1], o[2], o[3]));
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ df, const T* __restrict__ u, T* __restrict__ du,
                                                       int64_t rows, int F) {
  const int fv = F / VEC;
  const int64_t total = rows * fv;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = total <= 0x7fffffff ? (int64_t)((uint32_t)i / (uint32_t)fv) : i / fv;
    const int c = (int)(i - r * fv) * VEC;
    float a[8], b[8], g[8], da[8], db[8];
    if (VEC == 8) {
      load8<T>(u + r * 2 * F + c, a);
      load8<T>(u + r * 2 * F + F + c, b);
      load8<T>(df + r * F + c, g);
    } else {
      const float4 a4 = load4<T>(u + r * 2 * F + c), b4 = load4<T>(u + r * 2 * F + F + c), g4 = load4<T>(df + r * F + c);
      a[0] = a4.x; a[1] = a4.y; a[2] = a4.z; a[3] = a4.w;
      b[0] = b4.x; b[1] = b4.y; b[2] = b4.z; b[3] = b4.w;
      g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) swiglu_grad(a[j], b[j], g[j], da[j], db[j]);
    if (VEC == 8) {
      store8<T>(du + r * 2 * F + c, da);
      store8<T>(du + r * 2 * F + F + c, db);
    } else {
      store4<T>(du + r * 2 * F + c, make_float4(da[0], da[1], da[2], da[3]));
      store4<T>(du + r * 2 * F + F + c, make_float4(db[0], db[1], db[2], db[3]));
    }
  }
}

static int stream_grid(int64_t work_items, int block) {
  int64_t g = (work_items + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

void swiglu_fwd(const void* u, void* f, int64_t T, int F, bool bf16, cudaStream_t st) {
  const bool v8 = (F % 8 == 0);
  const int grid = stream_grid(T * (F / (v8 ? 8 : 4)), 256);
#define SEG_SW(TY, V) swiglu_fwd_kernel<TY, V><<<grid, 256, 0, st>>>((const TY*)u, (TY*)f, T, F)
  if (bf16) { if (v8) SEG_SW(__nv_bfloat16, 8); else SEG_SW(__nv_bfloat16, 4); }
  else { if (v8) SEG_SW(float, 8); else SEG_SW(float, 4); }
#undef SEG_SW
}

void swiglu_bwd(const void* df, const void* u, void* du, int64_t T, int F, bool bf16, cudaStream_t st) {
  const bool v8 = (F % 8 == 0);
  const int grid = stream_grid(T * (F / (v8 ? 8 : 4)), 256);
#define SEG_SWB(TY, V) swiglu_bwd_kernel<TY, V><<<grid, 256, 0, st>>>((const TY*)df, (const TY*)u, (TY*)du, T, F)
  if (bf16) { if (v8) SEG_SWB(__nv_bfloat16, 8); else SEG_SWB(__nv_bfloat16, 4); }
  else { if (v8) SEG_SWB(float, 8); else SEG_SWB(float, 4); }
#undef SEG_SWB
}

// One group of hd/8 threads per (token, head): 16-byte accesses, hd/8 is 8 (hd 64) or 16 (hd 128), so a warp holds 4 or 2
// heads.  The gate logits z (and their gradient) are addressed as [token * stride + head], so they can be columns of a
// wider projection output and no compact copy is needed.
template <typename T, int HD>
__global__ void __launch_bounds__(256) gate_fwd_kernel(const T* __restrict__ o, const T* __restrict__ z, T* __restrict__ g,
                                                     int64_t n_heads_total, int H, int64_t z_stride) {
  constexpr int TPH = HD / 8;
  const int64_t total = n_heads_total * TPH;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t head = i / TPH;
    const int64_t tok = total <= 0x7fffffff ? (int64_t)((uint32_t)head / (uint32_t)H) : head / H;
    const float s = 2.f * sigmoidf_(to_f<T>(z[tok * z_stride + (head - tok * H)]));
    float v[8];
    load8<T>(o + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= s;
    store8<T>(g + i * 8, v);
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(256) gate_bwd_kernel(const T* __restrict__ dg, const T* __restrict__ o, const T* __restrict__ z,
                                                     T* __restrict__ dout, T* __restrict__ dz, int64_t n_heads_total, int H,
                                                     int64_t z_stride, int64_t dz_stride) {
  constexpr int TPH = HD / 8;
  const int64_t total = n_heads_total * TPH;  // multiple of TPH; blockDim is a multiple of 32 >= TPH
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (total + stride - 1) / stride;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (int64_t it = 0; it < rounds; ++it, i += stride) {
    const bool live = i < total;
    const int64_t head = live ? i / TPH : 0;
    const int64_t tok = total <= 0x7fffffff ? (int64_t)((uint32_t)head / (uint32_t)H) : head / H;
    const int h = (int)(head - tok * H);
    float sg = 0.f, dot = 0.f;
    if (live) {
      sg = sigmoidf_(to_f<T>(z[tok * z_stride + h]));
      float a[8], b[8];
      load8<T>(dg + i * 8, a);
      load8<T>(o + i * 8, b);
      const float s2 = 2.f * sg;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dot += a[j] * b[j];
        a[j] *= s2;
      }
      store8<T>(dout + i * 8, a);
    }
#pragma unroll
    for (int off = TPH / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (live && (i % TPH) == 0) dz[tok * dz_stride + h] = from_f<T>(2.f * sg * (1.f - sg) * dot);
  }
}

void gate_fwd(const void* o, const void* z, void* g, int64_t T, int H, int hd, bool bf16, cudaStream_t st, int64_t z_stride) {
  const int64_t nh = T * H;
  const int grid = stream_grid(nh * (hd / 8), 256);
  if (z_stride <= 0) z_stride = H;
#define SEG_GATE(TY, HD) gate_fwd_kernel<TY, HD><<<grid, 256, 0, st>>>((const TY*)o, (const TY*)z, (TY*)g, nh, H, z_stride)
  if (bf16) { if (hd == 64) SEG_GATE(__nv_bfloat16, 64); else if (hd == 128) SEG_GATE(__nv_bfloat16, 128); else SEG_GATE(__nv_bfloat16, 32); }
  else { if (hd == 64) SEG_GATE(float, 64); else if (hd == 128) SEG_GATE(float, 128); else SEG_GATE(float, 32); }
#undef SEG_GATE
}

void gate_bwd(const void* dg, const void* o, const void* z, void* dout, void* dz, int64_t T, int H, int hd, bool bf16, cudaStream_t st,
              int64_t z_stride, int64_t dz_stride) {
  const int64_t nh = T * H;
  const int grid = stream_grid(nh * (hd / 8), 256);
  if (z_stride <= 0) z_stride = H;
  if (dz_stride <= 0) dz_stride = H;
#define SEG_GATE(TY, HD) \
  gate_bwd_kernel<TY, HD><<<grid, 256, 0, st>>>((const TY*)dg, (const TY*)o, (const TY*)z, (TY*)dout, (TY*)dz, nh, H, z_stride, dz_stride)
  if (bf16) { if (hd == 64) SEG_GATE(__nv_bfloat16, 64); else if (hd == 128) SEG_GATE(__nv_bfloat16, 128); else SEG_GATE(__nv_bfloat16, 32); }
  else { if (hd == 64) SEG_GATE(float, 64); else if (hd == 128) SEG_GATE(float, 128); else SEG_GATE(float, 32); }
#undef SEG_GATE
}

}  // namespace seg
