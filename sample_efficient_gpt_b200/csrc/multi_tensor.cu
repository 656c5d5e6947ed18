// Multi-tensor element-wise kernels: one launch updates every tensor of a list.
// The list is described by device arrays of base pointers and sizes plus a chunk table: chunk c covers
// elements [chunk_offset[c], chunk_offset[c] + chunk_elems) of tensor chunk_tensor[c]; one CTA per chunk.
//   AdamW (training/optimizer.py:45-112 of the reference): g[nan] = 0; p *= 1 - lr*wd; m = b1 m + (1-b1) g;
//         v = b2 v + (1-b2) g^2; p -= step_size * m / (sqrt(v) + eps); optional bf16 shadow of p written too.
//   EMA   (scripts/data_processing/sft/ema_posthoc.py:88-98): ema = d*ema + (1-d)*p.
//   cast  fp32 -> bf16 shadow copies of the GEMM weights.
#include "common.cuh"
#include "kernels.h"

namespace seg {

// A chunk is walked four elements per thread and access when the tensor's arrays and the chunk start are 16-byte aligned
// (chunk sizes are multiples of 4; a tensor's ragged end is finished one element at a time).
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ void adamw_one(float& pi, float gi, float& mi, float& vi, float decay, float b1, float b2, float eps, float step_size) {
  if (gi != gi) gi = 0.f;
  mi = b1 * mi + (1.f - b1) * gi;
  vi = b2 * vi + (1.f - b2) * gi * gi;
  pi = pi * decay - step_size * mi / (sqrtf(vi) + eps);
}

__global__ void __launch_bounds__(256) adamw_multi_kernel(float** p, const float** g, float** m, float** v, void** shadow,
                                                        const int64_t* sizes, const int32_t* chunk_tensor,
                                                        const int64_t* chunk_offset, int chunk_elems, float lr, float wd, float b1,
                                                        float b2, float eps, float step_size) {
  const int t = chunk_tensor[blockIdx.x];
  const int64_t off = chunk_offset[blockIdx.x];
  const int64_t n = sizes[t];
  const int64_t end = (off + chunk_elems < n) ? off + chunk_elems : n;
  float* __restrict__ pp = p[t];
  const float* __restrict__ gg = g[t];
  float* __restrict__ mm = m[t];
  float* __restrict__ vv = v[t];
  __nv_bfloat16* __restrict__ sh = (__nv_bfloat16*)shadow[t];
  const float decay = 1.f - lr * wd;
  int64_t i0 = off;
  if ((off & 3) == 0 && aligned16(pp) && aligned16(gg) && aligned16(mm) && aligned16(vv) && (sh == nullptr || (reinterpret_cast<uintptr_t>(sh) & 7) == 0)) {
    const int64_t vend = off + ((end - off) & ~(int64_t)3);
    for (int64_t i = off + 4 * (int64_t)threadIdx.x; i < vend; i += 4 * (int64_t)blockDim.x) {
      float4 p4 = *reinterpret_cast<const float4*>(pp + i);
      const float4 g4 = *reinterpret_cast<const float4*>(gg + i);
      float4 m4 = *reinterpret_cast<const float4*>(mm + i);
      float4 v4 = *reinterpret_cast<const float4*>(vv + i);
      adamw_one(p4.x, g4.x, m4.x, v4.x, decay, b1, b2, eps, step_size);
      adamw_one(p4.y, g4.y, m4.y, v4.y, decay, b1, b2, eps, step_size);
      adamw_one(p4.z, g4.z, m4.z, v4.z, decay, b1, b2, eps, step_size);
      adamw_one(p4.w, g4.w, m4.w, v4.w, decay, b1, b2, eps, step_size);
      *reinterpret_cast<float4*>(mm + i) = m4;
      *reinterpret_cast<float4*>(vv + i) = v4;
      *reinterpret_cast<float4*>(pp + i) = p4;
      if (sh != nullptr) store4<__nv_bfloat16>(sh + i, p4);
    }
    i0 = vend;
  }
  for (int64_t i = i0 + threadIdx.x; i < end; i += blockDim.x) {
    float pi = pp[i], mi = mm[i], vi = vv[i];
    adamw_one(pi, gg[i], mi, vi, decay, b1, b2, eps, step_size);
    mm[i] = mi;
    vv[i] = vi;
    pp[i] = pi;
    if (sh != nullptr) sh[i] = __float2bfloat16_rn(pi);
  }
}

__global__ void __launch_bounds__(256) ema_multi_kernel(float** ema, const float** src, const int64_t* sizes,
                                                      const int32_t* chunk_tensor, const int64_t* chunk_offset, int chunk_elems,
                                                      float decay) {
  const int t = chunk_tensor[blockIdx.x];
  const int64_t off = chunk_offset[blockIdx.x];
  const int64_t n = sizes[t];
  const int64_t end = (off + chunk_elems < n) ? off + chunk_elems : n;
  float* __restrict__ e = ema[t];
  const float* __restrict__ s = src[t];
  int64_t i0 = off;
  if ((off & 3) == 0 && aligned16(e) && aligned16(s)) {
    const int64_t vend = off + ((end - off) & ~(int64_t)3);
    for (int64_t i = off + 4 * (int64_t)threadIdx.x; i < vend; i += 4 * (int64_t)blockDim.x) {
      float4 a = *reinterpret_cast<const float4*>(e + i);
      const float4 b = *reinterpret_cast<const float4*>(s + i);
      a.x = decay * a.x + (1.f - decay) * b.x;
      a.y = decay * a.y + (1.f - decay) * b.y;
      a.z = decay * a.z + (1.f - decay) * b.z;
      a.w = decay * a.w + (1.f - decay) * b.w;
      *reinterpret_cast<float4*>(e + i) = a;
    }
    i0 = vend;
  }
  for (int64_t i = i0 + threadIdx.x; i < end; i += blockDim.x) e[i] = decay * e[i] + (1.f - decay) * s[i];
}

__global__ void __launch_bounds__(256) cast_multi_kernel(void** dst, const float** src, const int64_t* sizes,
                                                       const int32_t* chunk_tensor, const int64_t* chunk_offset, int chunk_elems) {
  const int t = chunk_tensor[blockIdx.x];
  const int64_t off = chunk_offset[blockIdx.x];
  const int64_t n = sizes[t];
  const int64_t end = (off + chunk_elems < n) ? off + chunk_elems : n;
  __nv_bfloat16* __restrict__ d = (__nv_bfloat16*)dst[t];
  const float* __restrict__ s = src[t];
  int64_t i0 = off;
  if ((off & 3) == 0 && aligned16(s) && (reinterpret_cast<uintptr_t>(d) & 7) == 0) {
    const int64_t vend = off + ((end - off) & ~(int64_t)3);
    for (int64_t i = off + 4 * (int64_t)threadIdx.x; i < vend; i += 4 * (int64_t)blockDim.x)
      store4<__nv_bfloat16>(d + i, *reinterpret_cast<const float4*>(s + i));
    i0 = vend;
  }
  for (int64_t i = i0 + threadIdx.x; i < end; i += blockDim.x) d[i] = __float2bfloat16_rn(s[i]);
}

void adamw_multi(float** p, const float** g, float** m, float** v, void** shadow, const int64_t* sizes, const int32_t* chunk_tensor,
                 const int64_t* chunk_offset, int n_chunks, int chunk_elems, float lr, float wd, float b1, float b2, float eps,
                 float step_size, cudaStream_t st) {
  if (n_chunks == 0) return;
  adamw_multi_kernel<<<n_chunks, 256, 0, st>>>(p, g, m, v, shadow, sizes, chunk_tensor, chunk_offset, chunk_elems, lr, wd, b1, b2,
                                               eps, step_size);
}

void ema_multi(float** ema, const float** src, const int64_t* sizes, const int32_t* chunk_tensor, const int64_t* chunk_offset,
               int n_chunks, int chunk_elems, float decay, cudaStream_t st) {
  if (n_chunks == 0) return;
  ema_multi_kernel<<<n_chunks, 256, 0, st>>>(ema, src, sizes, chunk_tensor, chunk_offset, chunk_elems, decay);
}

void cast_multi(void** dst_bf16, const float** src, const int64_t* sizes, const int32_t* chunk_tensor, const int64_t* chunk_offset,
                int n_chunks, int chunk_elems, cudaStream_t st) {
  if (n_chunks == 0) return;
  cast_multi_kernel<<<n_chunks, 256, 0, st>>>(dst_bf16, src, sizes, chunk_tensor, chunk_offset, chunk_elems);
}

}  // namespace seg
