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

__global__ void __launch_bounds__(256) adamw_multi_kernel(float** p, const float** g, float** m, float** v, void** shadow,
                                                        const int64_t* sizes, const int32_t* chunk_tensor,
                                                        const int64_t* chunk_offset, int chunk_elems, float lr, float wd, float b1,
                                                        float b2, float eps, float step_size) {
  const int t = chunk_tensor[blockIdx.x];
  const int64_t off = chunk_offset[blockIdx.x];
  const int64_t n = sizes[t];
  const int64_t end = (off + chunk_elems < n) ? off + chunk_elems : n;
  float* pp = p[t];
  const float* gg = g[t];
  float* mm = m[t];
  float* vv = v[t];
  __nv_bfloat16* sh = (__nv_bfloat16*)shadow[t];
  const float decay = 1.f - lr * wd;
  for (int64_t i = off + threadIdx.x; i < end; i += blockDim.x) {
    float gi = gg[i];
    if (gi != gi) gi = 0.f;
    const float mi = b1 * mm[i] + (1.f - b1) * gi;
    const float vi = b2 * vv[i] + (1.f - b2) * gi * gi;
    const float pi = pp[i] * decay - step_size * mi / (sqrtf(vi) + eps);
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
  float* e = ema[t];
  const float* s = src[t];
  for (int64_t i = off + threadIdx.x; i < end; i += blockDim.x) e[i] = decay * e[i] + (1.f - decay) * s[i];
}

__global__ void __launch_bounds__(256) cast_multi_kernel(void** dst, const float** src, const int64_t* sizes,
                                                       const int32_t* chunk_tensor, const int64_t* chunk_offset, int chunk_elems) {
  const int t = chunk_tensor[blockIdx.x];
  const int64_t off = chunk_offset[blockIdx.x];
  const int64_t n = sizes[t];
  const int64_t end = (off + chunk_elems < n) ? off + chunk_elems : n;
  __nv_bfloat16* d = (__nv_bfloat16*)dst[t];
  const float* s = src[t];
  for (int64_t i = off + threadIdx.x; i < end; i += blockDim.x) d[i] = __float2bfloat16_rn(s[i]);
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
