// Softmax cross-entropy with z-loss over a chunk of bf16 logits, gradient written in place.
//   lse = logsumexp(x);  loss = lse - x_y + s*lse^2;  z = s*lse^2
//   dx  = grad_scale * (softmax(x) * (1 + 2 s lse) - onehot(y));  ignored rows: loss = z = 0, dx = 0
// (same definitions as the reference's kernel, transformer/ops/cross_entropy.py:96-247, which makes two passes over
// the row in global memory).  Here one CTA owns a row and keeps it in registers (up to 8 x 8 bf16 per thread at 1024
// threads = 65536 columns), so the chunk is read once and written once.
#include "common.cuh"
#include "kernels.h"

namespace seg {

template <int NV>
__global__ void __launch_bounds__(1024) ce_rows_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                     float* __restrict__ loss, float* __restrict__ z, float* __restrict__ lse_out,
                                                     int V, float s, int64_t ignore_index, float grad_scale, float logit_scale,
                                                     bool write_grad) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  __nv_bfloat16* x = logits + (size_t)row * V;
  const int64_t tgt = targets[row];
  const bool valid = tgt != ignore_index;
  const float xt = valid ? __bfloat162float(x[tgt]) * logit_scale : 0.f;
  const int nvec = V >> 3;
  float f[NV][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      const bf16x8 p = reinterpret_cast<const bf16x8*>(x)[vi];
      unpack8(p, f[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[i][j] *= logit_scale;
        mx = fmaxf(mx, f[i][j]);
      }
    }
  }
  mx = block_max(mx, red);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[i][j] = __expf(f[i][j] - mx);
        sum += f[i][j];
      }
    }
  }
  sum = block_sum(sum, red);  // contains a __syncthreads after every thread has read x[tgt]
  const float lse = mx + __logf(sum);
  if (threadIdx.x == 0) {
    const float zz = s * lse * lse;
    loss[row] = valid ? (lse - xt + zz) : 0.f;
    z[row] = valid ? zz : 0.f;
    lse_out[row] = lse;
  }
  if (!write_grad) return;
  const float k = valid ? grad_scale * logit_scale * (1.f + 2.f * s * lse) / sum : 0.f;
  const float gs = valid ? grad_scale * logit_scale : 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      float g[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        g[j] = f[i][j] * k;
        if ((int64_t)vi * 8 + j == tgt) g[j] -= gs;
      }
      reinterpret_cast<bf16x8*>(x)[vi] = pack8(g);
    }
  }
}

void ce_chunk_fwd_bwd(void* logits, const int64_t* targets, float* loss, float* z, float* lse, int rows, int V,
                      float lse_square_scale, int64_t ignore_index, float grad_scale, float logit_scale, bool write_grad,
                      cudaStream_t st) {
  __nv_bfloat16* lg = (__nv_bfloat16*)logits;
  const int nvec = V / 8;
  int threads = 1024;
  if (nvec < 1024) threads = ((nvec + 31) / 32) * 32;
  const int nv = (nvec + threads - 1) / threads;
#define SEG_CE(N)                                                                                                        \
  ce_rows_kernel<N><<<rows, threads, 0, st>>>(lg, targets, loss, z, lse, V, lse_square_scale, ignore_index, grad_scale, \
                                              logit_scale, write_grad)
  if (nv <= 1) SEG_CE(1);
  else if (nv <= 2) SEG_CE(2);
  else if (nv <= 4) SEG_CE(4);
  else if (nv <= 6) SEG_CE(6);
  else SEG_CE(8);
#undef SEG_CE
}

}  // namespace seg
