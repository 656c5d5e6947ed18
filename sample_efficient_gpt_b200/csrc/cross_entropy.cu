// Softmax cross-entropy with z-loss over a chunk of bf16 logits, gradient written in place.
//   lse = logsumexp(x);  loss = lse - x_y + s*lse^2;  z = s*lse^2
//   dx  = grad_scale * (softmax(x) * (1 + 2 s lse) - onehot(y));  ignored rows: loss = z = 0, dx = 0
// (same definitions as the reference's kernel, transformer/ops/cross_entropy.py:96-247, which makes two passes over
// the row in global memory).  One CTA owns a row.  Pass 1 streams the row once with an online max / sum per thread (nothing
// is kept in registers, so several CTAs share an SM and one CTA's loads overlap another's arithmetic); pass 2 re-reads
// the row, which is still in L2 (96 KB per row at 49152 columns, a few hundred rows in flight on the whole GPU), and
// overwrites it with the gradient: DRAM sees one read and one write of the chunk.
#include "common.cuh"
#include "kernels.h"

namespace seg {

constexpr int kCeThreads = 512;

__global__ void __launch_bounds__(kCeThreads, 2) ce_rows_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                              float* __restrict__ loss, float* __restrict__ z,
                                                              float* __restrict__ lse_out, int V, float s, int64_t ignore_index,
                                                              float grad_scale, float logit_scale, bool write_grad) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  __nv_bfloat16* x = logits + (size_t)row * V;
  const int64_t tgt = targets[row];
  const bool valid = tgt != ignore_index;
  const float xt = valid ? __bfloat162float(x[tgt]) * logit_scale : 0.f;
  const int nvec = V >> 3;
  const float c2 = logit_scale * 1.4426950408889634f;  // logits -> exp2 domain
  float m = -INFINITY, sum = 0.f;                        // running maximum (exp2 domain) and sum of 2^(x - m)
#pragma unroll 4
  for (int vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[vi], f);
    float vm = f[0] * c2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] *= c2;
      vm = fmaxf(vm, f[j]);
    }
    if (vm > m) {
      sum *= exp2f(m - vm);  // 0 on the first vector (m = -inf)
      m = vm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += exp2f(f[j] - m);
  }
  const float mx = block_max(m, red);
  sum = block_sum(m > -INFINITY ? sum * exp2f(m - mx) : 0.f, red);  // contains a __syncthreads after every thread has read x[tgt]
  const float lse = (mx + log2f(sum)) * 0.6931471805599453f;
  if (threadIdx.x == 0) {
    const float zz = s * lse * lse;
    loss[row] = valid ? (lse - xt + zz) : 0.f;
    z[row] = valid ? zz : 0.f;
    lse_out[row] = lse;
  }
  if (!write_grad) return;
  const float k = valid ? grad_scale * logit_scale * (1.f + 2.f * s * lse) / sum : 0.f;
  const float gs = valid ? grad_scale * logit_scale : 0.f;
#pragma unroll 4
  for (int vi = threadIdx.x; vi < nvec; vi += kCeThreads) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[vi], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      g[j] = exp2f(fmaf(f[j], c2, -mx)) * k;
      if ((int64_t)vi * 8 + j == tgt) g[j] -= gs;
    }
    reinterpret_cast<bf16x8*>(x)[vi] = pack8(g);
  }
}

void ce_chunk_fwd_bwd(void* logits, const int64_t* targets, float* loss, float* z, float* lse, int rows, int V,
                      float lse_square_scale, int64_t ignore_index, float grad_scale, float logit_scale, bool write_grad,
                      cudaStream_t st) {
  ce_rows_kernel<<<rows, kCeThreads, 0, st>>>((__nv_bfloat16*)logits, targets, loss, z, lse, V, lse_square_scale, ignore_index, grad_scale,
                                             logit_scale, write_grad);
}

}  // namespace seg
