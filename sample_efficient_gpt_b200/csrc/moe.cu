// Mixture-of-experts routing and expert-parallel token exchange over NVLink peer memory.
//
// The expert-parallel layout: E experts split evenly over `world` ranks (E_local each).  Every owner rank holds, per
// exchange buffer, rows laid out as [E_local][world (source rank)][cap][d] in symmetric (peer-mapped) memory.
//
//   route     softmax router (fp32 logits from the bf16 hidden row and the fp32 router weight), top-k, renormalised
//             weights, per-block assignment counts per expert
//   scan      exclusive scan of the per-block counts -> first slot of every block inside each expert, totals per expert
//   slot      slot of every (token, choice) assignment in (token, choice) order; -1 when the expert's capacity is exceeded
//   push      all-to-all dispatch fused with the permutation: every kept assignment's row is written straight into the
//             owner rank's buffer (16-byte peer stores), optionally scaled by its routing weight (backward: w * dout);
//             the unused tail of each (source, expert) region is zero-filled by the sender
//   pull      all-to-all combine fused with the un-permutation: every token reads its k rows from the owners' buffers
//             (16-byte peer loads), forms the weighted sum in fp32, and optionally the dot products <g[t], row> with a
//             second buffer (backward: d(weight) = <dout[t], y_k[t]>)
//   route_bwd gradient of the renormalised top-k weights, the load-balance term and the softmax -> d(logits)
//
// Ordering between ranks: outputs are written before the sources pull them because the device-side flag barrier of comm.cu
// runs between the kernels; rows are pushed before the owner's GEMM reads them either through that barrier or, in the
// overlapped mode, because the push kernel's last CTA releases a per-destination flag that the GEMM's producer acquires per
// source region (gemm.cu).  None of the kernels here waits on anything.
// The reference has no mixture-of-experts code; the specification is models/moe.py of this package.
#include "bounds.cuh"
#include "common.cuh"
#include "kernels.h"

namespace seg {

struct MoeBufs {
  void* p[kMaxRanks];
};

template <int EP>
__global__ void __launch_bounds__(kMoeTokensPerBlock * 32) moe_route_kernel(const __nv_bfloat16* __restrict__ x,
                                                                           const float* __restrict__ wr, int T, int d, int E, int k,
                                                                           float* __restrict__ probs, int* __restrict__ idx,
                                                                           float* __restrict__ w, int* __restrict__ block_counts) {
  __shared__ int counts[kMoeMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kMoeMaxExperts) counts[threadIdx.x] = 0;
  __syncthreads();
  const int t = blockIdx.x * kMoeTokensPerBlock + warp;
  if (t < T) {
    float acc[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) acc[e] = 0.f;
    const __nv_bfloat16* xr = x + (size_t)t * d;
    for (int v = lane; v < d / 8; v += 32) {
      float xv[8];
      load8<__nv_bfloat16>(xr + v * 8, xv);
#pragma unroll
      for (int e = 0; e < EP; ++e)
        if (e < E) {
          float wv[8];
          load8<float>(wr + (size_t)e * d + v * 8, wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[e] = fmaf(xv[j], wv[j], acc[e]);
        }
    }
    float mine = -INFINITY;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      const float s = warp_sum(acc[e]);
      if (lane == e && e < E) mine = s;
    }
    const float mx = warp_max(mine);
    const float ex = lane < E ? __expf(mine - mx) : 0.f;
    const float p = ex / warp_sum(ex);
    if (lane < E) probs[(size_t)t * E + lane] = p;
    float cur = lane < E ? p : -1.f;
    int sel[kMoeMaxTopK];
    float selp[kMoeMaxTopK];
    float total = 0.f;
#pragma unroll
    for (int c = 0; c < kMoeMaxTopK; ++c)
      if (c < k) {
        const float best = warp_max(cur);
        const unsigned m = __ballot_sync(0xffffffffu, cur == best && lane < E);
        const int who = __ffs(m) - 1;  // lowest expert index among equal probabilities
        sel[c] = who;
        selp[c] = best;
        total += best;
        if (lane == who) cur = -1.f;
      }
    if (lane == 0) {
#pragma unroll
      for (int c = 0; c < kMoeMaxTopK; ++c)
        if (c < k) {
          idx[(size_t)t * k + c] = sel[c];
          w[(size_t)t * k + c] = selp[c] / total;
          atomicAdd(&counts[sel[c]], 1);
        }
    }
  }
  __syncthreads();
  if (threadIdx.x < E) block_counts[(size_t)blockIdx.x * E + threadIdx.x] = counts[threadIdx.x];
}

// One block of 32 * E threads: warp e scans expert e over the blocks.
__global__ void moe_scan_kernel(const int* __restrict__ block_counts, int nblk, int E, int* __restrict__ block_off,
                                int* __restrict__ totals) {
  const int e = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (e >= E) return;
  int running = 0;
  for (int base = 0; base < nblk; base += 32) {
    const int i = base + lane;
    const int c = i < nblk ? block_counts[(size_t)i * E + e] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (i < nblk) block_off[(size_t)i * E + e] = running + incl - c;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) totals[e] = running;
}

// One block per kMoeTokensPerBlock tokens, kMoeTokensPerBlock * kMoeMaxTopK threads.
__global__ void moe_slot_kernel(const int* __restrict__ idx, const int* __restrict__ block_off, int T, int E, int k, int cap,
                                int* __restrict__ slot) {
  __shared__ int es[kMoeTokensPerBlock * kMoeMaxTopK];
  const int a = threadIdx.x;
  const int n_assign = kMoeTokensPerBlock * k;
  const int t = blockIdx.x * kMoeTokensPerBlock + a / k;
  const bool live = a < n_assign && t < T;
  const int e = live ? idx[(size_t)t * k + a % k] : -1;
  if (a < kMoeTokensPerBlock * kMoeMaxTopK) es[a] = e;
  __syncthreads();
  if (!live) return;
  int rank_in_block = 0;
  for (int b = 0; b < a; ++b) rank_in_block += (es[b] == e);
  const int pos = block_off[(size_t)blockIdx.x * E + e] + rank_in_block;
  slot[(size_t)t * k + a % k] = pos < cap ? pos : -1;
}

// Row blocks [0, n_row_blocks): one warp per token.  Tail blocks [n_row_blocks, n_row_blocks + E * kMoeTailBlocks): zero-fill.
__global__ void __launch_bounds__(256) moe_push_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                                     const int* __restrict__ slot, const float* __restrict__ w,
                                                     const int* __restrict__ totals, MoeBufs dst, int T, int d, int E, int k, int cap,
                                                     int e_local, int world, int rank, int n_row_blocks, MoeBufs flags,
                                                     uint32_t* done_counter, uint32_t seq, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = d / 8;
  if ((int)blockIdx.x < n_row_blocks) {
    const int t = blockIdx.x * 8 + warp;
    if (t < T) {
    __nv_bfloat16* rows[kMoeMaxTopK];
    float ws[kMoeMaxTopK];
#pragma unroll
    for (int c = 0; c < kMoeMaxTopK; ++c) {
      rows[c] = nullptr;
      ws[c] = 1.f;
      if (c < k) {
        const int s = slot[(size_t)t * k + c];
        if (s >= 0) {
          const int e = idx[(size_t)t * k + c];
          // expert and slot come from device tables: in the debug build both, and the row they address, are checked
          if (!SEG_IN_BOUNDS(status, 21, e, 1, E) || !SEG_IN_BOUNDS(status, 21, s, 1, cap) ||
              !SEG_IN_BOUNDS(status, 22, ((size_t)((e % e_local) * world + rank) * cap + s) * d, d, (size_t)e_local * world * cap * d))
            continue;
          rows[c] = reinterpret_cast<__nv_bfloat16*>(dst.p[e / e_local]) + ((size_t)((e % e_local) * world + rank) * cap + s) * d;
          if (w != nullptr) ws[c] = w[(size_t)t * k + c];
        }
      }
    }
    const __nv_bfloat16* xr = x + (size_t)t * d;
    for (int v = lane; v < vecs; v += 32) {
      const bf16x8 raw = *reinterpret_cast<const bf16x8*>(xr + v * 8);
#pragma unroll
      for (int c = 0; c < kMoeMaxTopK; ++c)
        if (rows[c] != nullptr) {
          if (w != nullptr) {
            float f[8];
            unpack8(raw, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= ws[c];
            *reinterpret_cast<bf16x8*>(rows[c] + v * 8) = pack8(f);
          } else {
            *reinterpret_cast<bf16x8*>(rows[c] + v * 8) = raw;
          }
        }
    }
    }
  } else {
    const int b = blockIdx.x - n_row_blocks;
    const int e = b / kMoeTailBlocks, part = b % kMoeTailBlocks;
    const int first = min(totals[e], cap);
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(dst.p[e / e_local]) + (size_t)((e % e_local) * world + rank) * cap * d;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int r = first + part * 8 + warp; r < cap; r += kMoeTailBlocks * 8)
      for (int v = lane; v < vecs; v += 32) *reinterpret_cast<uint4*>(base + (size_t)r * d + v * 8) = zero;
  }
  if (done_counter == nullptr) return;
  // Completion signal: the last CTA to finish tells every destination rank that this rank's rows have landed.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;  // ready for the next launch (launches on one stream do not overlap)
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(flags.p[r]) + rank), "r"(seq) : "memory");
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256) moe_pull_kernel(MoeBufs src, MoeBufs src2, const int* __restrict__ idx,
                                                     const int* __restrict__ slot, const float* __restrict__ w,
                                                     const __nv_bfloat16* __restrict__ g, OutT* __restrict__ out,
                                                     float* __restrict__ dots, int T, int d, int k, int cap, int e_local, int world,
                                                     int rank) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  const int vecs = d / 8;
  const __nv_bfloat16* rows[kMoeMaxTopK];
  const __nv_bfloat16* rows2[kMoeMaxTopK];
  float ws[kMoeMaxTopK], dot[kMoeMaxTopK];
#pragma unroll
  for (int c = 0; c < kMoeMaxTopK; ++c) {
    rows[c] = rows2[c] = nullptr;
    ws[c] = 1.f;
    dot[c] = 0.f;
    if (c < k) {
      const int s = slot[(size_t)t * k + c];
      if (s >= 0) {
        const int e = idx[(size_t)t * k + c];
        const size_t off = ((size_t)((e % e_local) * world + rank) * cap + s) * d;
        rows[c] = reinterpret_cast<const __nv_bfloat16*>(src.p[e / e_local]) + off;
        if (dots != nullptr) rows2[c] = reinterpret_cast<const __nv_bfloat16*>(src2.p[e / e_local]) + off;
        if (w != nullptr) ws[c] = w[(size_t)t * k + c];
      }
    }
  }
  for (int v = lane; v < vecs; v += 32) {
    bf16x8 in[kMoeMaxTopK], in2[kMoeMaxTopK];
#pragma unroll
    for (int c = 0; c < kMoeMaxTopK; ++c) {
      if (rows[c] != nullptr) in[c] = *reinterpret_cast<const bf16x8*>(rows[c] + v * 8);
      if (rows2[c] != nullptr) in2[c] = *reinterpret_cast<const bf16x8*>(rows2[c] + v * 8);
    }
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    float gv[8];
    if (dots != nullptr) load8<__nv_bfloat16>(g + (size_t)t * d + v * 8, gv);
#pragma unroll
    for (int c = 0; c < kMoeMaxTopK; ++c) {
      if (rows[c] != nullptr) {
        float f[8];
        unpack8(in[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(ws[c], f[j], acc[j]);
      }
      if (rows2[c] != nullptr) {
        float f[8];
        unpack8(in2[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) dot[c] = fmaf(gv[j], f[j], dot[c]);
      }
    }
    store8<OutT>(out + (size_t)t * d + v * 8, acc);
  }
  if (dots != nullptr) {
#pragma unroll
    for (int c = 0; c < kMoeMaxTopK; ++c)
      if (c < k) {
        const float s = warp_sum(dot[c]);
        if (lane == 0) dots[(size_t)t * k + c] = s;
      }
  }
}

// One warp per token, lane = expert.
__global__ void __launch_bounds__(256) moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ idx,
                                                          const float* __restrict__ dw, const float* __restrict__ aux_vec, int T,
                                                          int E, int k, float* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  const float p = lane < E ? probs[(size_t)t * E + lane] : 0.f;
  float dp = lane < E ? aux_vec[lane] : 0.f;
  int sel[kMoeMaxTopK];
  float pr[kMoeMaxTopK], g[kMoeMaxTopK];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < kMoeMaxTopK; ++c)
    if (c < k) {
      sel[c] = idx[(size_t)t * k + c];
      pr[c] = __shfl_sync(0xffffffffu, p, sel[c]);
      g[c] = dw[(size_t)t * k + c];
      s += pr[c];
    }
  float mix = 0.f;  // sum_j dw_j * w_j with w_j = pr_j / s
#pragma unroll
  for (int c = 0; c < kMoeMaxTopK; ++c)
    if (c < k) mix += g[c] * pr[c] / s;
#pragma unroll
  for (int c = 0; c < kMoeMaxTopK; ++c)
    if (c < k && lane == sel[c]) dp += (g[c] - mix) / s;
  const float inner = warp_sum(dp * p);
  if (lane < E) dlogits[(size_t)t * E + lane] = p * (dp - inner);
}

static MoeBufs make_bufs(void* const* ptrs, int world) {
  MoeBufs b;
  for (int i = 0; i < kMaxRanks; ++i) b.p[i] = (ptrs != nullptr && i < world) ? ptrs[i] : nullptr;
  return b;
}

int moe_route(const void* x, const float* wr, int T, int d, int E, int k, float* probs, int* idx, float* w, int* block_counts,
              int* block_off, int* totals, cudaStream_t st) {
  if (E < 1 || E > kMoeMaxExperts || k < 1 || k > kMoeMaxTopK || k > E || d % 8 != 0) return 1;
  const int nblk = (T + kMoeTokensPerBlock - 1) / kMoeTokensPerBlock;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const dim3 block(kMoeTokensPerBlock * 32);
  if (E <= 8)
    moe_route_kernel<8><<<nblk, block, 0, st>>>(xp, wr, T, d, E, k, probs, idx, w, block_counts);
  else if (E <= 16)
    moe_route_kernel<16><<<nblk, block, 0, st>>>(xp, wr, T, d, E, k, probs, idx, w, block_counts);
  else
    moe_route_kernel<32><<<nblk, block, 0, st>>>(xp, wr, T, d, E, k, probs, idx, w, block_counts);
  moe_scan_kernel<<<1, 32 * E, 0, st>>>(block_counts, nblk, E, block_off, totals);
  return 0;
}

void moe_slots(const int* idx, const int* block_off, int T, int E, int k, int cap, int* slot, cudaStream_t st) {
  const int nblk = (T + kMoeTokensPerBlock - 1) / kMoeTokensPerBlock;
  moe_slot_kernel<<<nblk, kMoeTokensPerBlock * kMoeMaxTopK, 0, st>>>(idx, block_off, T, E, k, cap, slot);
}

void moe_push(const void* x, const int* idx, const int* slot, const float* w, const int* totals, void* const* dst, int T, int d,
              int E, int k, int cap, int world, int rank, cudaStream_t st, uint32_t* const* flags, uint32_t* done_counter,
              uint32_t seq, int* status) {
  const int n_row_blocks = (T + 7) / 8;
  const bool signal = flags != nullptr && done_counter != nullptr;
  moe_push_kernel<<<n_row_blocks + E * kMoeTailBlocks, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), idx, slot, w, totals, make_bufs(dst, world), T, d, E, k, cap, E / world, world, rank,
      n_row_blocks, make_bufs(signal ? reinterpret_cast<void* const*>(flags) : nullptr, world), signal ? done_counter : nullptr, seq, status);
}

void moe_pull(void* const* src, void* const* src2, const int* idx, const int* slot, const float* w, const void* g, void* out,
              bool out_f32, float* dots, int T, int d, int E, int k, int cap, int world, int rank, cudaStream_t st) {
  const int blocks = (T + 7) / 8;
  const MoeBufs a = make_bufs(src, world), b = make_bufs(src2, world);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(g);
  if (out_f32)
    moe_pull_kernel<float><<<blocks, 256, 0, st>>>(a, b, idx, slot, w, gp, static_cast<float*>(out), dots, T, d, k, cap, E / world,
                                                   world, rank);
  else
    moe_pull_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a, b, idx, slot, w, gp, static_cast<__nv_bfloat16*>(out), dots, T, d, k,
                                                           cap, E / world, world, rank);
}

void moe_route_bwd(const float* probs, const int* idx, const float* dw, const float* aux_vec, int T, int E, int k, float* dlogits,
                   cudaStream_t st) {
  moe_route_bwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(probs, idx, dw, aux_vec, T, E, k, dlogits);
}

}  // namespace seg
