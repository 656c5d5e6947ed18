// qkv post-processing (same math as qkv_post.cu; reference: transformer/rope.py:36-56, transformer/attention.py:51-63 and
// 222-228) staged through shared memory with bulk asynchronous copies.
//
// Why: a rotary pair is (x[j], x[j + hd/2]), so a thread that owns pairs reads two 16-byte pieces 64 bytes apart, and a
// warp's request touches eight 128-byte lines, half of each.  The L1 data pipe processes one line per wavefront, and
// the direct-from-global kernels of qkv_post.cu sit at ~70 % of its peak with DRAM at ~35 %.  Here whole token rows move
// global -> shared -> global as bulk copies (cp.async.bulk: full lines, no LSU wavefronts); the threads work on shared
// memory, where the unit is a bank, not a line: heads with an odd index read their second half first, so that one
// request covers all 32 banks once.  Results are written in place and leave as bulk stores; the value-residual
// gradient leaves as a bulk fp32 reduction (no read-modify-write of dv1 by threads).
//
// Roles per CTA: 256 consumer threads and one copy warp.  The copy warp's elected lane fills a two-stage ring (one
// mbarrier per stage counts the bytes of its loads), waits until the consumers have finished a stage (second mbarrier,
// 256 arrivals) and issues its stores; only that thread waits for store groups, so the consumers never stall on them.
// Every wait is bounded; on expiry the CTA raises its abort flag, sets the status word and unwinds.
// bf16, head_dim 64, sequence length a multiple of the token tile; everything else runs on the kernels of qkv_post.cu.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace seg {

using namespace sm100;

namespace {

constexpr float kQkEps = 1e-6f;
constexpr float kMixEps = 1e-8f;
constexpr int kConsumers = 256;
constexpr int kTileThreads = kConsumers + 32;
constexpr int kHeadBytes = 128;  // 64 bf16
constexpr int kStages = 2;
constexpr int kFwdTok = 8, kBwdTok = 4;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(dst)), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_f32(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(dst)), "r"(src),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return r;
}
// The two 16-byte pieces (first half, second half) of a head's 128 bytes that belong to lane group `sub`; `sw` = 64 for
// odd heads: they touch their second half first, so a warp's request covers banks 0-15 and 16-31 alike.
__device__ __forceinline__ void load_pair(const uint8_t* head, int sub, int sw, float* x1, float* x2) {
  const uint4 ra = *reinterpret_cast<const uint4*>(head + sw + sub * 16);
  const uint4 rb = *reinterpret_cast<const uint4*>(head + (64 - sw) + sub * 16);
  unpack8(sw ? rb : ra, x1);
  unpack8(sw ? ra : rb, x2);
}
__device__ __forceinline__ void store_pair(uint8_t* head, int sub, int sw, const float* x1, const float* x2) {
  const uint4 p1 = pack8(x1), p2 = pack8(x2);
  *reinterpret_cast<uint4*>(head + sw + sub * 16) = sw ? p2 : p1;
  *reinterpret_cast<uint4*>(head + (64 - sw) + sub * 16) = sw ? p1 : p2;
}
__device__ __forceinline__ void load8s(const float* p, float* f) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ float quad_sum(float v) {  // the four lanes that share a head
  const unsigned lane = threadIdx.x & 31u;
  const unsigned mask = 0xfu << (lane & ~3u);
  v += __shfl_xor_sync(mask, v, 2);
  v += __shfl_xor_sync(mask, v, 1);
  return v;
}

struct TileLayout {
  int row_b, q_b, kv_b;  // bytes per token: packed row, its q part, its k (= v) part
  int off_x, off_dq, off_dk, off_dv, off_v1, off_cos, off_sin, off_e, stage_b;
};
// fwd: [x | v1 | cos | sin]; bwd: [x | dq | dk | dv | v1 | cos | sin | e (fp32 value-residual gradient)]
__host__ __device__ inline TileLayout tile_layout(int H, int Hkv, int tok, bool bwd) {
  TileLayout L;
  L.q_b = H * kHeadBytes;
  L.kv_b = Hkv * kHeadBytes;
  L.row_b = L.q_b + 2 * L.kv_b;
  int o = 0;
  L.off_x = o; o += tok * L.row_b;
  L.off_dq = o; if (bwd) o += tok * L.q_b;
  L.off_dk = o; if (bwd) o += tok * L.kv_b;
  L.off_dv = o; if (bwd) o += tok * L.kv_b;
  L.off_v1 = o; o += tok * L.kv_b;
  L.off_cos = o; o += tok * 128;
  L.off_sin = o; o += tok * 128;
  L.off_e = o; if (bwd) o += tok * 2 * L.kv_b;
  L.stage_b = o;
  return L;
}
inline size_t tile_smem_bytes(int H, int Hkv, int tok, bool bwd) { return (size_t)kStages * tile_layout(H, Hkv, tok, bwd).stage_b + 128 + 128; }

template <int TOK>
__global__ void __launch_bounds__(kTileThreads, 2) qkv_post_fwd_tile_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                                            const __nv_bfloat16* __restrict__ v1,
                                                                            __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                                                            __nv_bfloat16* __restrict__ v, QkvPostParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  const TileLayout L = tile_layout(p.H, p.Hkv, TOK, false);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * L.stage_b);
  uint64_t* done = full + kStages;
  volatile int* cta_abort = reinterpret_cast<volatile int*>(done + kStages);
  const int nslots = p.H + 2 * p.Hkv, nrot = p.H + p.Hkv;
  const int64_t T = (int64_t)p.B * p.S;
  const int ntiles = (int)((T + TOK - 1) / TOK);
  const int tid = threadIdx.x;
  if (tid == 0) {
    *cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&done[s]), kConsumers);
    }
    fence_barrier_init();
  }
  __syncthreads();
  const AbortState ab{cta_abort, p.status, kWaitCycles};

  if (tid >= kConsumers) {
    // ------------------------------------------------------------------ copy warp
    if (tid == kConsumers) {
      bool ok = true;
      int n = 0;
      for (int tile = blockIdx.x;; tile += gridDim.x, ++n) {
        const bool have = tile < ntiles;
        if (have) {
          const int s = n % kStages;
          bulk_wait_group_read0();  // the stores that last left this stage (issued a whole tile ago) have read it
          uint8_t* st = smem + s * L.stage_b;
          const int64_t t0 = (int64_t)tile * TOK;
          const int ntok = (int)min((int64_t)TOK, T - t0);
          const uint32_t fb = smem_u32(&full[s]);
          mbar_expect_tx(fb, (uint32_t)ntok * (L.row_b + (v1 != nullptr ? L.kv_b : 0) + 256));
          for (int i = 0; i < ntok; ++i) bulk_load(smem_u32(st + L.off_x + i * L.row_b), qkv + (t0 + i) * p.qkv_stride, L.row_b, fb);
          if (v1 != nullptr) bulk_load(smem_u32(st + L.off_v1), v1 + t0 * p.Hkv * 64, ntok * L.kv_b, fb);
          const int s0 = (int)(t0 % p.S);
          bulk_load(smem_u32(st + L.off_cos), p.cos + (size_t)s0 * 32, ntok * 128, fb);
          bulk_load(smem_u32(st + L.off_sin), p.sin + (size_t)s0 * 32, ntok * 128, fb);
        }
        if (n > 0) {  // the tile before this one: once the consumers are through with it, its rows leave
          const int m = n - 1, s = m % kStages;
          if (!mbar_wait(smem_u32(&done[s]), (m / kStages) & 1, ab, 41)) { ok = false; break; }
          uint8_t* st = smem + s * L.stage_b;
          const int64_t t0 = (int64_t)(tile - gridDim.x) * TOK;
          const int ntok = (int)min((int64_t)TOK, T - t0);
          for (int i = 0; i < ntok; ++i) {
            const uint32_t row = smem_u32(st + L.off_x + i * L.row_b);
            bulk_store(q + (t0 + i) * p.H * 64, row, L.q_b);
            bulk_store(k + (t0 + i) * p.Hkv * 64, row + L.q_b, L.kv_b);
            bulk_store(v + (t0 + i) * p.Hkv * 64, row + L.q_b + L.kv_b, L.kv_b);
          }
          bulk_commit_group();
        }
        if (!have) break;
      }
      bulk_wait_group0();
      (void)ok;
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
    const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
    const float qg = *p.qgain;
    int n = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++n) {
      const int s = n % kStages;
      if (!mbar_wait(smem_u32(&full[s]), (n / kStages) & 1, ab, 40)) break;
      uint8_t* st = smem + s * L.stage_b;
      const int64_t t0 = (int64_t)tile * TOK;
      const int ntok = (int)min((int64_t)TOK, T - t0);
      const int items = ntok * nslots * 4;
      for (int i = tid; i < items; i += kConsumers) {
        const int sub = i & 3, hs = i >> 2;
        const int tok = hs / nslots, slot = hs - tok * nslots;
        const int sw = (slot & 1) * 64;
        uint8_t* head = st + L.off_x + tok * L.row_b + slot * kHeadBytes;
        float x1[8], x2[8];
        load_pair(head, sub, sw, x1, x2);
        if (slot < nrot) {
          float cs[8], sn[8];
          load8s(reinterpret_cast<const float*>(st + L.off_cos + tok * 128) + sub * 8, cs);
          load8s(reinterpret_cast<const float*>(st + L.off_sin + tok * 128) + sub * 8, sn);
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float r1 = x1[j] * cs[j] - x2[j] * sn[j], r2 = x1[j] * sn[j] + x2[j] * cs[j];
            x1[j] = r1;
            x2[j] = r2;
            ss += r1 * r1 + r2 * r2;
          }
          float mul = 1.f;
          if (p.qknorm) {
            ss = quad_sum(ss);
            mul = rsqrtf(ss / 64 + kQkEps);
            if (slot < p.H) mul *= qg;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            x1[j] *= mul;
            x2[j] *= mul;
          }
        } else {
          float w1[8], w2[8];
          if (v1 != nullptr) load_pair(st + L.off_v1 + tok * L.kv_b + (slot - nrot) * kHeadBytes, sub, sw, w1, w2);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float u1 = v1 ? w1[j] : x1[j], u2 = v1 ? w2[j] : x2[j];
            x1[j] = vs * c * (a1 * x1[j] + a2 * u1);
            x2[j] = vs * c * (a1 * x2[j] + a2 * u2);
          }
        }
        store_pair(head, sub, sw, x1, x2);
      }
      fence_proxy_async();  // the rows were written by threads and are read by the bulk stores
      mbar_arrive(smem_u32(&done[s]));
    }
  }
  if (*cta_abort != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);  // loads that may still be in flight land before shared memory is released
  }
  __syncthreads();
}

template <int TOK>
__global__ void __launch_bounds__(kTileThreads, 2) qkv_post_bwd_tile_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                                                            const __nv_bfloat16* __restrict__ dv, const __nv_bfloat16* __restrict__ qkv,
                                                                            const __nv_bfloat16* __restrict__ v1, __nv_bfloat16* __restrict__ dqkv,
                                                                            float* __restrict__ dv1_out, float* __restrict__ partial, QkvPostParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float red[32];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  const TileLayout L = tile_layout(p.H, p.Hkv, TOK, true);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * L.stage_b);
  uint64_t* done = full + kStages;
  volatile int* cta_abort = reinterpret_cast<volatile int*>(done + kStages);
  const int nslots = p.H + 2 * p.Hkv, nrot = p.H + p.Hkv;
  const int64_t T = (int64_t)p.B * p.S;
  const int ntiles = (int)((T + TOK - 1) / TOK);
  const int tid = threadIdx.x;
  if (tid == 0) {
    *cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&done[s]), kConsumers);
    }
    fence_barrier_init();
  }
  __syncthreads();
  const AbortState ab{cta_abort, p.status, kWaitCycles};
  float acc_qg = 0.f, acc_dvU = 0.f, acc_dvv = 0.f, acc_dvv1 = 0.f;

  if (tid >= kConsumers) {
    if (tid == kConsumers) {
      int n = 0;
      for (int tile = blockIdx.x;; tile += gridDim.x, ++n) {
        const bool have = tile < ntiles;
        if (have) {
          const int s = n % kStages;
          bulk_wait_group_read0();
          uint8_t* st = smem + s * L.stage_b;
          const int64_t t0 = (int64_t)tile * TOK;
          const int ntok = (int)min((int64_t)TOK, T - t0);
          const uint32_t fb = smem_u32(&full[s]);
          mbar_expect_tx(fb, (uint32_t)ntok * (L.row_b + L.q_b + 2 * L.kv_b + (v1 != nullptr ? L.kv_b : 0) + 256));
          for (int i = 0; i < ntok; ++i) bulk_load(smem_u32(st + L.off_x + i * L.row_b), qkv + (t0 + i) * p.qkv_stride, L.row_b, fb);
          bulk_load(smem_u32(st + L.off_dq), dq + t0 * p.H * 64, ntok * L.q_b, fb);
          bulk_load(smem_u32(st + L.off_dk), dk + t0 * p.Hkv * 64, ntok * L.kv_b, fb);
          bulk_load(smem_u32(st + L.off_dv), dv + t0 * p.Hkv * 64, ntok * L.kv_b, fb);
          if (v1 != nullptr) bulk_load(smem_u32(st + L.off_v1), v1 + t0 * p.Hkv * 64, ntok * L.kv_b, fb);
          const int s0 = (int)(t0 % p.S);
          bulk_load(smem_u32(st + L.off_cos), p.cos + (size_t)s0 * 32, ntok * 128, fb);
          bulk_load(smem_u32(st + L.off_sin), p.sin + (size_t)s0 * 32, ntok * 128, fb);
        }
        if (n > 0) {
          const int m = n - 1, s = m % kStages;
          if (!mbar_wait(smem_u32(&done[s]), (m / kStages) & 1, ab, 43)) break;
          uint8_t* st = smem + s * L.stage_b;
          const int64_t t0 = (int64_t)(tile - gridDim.x) * TOK;
          const int ntok = (int)min((int64_t)TOK, T - t0);
          for (int i = 0; i < ntok; ++i) bulk_store(dqkv + (t0 + i) * p.qkv_stride, smem_u32(st + L.off_x + i * L.row_b), L.row_b);
          if (dv1_out != nullptr) {
            if (p.dv1_accumulate)
              bulk_reduce_add_f32(dv1_out + t0 * p.Hkv * 64, smem_u32(st + L.off_e), ntok * 2 * L.kv_b);
            else
              bulk_store(dv1_out + t0 * p.Hkv * 64, smem_u32(st + L.off_e), ntok * 2 * L.kv_b);
          }
          bulk_commit_group();
        }
        if (!have) break;
      }
      bulk_wait_group0();
    }
  } else {
    const float a1 = *p.alpha1, a2 = *p.alpha2, vs = *p.vscale;
    const float c = rsqrtf(a1 * a1 + a2 * a2 + kMixEps);
    const float qg = *p.qgain;
    const float kself = vs * c * (v1 ? a1 : (a1 + a2));
    const float kother = vs * c * a2;
    int n = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++n) {
      const int s = n % kStages;
      if (!mbar_wait(smem_u32(&full[s]), (n / kStages) & 1, ab, 42)) break;
      uint8_t* st = smem + s * L.stage_b;
      const int64_t t0 = (int64_t)tile * TOK;
      const int ntok = (int)min((int64_t)TOK, T - t0);
      const int items = ntok * nslots * 4;
      for (int i = tid; i < items; i += kConsumers) {
        const int sub = i & 3, hs = i >> 2;
        const int tok = hs / nslots, slot = hs - tok * nslots;
        const int sw = (slot & 1) * 64;
        uint8_t* head = st + L.off_x + tok * L.row_b + slot * kHeadBytes;
        float x1[8], x2[8], g1[8], g2[8];
        load_pair(head, sub, sw, x1, x2);
        if (slot < nrot) {
          const bool is_q = slot < p.H;
          const uint8_t* gh = is_q ? st + L.off_dq + tok * L.q_b + slot * kHeadBytes : st + L.off_dk + tok * L.kv_b + (slot - p.H) * kHeadBytes;
          load_pair(gh, sub, sw, g1, g2);
          float cs[8], sn[8];
          load8s(reinterpret_cast<const float*>(st + L.off_cos + tok * 128) + sub * 8, cs);
          load8s(reinterpret_cast<const float*>(st + L.off_sin + tok * 128) + sub * 8, sn);
          float ss = 0.f, dot = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float r1 = x1[j] * cs[j] - x2[j] * sn[j], r2 = x1[j] * sn[j] + x2[j] * cs[j];
            x1[j] = r1;
            x2[j] = r2;
            ss += r1 * r1 + r2 * r2;
            dot += r1 * g1[j] + r2 * g2[j];
          }
          if (p.qknorm) {
            ss = quad_sum(ss);
            dot = quad_sum(dot);
            const float r = rsqrtf(ss / 64 + kQkEps);
            const float gamma = is_q ? qg : 1.f;
            if (is_q && sub == 0) acc_qg += r * dot;
            const float ka = gamma * r, kb = gamma * r * r * r * dot / 64;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              g1[j] = ka * g1[j] - kb * x1[j];
              g2[j] = ka * g2[j] - kb * x2[j];
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // transpose of the rotation
            x1[j] = g1[j] * cs[j] + g2[j] * sn[j];
            x2[j] = -g1[j] * sn[j] + g2[j] * cs[j];
          }
        } else {
          const int kvh = slot - nrot;
          load_pair(st + L.off_dv + tok * L.kv_b + kvh * kHeadBytes, sub, sw, g1, g2);
          float w1[8], w2[8];
          if (v1 != nullptr) load_pair(st + L.off_v1 + tok * L.kv_b + kvh * kHeadBytes, sub, sw, w1, w2);
          float e1[8], e2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d1 = g1[j], d2 = g2[j];
            const float u1 = v1 ? w1[j] : x1[j], u2 = v1 ? w2[j] : x2[j];
            acc_dvU += d1 * (a1 * x1[j] + a2 * u1) + d2 * (a1 * x2[j] + a2 * u2);
            acc_dvv += d1 * x1[j] + d2 * x2[j];
            acc_dvv1 += d1 * u1 + d2 * u2;
            x1[j] = kself * d1;
            x2[j] = kself * d2;
            e1[j] = kother * d1;
            e2[j] = kother * d2;
          }
          if (dv1_out != nullptr) {
            float* e = reinterpret_cast<float*>(st + L.off_e + tok * 2 * L.kv_b + kvh * 2 * kHeadBytes);
            float4* ea = reinterpret_cast<float4*>(e + sub * 8);
            float4* eb = reinterpret_cast<float4*>(e + 32 + sub * 8);
            ea[0] = make_float4(e1[0], e1[1], e1[2], e1[3]);
            ea[1] = make_float4(e1[4], e1[5], e1[6], e1[7]);
            eb[0] = make_float4(e2[0], e2[1], e2[2], e2[3]);
            eb[1] = make_float4(e2[4], e2[5], e2[6], e2[7]);
          }
        }
        store_pair(head, sub, sw, x1, x2);
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&done[s]));
    }
  }
  if (*cta_abort != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
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

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

bool tile_path_ok(const QkvPostParams& p, bool bf16, int tok) {
  static const bool off = [] {
    const char* e = std::getenv("SEGPT_QKV_POST_TILE");
    return e != nullptr && e[0] == '0';
  }();
  return !off && bf16 && p.hd == 64 && p.pos == nullptr && p.status != nullptr && p.S % tok == 0 && (p.qkv_stride * 2) % 16 == 0 &&
         aligned16(p.cos) && aligned16(p.sin) && p.H >= 1 && p.Hkv >= 1;
}

int sm_count_cached() {
  static const int n = [] {
    int dev = 0, v = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v;
  }();
  return n;
}

}  // namespace

bool qkv_post_fwd_tile(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  if (!tile_path_ok(p, bf16, kFwdTok)) return false;
  for (const void* ptr : {qkv, v1, (const void*)q, (const void*)k, (const void*)v})
    if (!aligned16(ptr)) return false;
  const size_t smem = tile_smem_bytes(p.H, p.Hkv, kFwdTok, false);
  if (smem > 110 * 1024) return false;
  auto kern = qkv_post_fwd_tile_kernel<kFwdTok>;
  static size_t configured = 0;
  if (configured < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    configured = smem;
  }
  const int64_t T = (int64_t)p.B * p.S;
  const int64_t ntiles = (T + kFwdTok - 1) / kFwdTok;
  const int grid = (int)std::min<int64_t>(ntiles, 2 * sm_count_cached());
  kern<<<grid, kTileThreads, smem, st>>>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)v1, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                                         (__nv_bfloat16*)v, p);
  return cudaGetLastError() == cudaSuccess;
}

// Returns the number of rows of `partial` it filled (the grid), 0 if the shape is not served here.
int qkv_post_bwd_tile(const void* dq, const void* dk, const void* dv, const void* qkv, const void* v1, void* dqkv, float* dv1_out,
                      float* partial, int partial_rows, const QkvPostParams& p, bool bf16, cudaStream_t st) {
  if (!tile_path_ok(p, bf16, kBwdTok)) return 0;
  for (const void* ptr : {dq, dk, dv, qkv, v1, (const void*)dqkv, (const void*)dv1_out})
    if (!aligned16(ptr)) return 0;
  const size_t smem = tile_smem_bytes(p.H, p.Hkv, kBwdTok, true);
  if (smem > 110 * 1024) return 0;
  auto kern = qkv_post_bwd_tile_kernel<kBwdTok>;
  static size_t configured = 0;
  if (configured < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
    configured = smem;
  }
  const int64_t T = (int64_t)p.B * p.S;
  const int64_t ntiles = (T + kBwdTok - 1) / kBwdTok;
  const int grid = (int)std::min<int64_t>(std::min<int64_t>(ntiles, 2 * sm_count_cached()), partial_rows);
  if (grid < 1) return 0;
  kern<<<grid, kTileThreads, smem, st>>>((const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv,
                                         (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)v1, (__nv_bfloat16*)dqkv, dv1_out, partial, p);
  return cudaGetLastError() == cudaSuccess ? grid : 0;
}

}  // namespace seg
