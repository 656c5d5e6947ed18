// Causal flash-attention backward for sm_100a on tcgen05 tensor cores, native GQA, head_dim 64, bf16.
//
// Given q [B,S,H,hd], k/v [B,S,Hkv,hd], o, dO [B,S,H,hd], lse [B,H,S] (natural log) it produces dq [B,S,H,hd] and
// dk/dv [B,S,Hkv,hd].  With s = q k^T / sqrt(hd), P = exp(s - lse), D = rowsum(dO * o):
//   dV = P^T dO,   dP = dO V^T,   dS = P * (dP - D),   dQ = dS K / sqrt(hd),   dK = dS^T Q / sqrt(hd).
//
// One CTA owns one key tile (128 keys) of one (batch, kv head) and walks over the query heads that share the kv head and
// the query tiles at or after the key tile (causal).  Per step (one query tile of one head):
//   S  = Q K^T   and  dP = dO V^T          (both K-major x K-major, 128x128 fp32 accumulators in TMEM; TMEM lane = query, so the
//                                           thread that owns a lane holds the query's lse and D as two scalars)
//   P, dS -> bf16 into shared memory, rows = queries, in the 128-byte-swizzled layout
//   dV  += P^T  dO   (A = the P tile read as an MN-major operand, B = dO as MN-major operand; accumulates in TMEM over the walk)
//   dK  += dS^T Q    (same shapes, accumulates in TMEM over the whole walk)
//   dQ_i = dS  K     (A = the dS tile as a K-major operand, B = K as MN-major; fresh accumulator per step, drained through
//                     swizzled shared-memory boxes and TMA reductions (cp.reduce.async.bulk.tensor ... add) into an fp32 dQ
//                     buffer because other key tiles add to the same rows)
// TMEM: S 128 + dP 128 + dV 64 + dK 64 + dQ 2 x 64 = all 512 columns, one CTA per SM.
// Schedule (software pipeline over the steps n of the walk): the element-wise warps copy S^T / dP^T of step n into registers and
// release them at once, so the tensor core computes S^T / dP^T of step n+1 during the element-wise math of step n; P^T / dS^T
// are kept in registers until the dV / dK / dQ products of step n-1 have finished reading the operand buffers, so that those
// products also overlap the math; dQ alternates between two accumulators and step n-1's is drained while step n's products run.
// Roles (384 threads in three warpgroups): warp 0 TMA producer (K/V once; Q and dO tiles through a 3-stage ring, so that a tile is requested a
// whole step before its scores are issued; lse and D of the step's queries through a 2-stage ring of bulk copies; 4-D tensor
// maps, no multicast), warp 1 MMA issuer, warps 4-11 the element-wise stage (a key row and half of the query columns per thread).
// Two small kernels frame it: `attn_bwd_prep` (D and the negated lse in the exp2 domain) and `attn_bwd_finish` (dQ fp32 -> bf16).
// The reference relies on PyTorch SDPA's backward or a Triton kernel with fp32 atomics for dQ
// (transformer/ops/triton_flash_attn.py:104-201).  Every mbarrier wait is bounded.
#include <cuda.h>

#include "bounds.cuh"
#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace seg {

using namespace sm100;

constexpr int kBT = 128;   // keys per CTA and queries per step
constexpr int kBHD = 64;   // head dim
constexpr int kBwdThreads = 384;  // warpgroup 0: producer warp, MMA warp, two idle warps; warpgroups 1-2: 8 element-wise warps
constexpr int kBTile = kBT * kBHD * 2;   // 16 KB: one K, V, Q or dO tile
constexpr int kBPds = kBT * kBT * 2;     // 32 KB: P^T or dS^T (two 64-column atoms)
constexpr int kBDq = 8 * 32 * 32 * 4;     // 32 KB: one 32-row x 32-column fp32 box of dQ per element-wise warp
constexpr int kBStages = 3;              // Q / dO ring
// Register reallocation between the warpgroups.  The pool is what the CTA got at launch (three warpgroups at the kernel's
// register count, 168 under its launch bound), NOT the whole register file: a request beyond it blocks forever, so the
// launcher refuses to start the kernel unless kBRegsCtl + 2 * kBRegsEw fits into three times the compiled count.
constexpr int kBRegsCtl = 56, kBRegsEw = 224;
constexpr int kBwdSmem = 2 * kBTile /*K,V*/ + kBStages * 2 * kBTile /*Q,dO*/ + 2 * kBPds + kBDq + 2 * 2 * kBT * 4 /*lse2, D x 2*/ + 256;
static_assert(kBwdSmem <= 232448, "shared memory of the attention backward exceeds the per-block limit");

struct AttnBwdParams {
  int B, S, H, Hkv;
  float scale_log2;  // log2(e) / sqrt(hd)
  float scale;       // 1 / sqrt(hd)
  const float* lse2;  // [B,H,S] -lse * log2(e)
  const float* dsum;  // [B,H,S] rowsum(dO * o)
  float* dq_acc;      // [B,S,H,hd] fp32, zero-initialised
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int* status;
  long long* prof;  // optional [16]: cycles per stage of CTA (0,0), see the slot list at the launcher
};

#define SEG_PROF_ADD(slot, t)              \
  if (prof_on) {                           \
    const long long now_ = clock64();      \
    prof_s[slot] += now_ - t;              \
    t = now_;                              \
  }

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
// TMA reduction: global[box at coords] += shared box (fp32 add, element type and swizzle from the tensor map).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Eight consecutive keys of one query row: P = exp2(S * scale - lse2) and dS = P * (dP - D), as packed bf16.  nlse2 holds
// (-lse2, -lse2), so the exponent argument is one fused multiply-add on a pair; col0 is the first key of the eight and r the
// query row (kDiag: tile on the diagonal, keys after the query are masked).
template <bool kDiag>
__device__ __forceinline__ void bwd_math8(const uint32_t* s8, const uint32_t* dp8, uint64_t nlse2, uint64_t d2, uint64_t scale2, int col0, int r,
                                          bf16x8& pk, bf16x8& dk) {
  float pr[8], ds[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float x0, x1;
    unpack2(fma2(pack2(s8[2 * i], s8[2 * i + 1]), scale2, nlse2), x0, x1);
    float p0 = ex2_fast(x0), p1 = ex2_fast(x1);
    if (kDiag) {  // causal: the key must not follow the query
      if (col0 + 2 * i > r) p0 = 0.f;
      if (col0 + 2 * i + 1 > r) p1 = 0.f;
    }
    unpack2(mul2(pack2(p0, p1), sub2(pack2(dp8[2 * i], dp8[2 * i + 1]), d2)), ds[2 * i], ds[2 * i + 1]);
    pr[2 * i] = p0;
    pr[2 * i + 1] = p1;
  }
  pk = pack8(pr);
  dk = pack8(ds);
}

// Three warpgroups start with 168 registers per thread; the first one (producer, MMA issuer) hands most of its registers to
// the element-wise warpgroups, whose threads hold 128 accumulator values each (setmaxnreg: 56 + 2 x 224 = 3 x 168).
// kProf: with the stage timers (a separate instantiation, so that the production kernel carries none of their branches).
template <bool kProf>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_dq, AttnBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base: refuse instead of computing garbage
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 20);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + kBTile;
  uint8_t* sQdO = sV + kBTile;            // stage s: Q at s*32K, dO at s*32K + 16K
  uint8_t* sP = sQdO + kBStages * 2 * kBTile;
  uint8_t* sDS = sP + kBPds;
  uint8_t* sDQ = sDS + kBPds;  // [8 warps][32 rows][128 B], 128-byte swizzled boxes of the dQ tile
  float* sLse = reinterpret_cast<float*>(sDQ + kBDq);  // [2][128]
  float* sD = sLse + 2 * kBT;                            // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sD + 2 * kBT);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;    // [3]
  uint64_t* qdo_empty = bars + 4;   // [3]
  uint64_t* stat_full = bars + 7;   // [2]
  uint64_t* stat_empty = bars + 9;  // [2]
  uint64_t* s_full = bars + 11;     // S^T and dP^T are in TMEM
  uint64_t* pds_full = bars + 12;   // P^T and dS^T are in shared memory
  uint64_t* mma_done = bars + 13;   // dV/dK/dQ MMAs of the step finished
  uint64_t* s_read = bars + 14;     // S^T and dP^T of the step are in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  long long* prof_s = reinterpret_cast<long long*>(bars + 16);
  const bool prof_cta = kProf && p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = p.S / kBT;
  const int jt = blockIdx.x;  // key tile; small j = long walk, scheduled first
  const int bg = blockIdx.y;
  const int b = bg / p.Hkv, g = bg % p.Hkv;
  const int group = p.H / p.Hkv;
  const int per_head = n_t - jt;       // query tiles jt .. n_t-1
  const int n_steps = group * per_head;
  const AbortState ab{cta_abort, p.status};

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < kBStages; ++s) {
      mbar_init(smem_u32(&qdo_full[s]), 1);
      mbar_init(smem_u32(&qdo_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&stat_full[s]), 1);
      mbar_init(smem_u32(&stat_empty[s]), 8);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(pds_full), 8);
    mbar_init(smem_u32(mma_done), 1);
    mbar_init(smem_u32(s_read), 8);
    for (int i = 0; i < 16; ++i) prof_s[i] = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_do);
    prefetch_tensormap(&map_dq);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 320, tm_dq = tmem_base + 384;  // dQ: two accumulators of 64 columns

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kBRegsCtl));
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      // Two queues, served as their slots become free: the Q / dO tiles (three stages, released by the products that read them)
      // and the per-query statistics (two stages, released by the element-wise warps).
      if (elect_one()) {
        mbar_expect_tx(smem_u32(kv_full), 2 * kBTile);
        tma_load_4d(smem_u32(sK), &map_k, smem_u32(kv_full), 0, g, jt * kBT, b);
        tma_load_4d(smem_u32(sV), &map_v, smem_u32(kv_full), 0, g, jt * kBT, b);
        int next_q = 0, next_s = 0;
        long long t0 = clock64();
        while (next_q < n_steps || next_s < n_steps) {
          bool progress = false;
          if (next_s < n_steps && mbar_test_wait(smem_u32(&stat_empty[next_s & 1]), ((next_s >> 1) & 1) ^ 1)) {
            const int h = g * group + next_s / per_head, it = jt + next_s % per_head;
            const size_t stat = ((size_t)b * p.H + h) * p.S + (size_t)it * kBT;  // 128 floats: 512-byte aligned
            const uint32_t fb = smem_u32(&stat_full[next_s & 1]);
            mbar_expect_tx(fb, 2 * kBT * 4);
            bulk_load(smem_u32(sLse + (next_s & 1) * kBT), p.lse2 + stat, kBT * 4, fb);
            bulk_load(smem_u32(sD + (next_s & 1) * kBT), p.dsum + stat, kBT * 4, fb);
            ++next_s;
            progress = true;
          }
          if (next_q < n_steps && mbar_test_wait(smem_u32(&qdo_empty[next_q % kBStages]), ((next_q / kBStages) & 1) ^ 1)) {
            const int st = next_q % kBStages;
            const int h = g * group + next_q / per_head, it = jt + next_q % per_head;
            const uint32_t fb = smem_u32(&qdo_full[st]);
            mbar_expect_tx(fb, 2 * kBTile);
            tma_load_4d(smem_u32(sQdO + st * 2 * kBTile), &map_q, fb, 0, h, it * kBT, b);
            tma_load_4d(smem_u32(sQdO + st * 2 * kBTile + kBTile), &map_do, fb, 0, h, it * kBT, b);
            ++next_q;
            progress = true;
          }
          if (progress) {
            t0 = clock64();
          } else {
            if (*ab.cta_abort != 0) break;
            if (clock64() - t0 > ab.limit) {
              *ab.cta_abort = 1;
              atomicCAS(ab.global_status, 0, 21);
              break;
            }
            __nanosleep(40);
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (elect_one()) {
        constexpr uint32_t id_s = make_idesc_bf16(kBT, kBT, false, false);    // Q / dO (K-major) x K / V (K-major)
        constexpr uint32_t id_kv = make_idesc_bf16(kBT, kBHD, true, true);    // P^T / dS^T (MN-major views of P / dS) x dO / Q (MN-major)
        constexpr uint32_t id_dq = make_idesc_bf16(kBT, kBHD, false, true);   // dS (K-major) x K (MN-major)
        const uint32_t sk = smem_u32(sK), sv = smem_u32(sV), sp = smem_u32(sP), sds = smem_u32(sDS);
        // Descriptors advance by adding to their address field (units of 16 bytes); the loops are not unrolled so that this
        // thread stays within the few registers its warpgroup keeps.
        const uint64_t d_k = make_smem_desc(sk, 16, 1024), d_v = make_smem_desc(sv, 16, 1024);
        auto issue_s = [&](int n) {
          const uint32_t sq = smem_u32(sQdO + (n % kBStages) * 2 * kBTile);
          const uint64_t d_q = make_smem_desc(sq, 16, 1024), d_do = make_smem_desc(sq + kBTile, 16, 1024);
#pragma unroll 2
          for (int k = 0; k < kBHD / 16; ++k) umma_bf16(tm_s, d_q + 2 * k, d_k + 2 * k, id_s, k > 0);
#pragma unroll 2
          for (int k = 0; k < kBHD / 16; ++k) umma_bf16(tm_dp, d_do + 2 * k, d_v + 2 * k, id_s, k > 0);
          umma_commit(smem_u32(s_full));
        };
        const bool prof_on = prof_cta;
        long long t = prof_on ? clock64() : 0;
        bool ok = mbar_wait(smem_u32(kv_full), 0, ab, 22) && mbar_wait(smem_u32(&qdo_full[0]), 0, ab, 23);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
        for (int n = 0; n < n_steps && ok; ++n) {
          const int st = n % kBStages;
          const uint32_t sq = smem_u32(sQdO + st * 2 * kBTile), sdo = sq + kBTile;
          // Two jobs per step, served in the order in which their inputs become ready: the scores of step n+1 (Q / dO landed
          // and the element-wise warps hold step n's accumulators in registers) and the products of step n (operands written).
          bool s_done = !(n + 1 < n_steps), p_done = false;
          const long long t0 = clock64();
          while (!(s_done && p_done)) {
            if (!s_done && mbar_test_wait(smem_u32(&qdo_full[(n + 1) % kBStages]), ((n + 1) / kBStages) & 1) &&
                mbar_test_wait(smem_u32(s_read), n & 1)) {
              SEG_PROF_ADD(8, t)
              tc_fence_after();
              issue_s(n + 1);
              s_done = true;
              SEG_PROF_ADD(10, t)
            }
            if (!p_done && mbar_test_wait(smem_u32(pds_full), n & 1)) {
              SEG_PROF_ADD(11, t)
              tc_fence_after();
              const uint32_t dq_acc = tm_dq + (n & 1) * kBHD;
              // P / dS tiles: rows = queries (128 bytes per 64 keys, two 64-key atoms 16 KB apart).  As A^T operands (M = keys, contraction
              // over queries) they are MN-major: 16 query rows = 2048 bytes per k-step; as the A operand of dQ (M = queries, contraction
              // over keys) K-major: 16 keys = 32 bytes per k-step inside an atom.
              const uint64_t d_p_mn = make_smem_desc(sp, kBT * 128, 1024), d_ds_mn = make_smem_desc(sds, kBT * 128, 1024);
              const uint64_t d_do_mn = make_smem_desc(sdo, kBTile, 1024), d_q_mn = make_smem_desc(sq, kBTile, 1024);
#pragma unroll 2
              for (int k = 0; k < kBT / 16; ++k) {  // contraction over the 128 queries of the step
                umma_bf16(tm_dv, d_p_mn + (uint64_t)(k * 128), d_do_mn + (uint64_t)(k * 128), id_kv, (n > 0 || k > 0) ? 1u : 0u);
                umma_bf16(tm_dk, d_ds_mn + (uint64_t)(k * 128), d_q_mn + (uint64_t)(k * 128), id_kv, (n > 0 || k > 0) ? 1u : 0u);
              }
              const uint64_t d_ds = make_smem_desc(sds, 16, 1024), d_k_mn = make_smem_desc(sk, kBTile, 1024);
#pragma unroll 2
              for (int k = 0; k < kBT / 16; ++k)  // contraction over the 128 keys
                umma_bf16(dq_acc, d_ds + (uint64_t)(((k >> 2) * (kBT * 128) + (k & 3) * 32) >> 4), d_k_mn + (uint64_t)(k * 128), id_dq, k > 0);
              umma_commit(smem_u32(mma_done));
              umma_commit(smem_u32(&qdo_empty[st]));
              p_done = true;
              SEG_PROF_ADD(12, t)
            }
            if (!(s_done && p_done)) {
              if (*ab.cta_abort != 0) { ok = false; break; }
              if (clock64() - t0 > ab.limit) {
                *ab.cta_abort = 1;
                atomicCAS(ab.global_status, 0, 24);
                ok = false;
                break;
              }
            }
          }
        }
      }
      __syncwarp();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kBRegsEw));
    // ------------------------------------------------------------------ element-wise stage
    // Eight warps: warp % 4 selects the TMEM sub-partition (32 query rows), the two warps of a sub-partition split the
    // 128 key columns in halves, so that every scheduler has two warps to alternate between.
    const int sub = warp & 3;
    const int half = (warp - 4) >> 2;
    const int r = sub * 32 + lane;  // query row inside the tile == TMEM lane; the key row in the dV / dK epilogue
    const uint32_t lane_addr = (uint32_t)(sub * 32) << 16;
    uint8_t* box = sDQ + (warp - 4) * 4096;
    bool ok = true;
    const bool prof_on = prof_cta && threadIdx.x == 128;
    long long t = prof_on ? clock64() : 0;
    // dQ of step m (lane = query row; each half takes 32 of the 64 columns): TMEM -> registers -> this warp's swizzled 4 KB
    // box in shared memory; after the next proxy fence one TMA reduction adds the box to the fp32 accumulator (other key
    // tiles add to the same rows).
    uint32_t qv[32];
    auto load_dq = [&](int m) {  // issue the TMEM load of this warp's 32 x 32 piece of dQ of step m; stage_dq waits for it
      tmem_ld_32x32(tm_dq + (m & 1) * kBHD + lane_addr + half * 32, qv);
    };
    auto stage_dq = [&](int m) {
      if (m > 0) {  // the previous reduction must have read the box
        if (lane == 0) bulk_wait_read0();
        __syncwarp();
      }
      tmem_ld_wait_regs(qv);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 f = make_float4(__uint_as_float(qv[c * 4]) * p.scale, __uint_as_float(qv[c * 4 + 1]) * p.scale,
                                     __uint_as_float(qv[c * 4 + 2]) * p.scale, __uint_as_float(qv[c * 4 + 3]) * p.scale);
        *reinterpret_cast<float4*>(box + lane * 128 + ((c ^ (lane & 7)) << 4)) = f;
      }
    };
    auto reduce_dq = [&](int m) {  // by one lane, after the fence that follows stage_dq
      const int h = g * group + m / per_head, it = jt + m % per_head;
      tma_reduce_add_4d(&map_dq, smem_u32(box), half * 32, h, it * kBT + sub * 32, b);
      bulk_commit();
    };
    for (int n = 0; n < n_steps && ok; ++n) {
      const int it = jt + n % per_head;
      const int st = n & 1;
      if (!mbar_wait(smem_u32(&stat_full[st]), (n >> 1) & 1, ab, 28)) { ok = false; break; }
      if (!mbar_wait(smem_u32(s_full), n & 1, ab, 26)) { ok = false; break; }
      SEG_PROF_ADD(0, t)
      tc_fence_after();
      const bool diag = (it == jt);
      const float nlse = sLse[st * kBT + r], dq_row = sD[st * kBT + r];  // this query's -lse2 and D
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&stat_empty[st]));  // the statistics of the step have been read
      uint32_t sv_[64], dpv[64];  // this thread's query row, 64 key columns of S and dP
      tmem_ld_32x32(tm_s + lane_addr + half * 64, sv_);
      tmem_ld_32x32(tm_s + lane_addr + half * 64 + 32, sv_ + 32);
      tmem_ld_32x32(tm_dp + lane_addr + half * 64, dpv);
      tmem_ld_32x32(tm_dp + lane_addr + half * 64 + 32, dpv + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_read));  // the next S / dP may overwrite the accumulators
      SEG_PROF_ADD(1, t)
      bf16x8 pk[8], dk8[8];  // P and dS of the row as packed bf16, held until the operand buffers are free
      const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), nlse2 = pack2(nlse, nlse), d2 = pack2(dq_row, dq_row);
      if (diag) {
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16)
          bwd_math8<true>(sv_ + c16 * 8, dpv + c16 * 8, nlse2, d2, scale2, half * 64 + c16 * 8, r, pk[c16], dk8[c16]);
      } else {
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16)
          bwd_math8<false>(sv_ + c16 * 8, dpv + c16 * 8, nlse2, d2, scale2, half * 64 + c16 * 8, r, pk[c16], dk8[c16]);
      }
      SEG_PROF_ADD(2, t)
      if (n > 0) {  // the products of step n-1 have read P^T / dS^T, and its dQ is complete
        if (!mbar_wait(smem_u32(mma_done), (n - 1) & 1, ab, 27)) { ok = false; break; }
        tc_fence_after();
      }
      SEG_PROF_ADD(3, t)
      if (n > 0) load_dq(n - 1);  // in flight during the operand stores
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        const int chunk = half * 8 + c16;  // 16-byte chunk index along the row (16 chunks of 8 columns)
        const int off = (chunk >> 3) * (kBT * 128) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
        *reinterpret_cast<bf16x8*>(sP + off) = pk[c16];
        *reinterpret_cast<bf16x8*>(sDS + off) = dk8[c16];
      }
      if (n > 0) stage_dq(n - 1);  // same proxy fence as the operands
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(pds_full));
        if (n > 0) reduce_dq(n - 1);  // runs while the tensor core works on this step's products
      }
      SEG_PROF_ADD(4, t)
    }
    if (ok && n_steps > 0) {
      if (!mbar_wait(smem_u32(mma_done), (n_steps - 1) & 1, ab, 27)) ok = false;
      tc_fence_after();
      if (ok) {
        load_dq(n_steps - 1);
        stage_dq(n_steps - 1);
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) reduce_dq(n_steps - 1);
      }
      SEG_PROF_ADD(6, t)
    }
    if (ok && n_steps > 0) {
      // dV (first four warps) and dK (the other four) of this key tile: the last mma_done has been waited for above
      const size_t row = (((size_t)b * p.S + (size_t)jt * kBT + r) * p.Hkv + g) * kBHD;
      const uint32_t src = half == 0 ? tm_dv : tm_dk;
      __nv_bfloat16* dst = (half == 0 ? p.dv : p.dk) + row;
      const float mul = half == 0 ? 1.f : p.scale;
#pragma unroll
      for (int c = 0; c < kBHD / 32; ++c) {
        uint32_t a[32];
        tmem_ld_32x32(src + lane_addr + c * 32, a);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(a[e]) * mul;
        if (SEG_IN_BOUNDS(p.status, 33, row + c * 32, 32, (size_t)p.B * p.S * p.Hkv * kBHD)) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) reinterpret_cast<bf16x8*>(dst + c * 32)[q4] = pack8(f + q4 * 8);
        }
      }
    }
  }

  if (warp >= 4 && lane == 0) bulk_wait0();  // outstanding dQ reductions of this warp are complete before the CTA ends
  if (*cta_abort != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
  if (prof_cta && threadIdx.x == 0) {
    for (int i = 0; i < 15; ++i) p.prof[i] = prof_s[i];
    p.prof[15] = n_steps;
  }
}

// D[b,h,s] = sum_hd dO * o, lse2 = -lse * log2(e).  Eight lanes per (token, head) row of 64 elements: one 16-byte load per
// lane and tensor, four consecutive rows (512 contiguous bytes) per warp.
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                          const float* __restrict__ lse, float* __restrict__ dsum,
                                                          float* __restrict__ lse2, int B, int S, int H) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t row = tid >> 3;  // index over [B,S,H]
  const int part = (int)(tid & 7);
  const size_t rows = (size_t)B * S * H;
  float s = 0.f;
  if (row < rows) {
    float fa[8], fg[8];
    load8<__nv_bfloat16>(o + row * kBHD + part * 8, fa);
    load8<__nv_bfloat16>(d_o + row * kBHD + part * 8, fg);
#pragma unroll
    for (int e = 0; e < 8; ++e) s = fmaf(fa[e], fg[e], s);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (row < rows && part == 0) {
    const int h = (int)(row % H);
    const size_t bs = row / H;
    const size_t sidx = bs % S, b = bs / S;
    const size_t out = (b * H + h) * S + sidx;
    dsum[out] = s;
    lse2[out] = -lse[out] * 1.4426950408889634f;  // negated: the exponent argument becomes one multiply-add
  }
}

__global__ void __launch_bounds__(256) attn_bwd_finish_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float f[8];
  load8<float>(acc + i * 8, f);
  store8<__nv_bfloat16>(dq + i * 8, f);
}

typedef CUresult (*EncodeTiledFnB)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_map_bshd_b(CUtensorMap* map, const void* base, int B, int S, int heads, int hd) {
  static EncodeTiledFnB fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFnB>(ptr);
  }
  cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)heads * hd * 2, (cuuint64_t)S * heads * hd * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int make_map_dq_acc(CUtensorMap* map, const float* base, int B, int S, int H, int hd) {
  static EncodeTiledFnB fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFnB>(ptr);
  }
  cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)hd * 4, (cuuint64_t)H * hd * 4, (cuuint64_t)S * H * hd * 4};
  cuuint32_t box[4] = {32, 1, 32, 1};  // 32 fp32 = 128 bytes: one swizzle row
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// prof (optional, 16 int64): cycles that one element-wise thread and the MMA thread of the CTA with the longest walk spent per
// stage - element-wise: 0 wait S/dP, 1 accumulators -> registers, 2 math, 3 wait previous products, 4 store operands, stage
// the previous dQ, fence, signal, issue the dQ reduction (about a third each), 6 last dQ; MMA: 8 wait Q/dO, 9 wait accumulators read, 10 issue S^T/dP^T, 11 wait operands,
// 12 issue dV/dK/dQ; 15 = steps walked.
int attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
             float* dq_acc, float* dsum, float* lse2, int B, int S, int H, int Hkv, int hd, int* status, cudaStream_t st,
             long long* prof) {
  if (hd != kBHD || S % kBT != 0 || H % Hkv != 0) return -10;
  CUtensorMap mq, mk, mv, mdo, mdq;
  int r = make_map_dq_acc(&mdq, dq_acc, B, S, H, hd);
  if (r == 0) r = make_map_bshd_b(&mq, q, B, S, H, hd);
  if (r == 0) r = make_map_bshd_b(&mk, k, B, S, Hkv, hd);
  if (r == 0) r = make_map_bshd_b(&mv, v, B, S, Hkv, hd);
  if (r == 0) r = make_map_bshd_b(&mdo, d_o, B, S, H, hd);
  if (r != 0) return 100 + r;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem) != cudaSuccess) return -2;
    cudaFuncAttributes fa, fb;
    if (cudaFuncGetAttributes(&fa, attn_bwd_kernel<false>) != cudaSuccess || cudaFuncGetAttributes(&fb, attn_bwd_kernel<true>) != cudaSuccess) return -2;
    const int regs = fa.numRegs < fb.numRegs ? fa.numRegs : fb.numRegs;
    if (kBRegsCtl + 2 * kBRegsEw > 3 * regs) return -6;  // the register requests would never be granted
    configured = true;
  }
  const size_t n = (size_t)B * S * H * hd;
  if (cudaMemsetAsync(dq_acc, 0, n * sizeof(float), st) != cudaSuccess) return -4;
  const int rows = B * S * H;
  attn_bwd_prep_kernel<<<(unsigned)(((size_t)rows * 8 + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o),
                                                                lse, dsum, lse2, B, S, H);
  AttnBwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.scale = 1.f / sqrtf((float)hd);
  p.scale_log2 = 1.4426950408889634f * p.scale;
  p.lse2 = lse2;
  p.dsum = dsum;
  p.dq_acc = dq_acc;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.status = status;
  p.prof = prof;
  dim3 grid(S / kBT, B * Hkv);
  if (prof != nullptr)
    attn_bwd_kernel<true><<<grid, kBwdThreads, kBwdSmem, st>>>(mq, mk, mv, mdo, mdq, p);
  else
    attn_bwd_kernel<false><<<grid, kBwdThreads, kBwdSmem, st>>>(mq, mk, mv, mdo, mdq, p);
  attn_bwd_finish_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace seg
