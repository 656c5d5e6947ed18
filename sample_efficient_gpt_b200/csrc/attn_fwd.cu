// Causal flash-attention forward for sm_100a on tcgen05 tensor cores, native GQA, head_dim 64, bf16.
//
//   S = Q K^T / sqrt(hd) (causal), P = softmax(S), O = P V, LSE = log sum exp(S)      per (batch, query head)
// q [B,S,H,hd], k/v [B,S,Hkv,hd] (token-major, as written by the qkv post-processing kernel), o like q, lse [B,H,S].
// Any S >= 1: the last 128-row tile may be partial (TMA fills rows beyond S with zeros; the causal mask keeps their
// keys out of every real query's softmax; their outputs are not stored).
//
// One CTA per (256 queries, batch, head), one CTA per SM.  The 256 queries are two tiles of 128 rows, each with its own
// score accumulator S (128x128 fp32) and output accumulator O (128x64 fp32) in TMEM and its own softmax warpgroup; both
// tiles walk over the same K/V tiles, which are loaded once.  While one warpgroup runs the softmax of its tile, the tensor
// core computes the other tile's products.  Roles (384 threads in three warpgroups):
//   warpgroup 0, warps 0 and 1: control - one thread per query tile x issues its MMAs: S_x(j) = Q_x K_j^T and, once the
//              warpgroup has written P_x(j) to shared memory, O_x += P_x(j) V_j; the thread of warp 0 also issues the TMA
//              loads (both Q tiles once, K/V tiles of 128 keys into a 3-stage ring; 4-D tensor maps, 128-byte swizzle, no
//              multicast).  V is consumed in place as an MN-major operand,
//              K as a K-major one.  The queues are served in the order their inputs become ready; Q K^T of tile j+1 runs
//              ahead of the softmax of tile j.  The warpgroup gives most of its registers to the other two (setmaxnreg).
//   warpgroups 1, 2: softmax of query tile 0 / 1 - every thread owns one query row: reads S with tcgen05.ld into registers
//              (and releases the accumulator at once), online max/sum in the exp2 domain with packed fp32-pair arithmetic,
//              writes P as bf16 into the swizzled operand layout.  O is rescaled lazily.
// The reference uses PyTorch SDPA on repeated K/V heads (transformer/attention.py:207-236) or a Triton kernel
// (transformer/ops/triton_flash_attn.py:12-101).
// Every mbarrier wait is bounded; on expiry the CTA unwinds, frees TMEM and sets the status word.
#include <cuda.h>

#include <type_traits>

#include "bounds.cuh"
#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace seg {

using namespace sm100;

constexpr int kAQ = 128;   // queries per softmax warpgroup (two per CTA)
constexpr int kAK = 128;   // keys per tile
constexpr int kAHD = 64;   // head dim
constexpr int kAStages = 3;  // K/V ring
constexpr int kAttnThreads = 384;
constexpr int kTileBytes = kAK * kAHD * 2;  // 16 KB: one Q, K or V tile
constexpr int kPBytes = kAQ * kAK * 2;      // 32 KB: P as two 64-column swizzle atoms
constexpr int kAttnSmem = 2 * kTileBytes /*Q x 2*/ + kAStages * 2 * kTileBytes /*K,V*/ + 2 * kPBytes + 256;
// Register reallocation between the warpgroups.  The pool is what the CTA got at launch (three warpgroups at the kernel's
// register count, 168 under its launch bound): a request beyond it blocks forever, so the launcher refuses to start the
// kernel unless kARegsCtl + 2 * kARegsSm fits into three times the compiled count.
constexpr int kARegsCtl = 56, kARegsSm = 224;
constexpr int kAEmu = 1;  // pairs out of every four whose exp2 runs as a polynomial on the FMA pipe (measured: 0 -> 341, 1 -> 346, 2 -> 336 TFLOP/s)

struct AttnParams {
  int B, S, H, Hkv;
  float scale_log2;  // log2(e) / sqrt(hd)
  __nv_bfloat16* o;
  float* lse;
  int* status;
  long long* prof;  // optional [16]: cycles per stage of CTA (0,0), see the slot list at the launcher
};

// Stage timers: one thread per role of one CTA adds clock64() differences to shared-memory slots.
#define SEG_PROF_ADD(slot, t)              \
  if (prof_on) {                           \
    const long long now_ = clock64();      \
    prof_s[slot] += now_ - t;              \
    t = now_;                              \
  }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kProf: with the stage timers (a separate instantiation, so that the production kernel carries none of their branches).
template <bool kProf>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base: refuse instead of computing garbage
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 10);
    return;
  }
  uint8_t* sQ = smem;                        // tile x at x*16K
  uint8_t* sKV = sQ + 2 * kTileBytes;        // stage s: K at s*32K, V at s*32K + 16K
  uint8_t* sP = sKV + kAStages * 2 * kTileBytes;  // tile x at x*32K
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [3]
  uint64_t* kv_empty = bars + 4;  // [3]
  uint64_t* s_full = bars + 7;    // [2] per query tile
  uint64_t* s_empty = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* pv_full = bars + 13;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  long long* prof_s = reinterpret_cast<long long*>(bars + 16);
  const bool prof_cta = kProf && p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (p.S + 2 * kAQ - 1) / (2 * kAQ);
  const int qb = n_qb - 1 - (int)blockIdx.x;  // heavy (late) query blocks first
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int kvh = h / (p.H / p.Hkv);
  // causal: query tile x (rows (2 qb + x) * 128 ...) walks over key tiles 0 .. 2 qb + x; a second tile that starts beyond the
  // sequence does not exist
  const int n_a = 2 * qb + 1;
  const int n_b = ((2 * qb + 1) * kAQ < p.S) ? 2 * qb + 2 : 0;
  const AbortState ab{cta_abort, p.status};

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int i = 0; i < 16; ++i) prof_s[i] = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), n_b > 0 ? 2 : 1);  // released by the P V of every tile that reads the stage
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&s_full[x]), 1);
      mbar_init(smem_u32(&s_empty[x]), 4);
      mbar_init(smem_u32(&p_full[x]), 4);
      mbar_init(smem_u32(&pv_full[x]), 1);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;  // columns [0,256): S of tile 0 / 1; [256,384): O of tile 0 / 1

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kARegsCtl));
    // ------------------------------------------------------------------ control threads: warp x serves query tile x
    // (warp 0 also the loads); two warps so that the issue work of the two tiles sits on two schedulers
    const int x = warp;
    const int n_x = x == 0 ? n_a : n_b;
    if (warp < 2 && (x == 0 || n_x > 0) && elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kAQ, kAK, false, false);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = make_idesc_bf16(kAQ, kAHD, false, true);  // P (K-major) x V (MN-major)
      const bool prof_on = prof_cta && x == 0;
      long long t = prof_on ? clock64() : 0;
      const int n_load = x == 0 ? (n_a > n_b ? n_a : n_b) : 0;
      if (x == 0) {
        mbar_expect_tx(smem_u32(q_full), 2 * kTileBytes);
        tma_load_4d(smem_u32(sQ), &map_q, smem_u32(q_full), 0, h, 2 * qb * kAQ, b);
        tma_load_4d(smem_u32(sQ) + kTileBytes, &map_q, smem_u32(q_full), 0, h, (2 * qb + 1) * kAQ, b);  // zeros beyond the sequence
      }
      const uint64_t d_q = make_smem_desc(smem_u32(sQ) + x * kTileBytes, 16, 1024);
      const uint64_t d_p = make_smem_desc(smem_u32(sP) + x * kPBytes, 16, 1024);
      const uint32_t t_s = tmem_base + x * kAK, t_o = tmem_base + 2 * kAK + x * kAHD;
      const uint32_t b_s_full = smem_u32(&s_full[x]), b_s_empty = smem_u32(&s_empty[x]), b_p_full = smem_u32(&p_full[x]),
                     b_pv_full = smem_u32(&pv_full[x]);
      int next_load = 0, next_qk = 0, next_pv = 0;
      bool q_in = false;
      long long t0 = clock64();
      while (next_pv < n_x || next_load < n_load) {
        bool progress = false;
        if (next_load < n_load && mbar_test_wait(smem_u32(&kv_empty[next_load % kAStages]), ((next_load / kAStages) & 1) ^ 1)) {
          const int st = next_load % kAStages;
          const uint32_t fb = smem_u32(&kv_full[st]);
          mbar_expect_tx(fb, 2 * kTileBytes);
          tma_load_4d(smem_u32(sKV + st * 2 * kTileBytes), &map_k, fb, 0, kvh, next_load * kAK, b);
          tma_load_4d(smem_u32(sKV + st * 2 * kTileBytes + kTileBytes), &map_v, fb, 0, kvh, next_load * kAK, b);
          ++next_load;
          progress = true;
          SEG_PROF_ADD(8, t)
        }
        if (!q_in) q_in = mbar_test_wait(smem_u32(q_full), 0);
        if (next_qk < n_x && q_in && mbar_test_wait(smem_u32(&kv_full[next_qk % kAStages]), (next_qk / kAStages) & 1) &&
            (next_qk == 0 || mbar_test_wait(b_s_empty, (next_qk - 1) & 1))) {
          const uint64_t d_k = make_smem_desc(smem_u32(sKV + (next_qk % kAStages) * 2 * kTileBytes), 16, 1024);
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kAHD / 16; ++k) umma_bf16(t_s, d_q + 2 * k, d_k + 2 * k, idesc_s, k > 0);
          umma_commit(b_s_full);
          ++next_qk;
          progress = true;
          SEG_PROF_ADD(10, t)
        }
        if (next_pv < next_qk && mbar_test_wait(b_p_full, next_pv & 1)) {
          const int st = next_pv % kAStages;
          const uint64_t d_v = make_smem_desc(smem_u32(sKV + st * 2 * kTileBytes) + kTileBytes, kTileBytes, 1024);
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kAK / 16; ++k)
            umma_bf16(t_o, d_p + (uint64_t)(((k >> 2) * (kAQ * 128) + (k & 3) * 32) >> 4), d_v + (uint64_t)(k * 128), idesc_pv,
                      (next_pv > 0 || k > 0) ? 1u : 0u);
          umma_commit(b_pv_full);
          umma_commit(smem_u32(&kv_empty[st]));
          ++next_pv;
          progress = true;
          SEG_PROF_ADD(12, t)
        }
        if (progress) {
          t0 = clock64();
        } else {
          if (*ab.cta_abort != 0) break;
          if (clock64() - t0 > ab.limit) {
            *ab.cta_abort = 1;
            atomicCAS(ab.global_status, 0, 12);
            break;
          }
          SEG_PROF_ADD(9, t)
        }
      }
    }
    __syncwarp();
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kARegsSm));
    // ------------------------------------------------------------------ softmax warpgroups: one query row per thread
    // O accumulates in TMEM across key tiles.  It is rescaled only when the running maximum grew by more than 2^8
    // since the last rescale (probabilities are then at most 256, harmless for bf16 operands and fp32 sums), which
    // after the first tiles is rare; the decision is taken per warp because TMEM loads/stores are warp-collective.
    const int x = (warp >> 2) - 1;  // query tile of this warpgroup
    const int n_tiles = x == 0 ? n_a : n_b;
    const int qt = 2 * qb + x;
    const int sub = warp & 3;
    const int r = sub * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(sub * 32) << 16;
    const uint32_t tmem_s = tmem_base + x * kAK, tmem_pv = tmem_base + 2 * kAK + x * kAHD;
    uint8_t* sPx = sP + x * kPBytes;
    const uint32_t b_s_full = smem_u32(&s_full[x]), b_s_empty = smem_u32(&s_empty[x]), b_p_full = smem_u32(&p_full[x]),
                   b_pv_full = smem_u32(&pv_full[x]);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const bool prof_on = prof_cta && threadIdx.x == 128;
    long long t = prof_on ? clock64() : 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(b_s_full, j & 1, ab, 17)) { ok = false; break; }
      SEG_PROF_ADD(0, t)
      tc_fence_after();
      uint32_t v[kAK];
#pragma unroll
      for (int c = 0; c < kAK / 32; ++c) tmem_ld_32x32(tmem_s + lane_addr + c * 32, v + c * 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(b_s_empty);  // S is in registers: the next Q K^T may overwrite it
      SEG_PROF_ADD(1, t)
      const bool diag = (j == qt);
      // four independent chains of three-input maxima: a single chain of dependent operations would leave the warps that share
      // a scheduler stalled on instruction latency
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (diag) {
#pragma unroll
        for (int e = 0; e < kAK; ++e)
          if (e <= r) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v[e]));
      } else {
#pragma unroll
        for (int e = 0; e < kAK; e += 8) {
#pragma unroll
          for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], __uint_as_float(v[e + 2 * c]), __uint_as_float(v[e + 2 * c + 1]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_ref, mx * p.scale_log2);
      const bool need = (m_new - m_ref) > 8.f;  // true on the first tile (m_ref = -inf)
      SEG_PROF_ADD(2, t)
      // P V(j-1) must have finished before O is rescaled or the P tile is overwritten.  The rescale is rare after the first
      // tiles, so the wait normally comes after the exponentials, which are kept in registers meanwhile.
      bool pv_waited = (j == 0);
      SEG_PROF_ADD(3, t)
      if (__any_sync(0xffffffffu, need)) {
        const float m_tgt = need ? m_new : m_ref;
        if (j > 0) {
          if (!mbar_wait(b_pv_full, (j - 1) & 1, ab, 18)) { ok = false; break; }
          tc_fence_after();
          pv_waited = true;
          const float alpha = ex2_approx(m_ref - m_tgt);
#pragma unroll
          for (int c = 0; c < kAHD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_pv + lane_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32(tmem_pv + lane_addr + c * 32, o);
          }
          tmem_st_wait();
          l *= alpha;
        }
        m_ref = m_tgt;
      }
      SEG_PROF_ADD(4, t)
      // probabilities -> bf16 operand tile (row r, 16-byte chunk c16 stored at c16 ^ (r & 7) inside its 64-column atom)
      const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m_ref, -m_ref);
      uint64_t l2[2] = {0ull, 0ull};  // four running sums as two packed pairs
      // The special-function unit delivers one exp2 per 8 cycles and warp, the bound of this stage; kAEmu of every four pairs
      // take the polynomial route over the otherwise idle FMA pipe instead.
      bf16x8 pk[kAK / 8];  // the row of P as packed bf16
      auto exp_row = [&](auto dg) {
        constexpr bool kDiag = decltype(dg)::value;
#pragma unroll
        for (int c16 = 0; c16 < kAK / 8; ++c16) {
          float pr[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c16 * 8 + 2 * i;
            const uint64_t x2 = fma2(pack2(v[col], v[col + 1]), scale2, neg_m2);
            float p0, p1;
            if (i >= 4 - kAEmu) {
              ex2_poly2(x2, p0, p1);
            } else {
              float x0, x1;
              unpack2(x2, x0, x1);
              p0 = ex2_approx(x0);
              p1 = ex2_approx(x1);
            }
            if (kDiag) {
              if (col > r) p0 = 0.f;
              if (col + 1 > r) p1 = 0.f;
            }
            pr[2 * i] = p0;
            pr[2 * i + 1] = p1;
            l2[i & 1] = add2(l2[i & 1], pack2(p0, p1));
          }
          pk[c16] = pack8(pr);
        }
      };
      if (diag)
        exp_row(std::true_type{});
      else
        exp_row(std::false_type{});
      {
        float a0, a1, a2, a3;
        unpack2(l2[0], a0, a1);
        unpack2(l2[1], a2, a3);
        l += (a0 + a1) + (a2 + a3);
      }
      SEG_PROF_ADD(5, t)
      if (!pv_waited) {
        if (!mbar_wait(b_pv_full, (j - 1) & 1, ab, 18)) { ok = false; break; }
        tc_fence_after();
      }
      // bf16 operand tile: row r, 16-byte chunk c16 stored at c16 ^ (r & 7) inside its 64-column atom
#pragma unroll
      for (int c16 = 0; c16 < kAK / 8; ++c16) {
        uint8_t* atom = sPx + (c16 >> 3) * (kAQ * 128) + r * 128;
        *reinterpret_cast<bf16x8*>(atom + (((c16 & 7) ^ (r & 7)) << 4)) = pk[c16];
      }
      tc_fence_before();
      fence_proxy_async();  // make the P tile visible to the tensor core's shared-memory reads
      __syncwarp();
      if (lane == 0) mbar_arrive(b_p_full);
      SEG_PROF_ADD(6, t)
    }
    if (ok && n_tiles > 0 && mbar_wait(b_pv_full, (n_tiles - 1) & 1, ab, 19)) {
      tc_fence_after();
      const float inv = 1.f / l;
      const int row = qt * kAQ + r;
      const bool in_range = row < p.S;  // TMEM loads are warp-collective: every lane loads, only rows of the sequence store
      __nv_bfloat16* orow = p.o + (((size_t)b * p.S + (in_range ? row : 0)) * p.H + h) * kAHD;
#pragma unroll
      for (int c = 0; c < kAHD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_pv + lane_addr + c * 32, o);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(o[e]) * inv;
        if (in_range && SEG_IN_BOUNDS(p.status, 31, (orow - p.o) + c * 32, 32, (size_t)p.B * p.S * p.H * kAHD)) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) reinterpret_cast<bf16x8*>(orow + c * 32)[q4] = pack8(f + q4 * 8);
        }
      }
      if (in_range && SEG_IN_BOUNDS(p.status, 32, ((size_t)b * p.H + h) * p.S + row, 1, (size_t)p.B * p.H * p.S))
        p.lse[((size_t)b * p.H + h) * p.S + row] = (m_ref + log2f(l)) * 0.6931471805599453f;
      SEG_PROF_ADD(7, t)
    }
  }

  if (*cta_abort != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
  if (prof_cta && threadIdx.x == 0) {
    for (int i = 0; i < 15; ++i) p.prof[i] = prof_s[i];
    p.prof[15] = n_a;
  }
}

// 4-D bf16 tensor map over [B, S, heads, hd] with a {64, 1, 128, 1} box and 128-byte swizzle.
typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_map_bshd(CUtensorMap* map, const void* base, int B, int S, int heads, int hd) {
  static EncodeTiledFn4 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFn4>(ptr);
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

// prof (optional, 16 int64): cycles that one softmax thread (first query tile) and the control thread of the CTA with the
// longest walk spent per stage - softmax: 0 wait S, 1 S -> registers, 2 row max, 3 wait previous P V, 4 rescale O, 5 exp + store P, 6 fence + signal,
// 7 epilogue; control thread: 8 issue K/V loads, 9 nothing ready, 10 issue Q K^T, 12 issue P V; 15 = key tiles walked by the first query tile.
int attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int H, int Hkv, int hd, int* status,
             cudaStream_t st, long long* prof) {
  if (hd != kAHD || S < 1 || H % Hkv != 0) return -10;
  CUtensorMap mq, mk, mv;
  int r = make_map_bshd(&mq, q, B, S, H, hd);
  if (r == 0) r = make_map_bshd(&mk, k, B, S, Hkv, hd);
  if (r == 0) r = make_map_bshd(&mv, v, B, S, Hkv, hd);
  if (r != 0) return 100 + r;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) != cudaSuccess) return -2;
    cudaFuncAttributes fa, fb;
    if (cudaFuncGetAttributes(&fa, attn_fwd_kernel<false>) != cudaSuccess || cudaFuncGetAttributes(&fb, attn_fwd_kernel<true>) != cudaSuccess) return -2;
    const int regs = fa.numRegs < fb.numRegs ? fa.numRegs : fb.numRegs;
    if (kARegsCtl + 2 * kARegsSm > 3 * regs) return -6;  // the register requests would never be granted
    configured = true;
  }
  AttnParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.status = status;
  p.prof = prof;
  dim3 grid((S + 2 * kAQ - 1) / (2 * kAQ), B * H);
  if (prof != nullptr)
    attn_fwd_kernel<true><<<grid, kAttnThreads, kAttnSmem, st>>>(mq, mk, mv, p);
  else
    attn_fwd_kernel<false><<<grid, kAttnThreads, kAttnSmem, st>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace seg
