// bf16 GEMM for sm_100a on CTA pairs: one 256 x 256 output tile per pair of SMs (tcgen05 cta_group::2).
//
//   D[b] = alpha * A[b] * B[b]^T(or B[b]) + beta * C[b]        fp32 accumulation in tensor memory
//
// A cluster of two CTAs (the two SMs of a TPC) owns a tile.  CTA r of the pair holds rows [128 r, 128 r + 128) of the
// tile's A operand and columns [r nt/2, (r+1) nt/2) of its B operand (nt = the tile's width: 256, or the rounded-up
// remainder for the last column tile, whose B halves are loaded in 64-column boxes so that a narrow tile moves fewer
// bytes) in its own shared memory - each CTA loads its own halves with plain, non-multicast
// TMA loads whose completion bytes are counted on the leader's barrier - and one tcgen05.mma.cta_group::2 instruction of
// the leader (M 256, N nt, K 16) reads both halves and accumulates 128 rows into each CTA's tensor memory.  Against one
// CTA per 128-row tile this halves the B bytes a CTA has to stage and read per FLOP, and the ring gets six stages.
//
// Roles (320 threads per CTA): warp 0 TMA producer (both CTAs), warp 1 MMA issuer (leader only), warps 2-9 epilogue
// (both CTAs, each on its own 128 accumulator rows; two accumulators of 256 columns so that a tile's epilogue overlaps
// the next tile's mainloop).  Epilogues:
//   EPI_TMA        : plain outputs.  tcgen05.ld -> registers -> 128-byte-swizzled staging tile -> TMA store, or TMA
//                    reduce-add for fp32 outputs that accumulate into themselves (weight gradients).
//   EPI_TMA_C      : bf16 outputs with an addend: boxes of C are fetched by TMA into the warp's staging tiles ahead of
//                    the accumulator, the result overwrites them in place and is stored by TMA.
//                    Both TMA epilogues store every staging tile once more per further destination (tensor maps of
//                    the peers' copies of D: the all-gather of a result that is sharded over ranks).
//   EPI_SWIGLU     : up projection of a SwiGLU feed-forward: gate and up columns of the same hidden units sit 128
//                    accumulator columns apart; u = (gate | up) and f = silu(gate) * up leave from the same tile.
//   EPI_SWIGLU_BWD : data gradient of the down projection: the accumulator is df, gate and up arrive by TMA, their
//                    gradients replace them in the staging tiles and leave by TMA; df is never stored.
//   EPI_GENERIC    : symmetric (mirrored) outputs, routed outputs, fp32 addends, destinations that are not 16-byte aligned.
// Schedule (gemm_pair_sched.h): whole tiles dealt round-robin to the pairs; the tiles of the last, partly filled wave (or
// all of them when there are fewer tiles than pairs) are cut into ranges of the contraction whose raw accumulators meet
// in a workspace and are summed in a fixed order by the item of the last range, which also runs the epilogue.
// Every wait on an mbarrier or a flag is bounded (sm100.cuh); the two cluster barriers are reached by every thread after
// a bounded time.
//
// The reference runs these products through cuBLAS (transformer/core.py:9-29 nn.Linear, torch.addmm) and Triton
// (training/optimizers/muon_triton.py:58-252).
#include <cuda.h>

#include <cstdlib>

#include "bounds.cuh"
#include "common.cuh"
#include "gemm_pair_sched.h"
#include "gemm_params.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace seg {

using namespace sm100;

constexpr int kPairThreads = 320;
constexpr int kEpiGeneric = 0, kEpiTma = 1, kEpiTmaC = 2, kEpiSwiglu = 3, kEpiSwigluBwd = 4;
// The addend variant keeps two 4 KB tiles per epilogue warp (each receives a box of C, is overwritten with the result and
// stored), paid for with one stage of the ring; so do the SwiGLU variants (gate and up columns travel side by side).
__host__ __device__ constexpr int pair_stages(int epi) { return epi >= kEpiTmaC ? 5 : 6; }
__host__ __device__ constexpr int pair_staging_bytes(int epi) { return epi >= kEpiTmaC ? 8 * 8192 : 8 * 4096; }
constexpr int kPairABytes = 128 * kPairK * 2;
constexpr int kPairBBytes = 128 * kPairK * 2;
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairBarrierBytes = 512;
__host__ __device__ constexpr int pair_smem_total(int epi) {
  return pair_stages(epi) * kPairStageBytes + pair_staging_bytes(epi) + kPairBarrierBytes + 1024;  // + alignment slack
}

// A contributor's raw accumulator chunk goes to its slot; consecutive lanes write consecutive 16-byte pieces.
__device__ __forceinline__ void slot_store(uint4* slot_chunk, int lane, const uint32_t* v) {
#pragma unroll
  for (int j = 0; j < 8; ++j) __stcg(slot_chunk + j * 32 + lane, make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
}
__device__ __forceinline__ void slot_add(const uint4* slot_chunk, int lane, uint32_t* v) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 u = __ldcg(slot_chunk + j * 32 + lane);
    v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + __uint_as_float(u.x));
    v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + __uint_as_float(u.y));
    v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + __uint_as_float(u.z));
    v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + __uint_as_float(u.w));
  }
}
__device__ __forceinline__ bool wait_slot_flag(uint32_t* flag, const AbortState& ab) {
  uint32_t v;
  const long long t0 = clock64();
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v != 0) return true;
    if (*ab.cta_abort != 0) return false;
    if (clock64() - t0 > ab.limit) {
      *ab.cta_abort = 1;
      atomicCAS(ab.global_status, 0, 7);
      return false;
    }
    __nanosleep(40);
  }
}

// Tensor maps of the further destinations of the TMA-store epilogues (peer-mapped copies of D on other ranks): every output
// tile leaves once per destination from the same staging tile, which makes the epilogue the all-gather of the result.
struct PairExtraMaps {
  CUtensorMap m[7];
};

template <bool A_MN, bool B_MN, typename OutT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_c,
                 const __grid_constant__ PairExtraMaps extra, GemmParams p) {
  constexpr int kStages = pair_stages(EPI);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_area = smem + kStages * kPairStageBytes;
  uint8_t* bar_area = stage_area + pair_staging_bytes(EPI);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);  // leader's: bytes of both CTAs' loads
  uint64_t* empty_bar = full_bar + kStages;                     // each CTA's: its stage has been read by the MMAs
  uint64_t* acc_full = empty_bar + kStages;                     // each CTA's: the accumulator is complete
  uint64_t* acc_empty = acc_full + 2;                           // leader's: 16 epilogue warps have drained it
  uint64_t* c_bar = acc_empty + 2;                              // EPI_TMA_C: per epilogue warp and staging tile, the box of C has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(c_bar + 16);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader
  const int n_pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const PairSched sch = make_pair_sched(p.M, p.N, p.K, p.batch, p.symmetric, p.n_static, p.splits);
  const AbortState ab{cta_abort, p.status, p.wait_limit > 0 ? p.wait_limit : (p.wait_flags != nullptr ? kPeerWaitCycles : kWaitCycles)};

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 16);  // one arrival per epilogue warp of either CTA
    }
    for (int a = 0; a < 16; ++a) mbar_init(smem_u32(&c_bar[a]), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (EPI != kEpiGeneric) prefetch_tensormap(&map_d);
    if (EPI >= kEpiTmaC) prefetch_tensormap(&map_c);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc_pair(smem_u32(tmem_slot), 2 * kPairN);
    tmem_relinquish_pair();
  }
  // barrier initialisation and the allocation of both CTAs become visible to the whole pair
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[0]), 0);
      int it = 0;
      bool ok = true;
      uint32_t regions_ready = 0;
      for (int item = pair; item < sch.n_items && ok; item += n_pairs) {
        const PairItem tl = pair_item(sch, item);
        const int a_row0 = tl.m * kPairM + (int)rank * 128;
        // SwiGLU variant: tile n covers hidden units [128 n, 128 n + 128); the leader's half of B holds their gate rows,
        // the peer's half their up rows (F rows further down), so accumulator column c + 128 is the partner of column c
        const int b_row0 = EPI == kEpiSwiglu ? (int)rank * p.swiglu_f + tl.n * 128 : tl.n * kPairN + (int)rank * (tl.nt >> 1);
        const int b_boxes = p.b_box_rows == 64 ? ((tl.nt >> 1) + 63) >> 6 : 128 / p.b_box_rows;  // boxes of this CTA's B half
        if (!A_MN && p.wait_flags != nullptr && a_row0 < p.M) {
          const int r0 = a_row0 / p.region_rows;
          const int last_row = min(a_row0 + 128, p.M) - 1;
          for (int r = r0; r <= last_row / p.region_rows && ok; ++r) {
            if (r < 32 && ((regions_ready >> r) & 1u)) continue;
            ok = wait_region_flag(p.wait_flags + r, p.wait_seq, ab, 4);
            if (r < 32) regions_ready |= 1u << r;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");  // rows written through the generic proxy, read by TMA
        }
        for (int kb = tl.kb0; kb < tl.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, ab, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * (kPairABytes + b_boxes * (B_MN ? 64 : p.b_box_rows) * kPairK * 2));
          const uint32_t fb = full_leader + s * 8;
          const uint32_t sa = smem_u32(smem + s * kPairStageBytes);
          const uint32_t sb = sa + kPairABytes;
          if (A_MN) {
            tma_load_3d_pair(sa, &map_a, fb, a_row0, kb * kPairK, tl.b);
            tma_load_3d_pair(sa + 64 * kPairK * 2, &map_a, fb, a_row0 + 64, kb * kPairK, tl.b);
          } else {
            tma_load_3d_pair(sa, &map_a, fb, kb * kPairK, a_row0, tl.b);
          }
          for (int j = 0; j < b_boxes; ++j) {
            if (B_MN)
              tma_load_3d_pair(sb + j * (64 * kPairK * 2), &map_b, fb, b_row0 + j * 64, kb * kPairK, tl.b);
            else
              tma_load_3d_pair(sb + j * (p.b_box_rows * kPairK * 2), &map_b, fb, kb * kPairK, b_row0 + j * p.b_box_rows, tl.b);
          }
        }
      }
      // Drain: every stage this CTA filled has been read (the commits of the leader have arrived here), so neither CTA
      // leaves while the other can still signal into its shared memory.
      for (int i = 0; i < kStages && ok; ++i, ++it) ok = mbar_wait(smem_u32(&empty_bar[it % kStages]), ((it / kStages) & 1) ^ 1, ab, 5);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t empty_peer = mapa_shared(smem_u32(&empty_bar[0]), 1);
      const uint32_t accfull_peer = mapa_shared(smem_u32(&acc_full[0]), 1);
      int it = 0, local_tile = 0;
      bool ok = true;
      for (int item = pair; item < sch.n_items && ok; item += n_pairs) {
        const PairItem tl = pair_item(sch, item);
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_ph ^ 1, ab, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairN;
        const uint32_t idesc = make_idesc_bf16(kPairM, tl.nt, A_MN, B_MN);
        for (int kb = tl.kb0; kb < tl.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, ab, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kPairStageBytes);
          const uint32_t sb = sa + kPairABytes;
#pragma unroll
          for (int k = 0; k < kPairK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 64 * kPairK * 2, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 64 * kPairK * 2, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb > tl.kb0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&empty_bar[s]));
          umma_commit_pair(empty_peer + s * 8);
        }
        if (ok) {
          umma_commit_pair(smem_u32(&acc_full[acc]));
          umma_commit_pair(accfull_peer + acc * 8);
        }
        ++local_tile;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps per CTA)
    // warp % 4 selects the TMEM sub-partition (32 lanes = 32 rows of this CTA's 128); warps 2-5 take columns [0, 128) of the
    // tile, warps 6-9 columns [128, 256), 32 at a time.  tcgen05.ld hands every lane one row of a chunk.
    const int sub = warp & 3;
    const int ep = warp - 2;
    const int half = ep >> 2;
    const uint32_t accempty_leader = mapa_shared(smem_u32(&acc_empty[0]), 0);
    uint8_t* stage_raw = stage_area + ep * (pair_staging_bytes(EPI) / 8);
    int local_tile = 0;
    bool ok = true;
    uint32_t c_phase = 0;  // EPI_TMA_C: phase bits of this warp's two addend barriers
    // EPI_TMA: one 4 KB staging tile per warp in the 128-byte-swizzle layout of the output's tensor map: 32 rows x 128
    // bytes (64 bf16 = two chunks, or 32 fp32 = one chunk); the 16-byte piece j of row r sits at slot j ^ (r & 7).
    constexpr bool kBf16 = sizeof(OutT) == 2;
    const uint32_t stage_u32 = smem_u32(stage_raw);
    uint4* row_slots = reinterpret_cast<uint4*>(stage_raw + lane * 128);
    // EPI_GENERIC: the chunk is transposed through the XOR-swizzled staging tile so that global accesses are coalesced
    // (8 consecutive lanes cover one row, 4 values each); the addend C is read in that layout one chunk ahead.
    float* stage = reinterpret_cast<float*>(stage_raw);
    const int q = lane & 7, rsub = lane >> 3;
    OutT* D = reinterpret_cast<OutT*>(p.D);
    const OutT* C = reinterpret_cast<const OutT*>(p.C);
    bool vec_ok = (p.ldd % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                  (p.C == nullptr || (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.batch_stride_d % 8 == 0);
    if (EPI == kEpiGeneric) {
      for (int d = 0; d < p.n_extra; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.D_extra[d]) & 15) == 0);
      if (p.route_rows > 0) {
        vec_ok = (p.ldd % 8 == 0) && ((p.route_base * sizeof(OutT)) % 16 == 0) && ((p.route_batch_stride * sizeof(OutT)) % 16 == 0);
        for (int d = 0; d < 8; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.D_route[d]) & 15) == 0);
      }
    }
    for (int item = pair; item < sch.n_items && ok; item += n_pairs) {
      const PairItem tl = pair_item(sch, item);
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      const bool owner = pair_item_owns(sch, tl);
      // the sum of the ranges before this one sits in the slot of range ks - 1: every item adds it to its own accumulator,
      // so the parts are summed in range order and nobody reads more than one
      const int prev_slot = tl.ks > 0 ? pair_slot(sch, tl.ks - 1, tl.t) : -1;
      const uint4* const prev = prev_slot >= 0 ? p.ws + ((size_t)(prev_slot * 2 + (int)rank) * 8 + ep) * (4 * 8 * 32) : nullptr;
      const int row0 = tl.m * kPairM + (int)rank * 128 + sub * 32;  // first row of this warp's 32-row band
      if (EPI == kEpiTmaC && owner && row0 < p.M) {
        // the two boxes of C that this warp needs (64 columns each) are on their way before the accumulator is complete
        if (lane == 0) {
          bulk_wait_group_read0();  // the previous item's stores have left the staging tiles
          for (int k = 0; k < 2; ++k) {
            const int c0 = half * 128 + k * 64;
            if (c0 < tl.nt && tl.n * kPairN + c0 < p.N) {
              const uint32_t cb = smem_u32(&c_bar[ep * 2 + k]);
              mbar_expect_tx(cb, 4096);
              tma_load_3d(stage_u32 + k * 4096, &map_c, cb, tl.n * kPairN + c0, row0, tl.b);
            }
          }
        }
        __syncwarp();
      }
      if (EPI == kEpiSwigluBwd && row0 < p.M) {
        // gate and up values of this warp's first 64 columns are on their way before the accumulator is complete
        if (lane == 0) {
          bulk_wait_group_read0();  // the previous item's stores have left the staging tiles
          const int col = tl.n * kPairN + half * 128;
          mbar_expect_tx(smem_u32(&c_bar[ep * 2]), 4096);
          tma_load_3d(stage_u32, &map_c, smem_u32(&c_bar[ep * 2]), col, row0, tl.b);
          mbar_expect_tx(smem_u32(&c_bar[ep * 2 + 1]), 4096);
          tma_load_3d(stage_u32 + 4096, &map_c, smem_u32(&c_bar[ep * 2 + 1]), p.swiglu_f + col, row0, tl.b);
        }
        __syncwarp();
      }
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_ph, ab, 6, p.epi_backoff_ns)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + ((uint32_t)(sub * 32) << 16) + acc * kPairN;
      if (prev != nullptr) {
        if (lane == 0) ok = wait_slot_flag(p.ws_flags + (prev_slot * 2 + (int)rank) * 8 + ep, ab);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
      }
      if (!owner) {
        // -------- part of a tile: the raw accumulator goes to the item's slot, then the flag of this warp is raised
        const int slot = pair_slot(sch, tl.ks, tl.t);
        if (!SEG_IN_BOUNDS(p.status, 5, slot, 1, kPairMaxSlots)) { ok = false; break; }
        uint4* const my_slot = p.ws + ((size_t)(slot * 2 + (int)rank) * 8 + ep) * (4 * 8 * 32);
#pragma unroll 1
        for (int ci = 0; ci < 4; ++ci) {
          const int c0 = half * 128 + ci * 32;
          if (c0 >= tl.nt) break;
          uint32_t v[32];
          tmem_ld_32x32(tmem_acc + c0, v);
          tmem_ld_wait_regs(v);
          if (prev != nullptr) slot_add(prev + ci * (8 * 32), lane, v);
          slot_store(my_slot + ci * (8 * 32), lane, v);
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ws_flags + (slot * 2 + (int)rank) * 8 + ep), "r"(1u) : "memory");
        }
      } else {
        if (EPI == kEpiTmaC) {
          if (row0 < p.M) {
#pragma unroll 1
            for (int ci = 0; ci < 4; ++ci) {
              const int c0 = half * 128 + ci * 32;
              const int col = tl.n * kPairN + c0;
              if (c0 >= tl.nt || col >= p.N) break;  // warp-uniform
              const int k = ci >> 1;
              uint32_t v[32];
              tmem_ld_32x32(tmem_acc + c0, v);
              if ((ci & 1) == 0) {  // first chunk of a box: its addend has landed
                if (!mbar_wait(smem_u32(&c_bar[ep * 2 + k]), (c_phase >> k) & 1u, ab, 8)) { ok = false; break; }
                c_phase ^= 1u << k;
              }
              tmem_ld_wait_regs(v);
              if (prev != nullptr) slot_add(prev + ci * (8 * 32), lane, v);
              uint4* slots = reinterpret_cast<uint4*>(stage_raw + k * 4096 + lane * 128);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4& u = slots[((ci & 1) * 4 + j) ^ (lane & 7)];
                const uint4 cin = u;
                const uint32_t cw[4] = {cin.x, cin.y, cin.z, cin.w};
                uint32_t ow[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 cf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cw[e]));
                  const __nv_bfloat162 h = __floats2bfloat162_rn(p.alpha * __uint_as_float(v[8 * j + 2 * e]) + p.beta * cf.x,
                                                                 p.alpha * __uint_as_float(v[8 * j + 2 * e + 1]) + p.beta * cf.y);
                  ow[e] = *reinterpret_cast<const uint32_t*>(&h);
                }
                u = make_uint4(ow[0], ow[1], ow[2], ow[3]);
              }
              const bool last_chunk = (ci == 3) || (c0 + 32 >= tl.nt) || (col + 32 >= p.N);
              if ((ci & 1) == 1 || last_chunk) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  tma_store_3d(&map_d, stage_u32 + k * 4096, tl.n * kPairN + half * 128 + k * 64, row0, tl.b);
                  for (int d = 0; d < p.n_extra; ++d) tma_store_3d(&extra.m[d], stage_u32 + k * 4096, tl.n * kPairN + half * 128 + k * 64, row0, tl.b);
                  bulk_commit_group();
                }
              }
            }
            if (!ok) break;
          }
        } else if (EPI == kEpiSwiglu) {
          if (row0 < p.M) {
            // This warp: gate columns [64 half, 64 half + 64) of the tile and their up partners 128 columns further.  Both
            // leave as bf16 (tile 0 -> gate block of D, tile 1 -> up block of D); f = silu(gate) * up is formed from the
            // rounded values, exactly what a separate pass over D would compute, and follows through tile 0.
            const int hcol = tl.n * 128 + half * 64;
            uint32_t fpk[32];
            if (lane == 0) bulk_wait_group_read0();  // the previous item's stores have left both tiles
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t g[32], u[32];
              tmem_ld_32x32(tmem_acc + half * 64 + c * 32, g);
              tmem_ld_32x32(tmem_acc + 128 + half * 64 + c * 32, u);
              tmem_ld_wait_regs(g);
              tmem_ld_wait_regs(u);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t gw[4], uw[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const __nv_bfloat162 gh = __floats2bfloat162_rn(__uint_as_float(g[8 * j + 2 * e]), __uint_as_float(g[8 * j + 2 * e + 1]));
                  const __nv_bfloat162 uh = __floats2bfloat162_rn(__uint_as_float(u[8 * j + 2 * e]), __uint_as_float(u[8 * j + 2 * e + 1]));
                  gw[e] = *reinterpret_cast<const uint32_t*>(&gh);
                  uw[e] = *reinterpret_cast<const uint32_t*>(&uh);
                  const float2 a = __bfloat1622float2(gh), b = __bfloat1622float2(uh);
                  const __nv_bfloat162 fh = __floats2bfloat162_rn(a.x * sigmoidf_(a.x) * b.x, a.y * sigmoidf_(a.y) * b.y);
                  fpk[c * 16 + j * 4 + e] = *reinterpret_cast<const uint32_t*>(&fh);
                }
                row_slots[(c * 4 + j) ^ (lane & 7)] = make_uint4(gw[0], gw[1], gw[2], gw[3]);
                reinterpret_cast<uint4*>(stage_raw + 4096 + lane * 128)[(c * 4 + j) ^ (lane & 7)] = make_uint4(uw[0], uw[1], uw[2], uw[3]);
              }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&map_d, stage_u32, hcol, row0, tl.b);
              tma_store_3d(&map_d, stage_u32 + 4096, p.swiglu_f + hcol, row0, tl.b);
              bulk_commit_group();
              bulk_wait_group_read0();
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) row_slots[j ^ (lane & 7)] = make_uint4(fpk[4 * j], fpk[4 * j + 1], fpk[4 * j + 2], fpk[4 * j + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&map_c, stage_u32, hcol, row0, tl.b);
              bulk_commit_group();
            }
          }
        } else if (EPI == kEpiSwigluBwd) {
          if (row0 < p.M) {
            // The accumulator is df = dy W (gradient of f = silu(gate) * up), rounded to bf16 as a stored df would be.  Per
            // 64 columns: gate and up arrive in tiles 0 and 1, are replaced by their gradients and leave for the gate and up
            // blocks of the output; the second 64 columns reuse the tiles once the first stores have read them.
#pragma unroll 1
            for (int k = 0; k < 2; ++k) {
              const int c0g = half * 128 + k * 64;
              const int col = tl.n * kPairN + c0g;
              if (k == 1) {
                if (lane == 0) {
                  bulk_wait_group_read0();
                  mbar_expect_tx(smem_u32(&c_bar[ep * 2]), 4096);
                  tma_load_3d(stage_u32, &map_c, smem_u32(&c_bar[ep * 2]), col, row0, tl.b);
                  mbar_expect_tx(smem_u32(&c_bar[ep * 2 + 1]), 4096);
                  tma_load_3d(stage_u32 + 4096, &map_c, smem_u32(&c_bar[ep * 2 + 1]), p.swiglu_f + col, row0, tl.b);
                }
                __syncwarp();
              }
              if (!mbar_wait(smem_u32(&c_bar[ep * 2]), c_phase & 1u, ab, 8) || !mbar_wait(smem_u32(&c_bar[ep * 2 + 1]), (c_phase >> 1) & 1u, ab, 8)) {
                ok = false;
                break;
              }
              c_phase ^= 3u;
              uint4* ga = reinterpret_cast<uint4*>(stage_raw + lane * 128);
              uint4* ua = reinterpret_cast<uint4*>(stage_raw + 4096 + lane * 128);
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_acc + c0g + c * 32, v);
                tmem_ld_wait_regs(v);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int slot = (c * 4 + j) ^ (lane & 7);
                  const uint4 gq = ga[slot], uq = ua[slot];
                  const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w}, uw[4] = {uq.x, uq.y, uq.z, uq.w};
                  uint32_t aw[4], bw[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 d = __bfloat1622float2(__floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1])));
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[e]));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[e]));
                    float da0, db0, da1, db1;
                    swiglu_grad(a.x, b.x, d.x, da0, db0);
                    swiglu_grad(a.y, b.y, d.y, da1, db1);
                    const __nv_bfloat162 ah = __floats2bfloat162_rn(da0, da1), bh = __floats2bfloat162_rn(db0, db1);
                    aw[e] = *reinterpret_cast<const uint32_t*>(&ah);
                    bw[e] = *reinterpret_cast<const uint32_t*>(&bh);
                  }
                  ga[slot] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
                  ua[slot] = make_uint4(bw[0], bw[1], bw[2], bw[3]);
                }
              }
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&map_d, stage_u32, col, row0, tl.b);
                tma_store_3d(&map_d, stage_u32 + 4096, p.swiglu_f + col, row0, tl.b);
                bulk_commit_group();
              }
            }
            if (!ok) break;
          }
        } else if (EPI == kEpiTma) {
          if (row0 < p.M) {
#pragma unroll 1
            for (int ci = 0; ci < 4; ++ci) {
              const int c0 = half * 128 + ci * 32;
              const int col = tl.n * kPairN + c0;
              if (c0 >= tl.nt || col >= p.N) break;  // warp-uniform
              uint32_t v[32];
              tmem_ld_32x32(tmem_acc + c0, v);
              if (!kBf16 || (ci & 1) == 0) {  // a new staging tile: the previous store has finished reading it
                if (lane == 0) bulk_wait_group_read0();
                __syncwarp();
              }
              tmem_ld_wait_regs(v);
              if (prev != nullptr) slot_add(prev + ci * (8 * 32), lane, v);
              if (kBf16) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 u;
                  __nv_bfloat162 h;
                  h = __floats2bfloat162_rn(p.alpha * __uint_as_float(v[8 * j]), p.alpha * __uint_as_float(v[8 * j + 1]));
                  u.x = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2bfloat162_rn(p.alpha * __uint_as_float(v[8 * j + 2]), p.alpha * __uint_as_float(v[8 * j + 3]));
                  u.y = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2bfloat162_rn(p.alpha * __uint_as_float(v[8 * j + 4]), p.alpha * __uint_as_float(v[8 * j + 5]));
                  u.z = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2bfloat162_rn(p.alpha * __uint_as_float(v[8 * j + 6]), p.alpha * __uint_as_float(v[8 * j + 7]));
                  u.w = *reinterpret_cast<uint32_t*>(&h);
                  row_slots[((ci & 1) * 4 + j) ^ (lane & 7)] = u;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  uint4 u;
                  u.x = __float_as_uint(p.alpha * __uint_as_float(v[4 * j]));
                  u.y = __float_as_uint(p.alpha * __uint_as_float(v[4 * j + 1]));
                  u.z = __float_as_uint(p.alpha * __uint_as_float(v[4 * j + 2]));
                  u.w = __float_as_uint(p.alpha * __uint_as_float(v[4 * j + 3]));
                  row_slots[j ^ (lane & 7)] = u;
                }
              }
              const bool last_chunk = (ci == 3) || (c0 + 32 >= tl.nt) || (col + 32 >= p.N);
              if (!kBf16 || (ci & 1) == 1 || last_chunk) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  const int col_store = kBf16 ? tl.n * kPairN + half * 128 + (ci & ~1) * 32 : col;
                  if (p.reduce)
                    tma_reduce_add_3d(&map_d, stage_u32, col_store, row0, tl.b);
                  else
                    tma_store_3d(&map_d, stage_u32, col_store, row0, tl.b);
                  for (int d = 0; d < p.n_extra; ++d) tma_store_3d(&extra.m[d], stage_u32, col_store, row0, tl.b);
                  bulk_commit_group();
                }
              }
            }
          }
        } else if (row0 < p.M) {
          const int64_t boff = (int64_t)tl.b * p.batch_stride_d;
          OutT* rbase[8];
          if (p.route_rows > 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = row0 + rsub + 4 * i;
              const int reg = r / p.route_rows;
              rbase[i] = reinterpret_cast<OutT*>(p.D_route[reg < 8 ? reg : 7]) + p.route_base + (int64_t)tl.b * p.route_batch_stride +
                         (int64_t)(r - reg * p.route_rows) * p.ldd;
            }
          }
          float4 cnext[8];
          bool have_next = false;
          auto fetch_c = [&](int col, float4* dst) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = row0 + rsub + 4 * i;
              dst[i] = (r < p.M) ? load4<OutT>(C + boff + (int64_t)r * p.ldd + col + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          };
          {
            const int col = tl.n * kPairN + half * 128;
            if (C != nullptr && vec_ok && half * 128 < tl.nt && col + 32 <= p.N) {
              fetch_c(col, cnext);
              have_next = true;
            }
          }
#pragma unroll 1
          for (int ci = 0; ci < 4; ++ci) {
            const int c0 = half * 128 + ci * 32;
            const int col = tl.n * kPairN + c0;
            if (c0 >= tl.nt || col >= p.N) break;  // warp-uniform
            uint32_t v[32];
            tmem_ld_32x32(tmem_acc + c0, v);
            float4 ccur[8];
            const bool have_cur = have_next;
            if (have_cur) {
#pragma unroll
              for (int i = 0; i < 8; ++i) ccur[i] = cnext[i];
            }
            have_next = false;
            if (ci + 1 < 4 && c0 + 32 < tl.nt && C != nullptr && vec_ok && col + 64 <= p.N) {
              fetch_c(col + 32, cnext);
              have_next = true;
            }
            tmem_ld_wait_regs(v);
            if (prev != nullptr) slot_add(prev + ci * (8 * 32), lane, v);
            const int ncols = (p.N - col) < 32 ? (p.N - col) : 32;
            const bool fast = vec_ok && ncols == 32 && (C == nullptr || have_cur);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4*>(stage + lane * 32)[j ^ (lane & 7)] =
                  make_float4(p.alpha * __uint_as_float(v[4 * j]), p.alpha * __uint_as_float(v[4 * j + 1]),
                              p.alpha * __uint_as_float(v[4 * j + 2]), p.alpha * __uint_as_float(v[4 * j + 3]));
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = rsub + 4 * i, r = row0 + rl;
              float4 f = reinterpret_cast<const float4*>(stage + rl * 32)[q ^ (rl & 7)];
              if (r < p.M) {
                const int64_t off = boff + (int64_t)r * p.ldd + col + 4 * q;
                if (fast) {
                  if (C != nullptr) {
                    f.x += p.beta * ccur[i].x; f.y += p.beta * ccur[i].y; f.z += p.beta * ccur[i].z; f.w += p.beta * ccur[i].w;
                  }
                  if (p.route_rows > 0) {
                    const int reg = r / p.route_rows;
                    const int64_t roff = p.route_base + (int64_t)tl.b * p.route_batch_stride + (int64_t)(r - reg * p.route_rows) * p.ldd + col + 4 * q;
                    if (SEG_IN_BOUNDS(p.status, 3, reg < 8 ? roff : -1, 4, p.route_extent)) store4<OutT>(rbase[i] + col + 4 * q, f);
                  } else if (SEG_IN_BOUNDS(p.status, 1, off, 4, p.d_extent)) {
                    store4<OutT>(D + off, f);
                    for (int d = 0; d < p.n_extra; ++d) store4<OutT>(reinterpret_cast<OutT*>(p.D_extra[d]) + off, f);
                  }
                } else {
                  const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (4 * q + e < ncols) {
                      float val = fv[e];
                      if (C != nullptr) val += p.beta * to_f<OutT>(C[off + e]);
                      if (p.route_rows > 0) {
                        const int reg = r / p.route_rows;
                        const int64_t roff = p.route_base + (int64_t)tl.b * p.route_batch_stride + (int64_t)(r - reg * p.route_rows) * p.ldd + col + 4 * q + e;
                        if (SEG_IN_BOUNDS(p.status, 3, reg < 8 ? roff : -1, 1, p.route_extent)) rbase[i][col + 4 * q + e] = from_f<OutT>(val);
                      } else if (SEG_IN_BOUNDS(p.status, 1, off + e, 1, p.d_extent)) {
                        D[off + e] = from_f<OutT>(val);
                        for (int d = 0; d < p.n_extra; ++d) reinterpret_cast<OutT*>(p.D_extra[d])[off + e] = from_f<OutT>(val);
                      }
                      if (e == 0) f.x = val; else if (e == 1) f.y = val; else if (e == 2) f.z = val; else f.w = val;
                    }
                  }
                }
              }
              if (p.symmetric) reinterpret_cast<float4*>(stage + rl * 32)[q ^ (rl & 7)] = f;  // final values for the mirror pass
            }
            // symmetric outputs: the twin tile (this chunk's columns as rows) is not in the schedule when it lies wholly
            // below the diagonal, so its elements are written from here, consecutive lanes on consecutive addresses
            const int row = row0 + lane;
            const bool mirror = p.symmetric && (row0 / kPairN) < (col / kPairM);
            if (mirror) {
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 f = reinterpret_cast<const float4*>(stage + lane * 32)[j ^ (lane & 7)];
                const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int cc = 4 * j + e;
                  if (row < p.M && cc < ncols) {
                    const OutT val = from_f<OutT>(fv[e]);
                    const int64_t moff = boff + (int64_t)(col + cc) * p.ldd + row;
                    if (SEG_IN_BOUNDS(p.status, 4, moff, 1, p.d_extent)) {
                      D[moff] = val;
                      for (int d = 0; d < p.n_extra; ++d) reinterpret_cast<OutT*>(p.D_extra[d])[moff] = val;
                    }
                  }
                }
              }
            }
            __syncwarp();  // the staging tile is rewritten by the next chunk
          }
        }
      }
      if (prev != nullptr && lane == 0) p.ws_flags[(prev_slot * 2 + (int)rank) * 8 + ep] = 0;  // free for the next launch
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(accempty_leader + acc * 8);
      ++local_tile;
    }
    if (EPI != kEpiGeneric && lane == 0) bulk_wait_group0();  // this warp's stores have left its staging tile and are complete
  }

  // ------------------------------------------------------------------ teardown (also reached after an abort)
  if (*cta_abort != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);  // loads that may still be in flight land before shared memory is released
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA frees tensor memory or leaves while its peer may still use it
  tc_fence_after();
  if (warp == 0) tmem_dealloc_pair(tmem_base, 2 * kPairN);
}

// ------------------------------------------------------------------------------------------------ host side
size_t gemm_pair_workspace_bytes() { return (size_t)kPairMaxSlots * kPairSlotPieces * sizeof(uint4); }
size_t gemm_pair_flag_words() { return (size_t)kPairMaxSlots * 16; }

template <bool A_MN, bool B_MN, typename OutT, int EPI>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const CUtensorMap& mc, const GemmParams& p, int pairs,
                       cudaStream_t st, const PairExtraMaps* extra = nullptr) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OutT, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_total(EPI)) != cudaSuccess) return -2;
    configured = true;
  }
  PairExtraMaps ex;
  for (int i = 0; i < 7; ++i) ex.m[i] = (extra != nullptr) ? extra->m[i] : md;  // unused slots hold a valid map
  kern<<<2 * pairs, kPairThreads, pair_smem_total(EPI), st>>>(ma, mb, md, mc, ex, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int gemm_bf16_pair(const void* A, const void* B, const void* C, void* D, int M, int N, int K, int batch, int64_t lda, int64_t ldb,
                   int64_t ldd, int64_t bsa, int64_t bsb, int64_t bsd, bool a_mn_major, bool b_mn_major, bool out_f32, float alpha,
                   float beta, bool symmetric, void* const* d_extra, int n_extra, int* status, int sm_count, cudaStream_t st,
                   const uint32_t* wait_flags, uint32_t wait_seq, int region_rows, void* const* d_route, int n_route,
                   int route_rows, int64_t route_batch_stride, int64_t route_base, long long wait_limit, void* workspace,
                   uint32_t* ws_flags, int split_k) {
  if (n_route > 0 && (C != nullptr || symmetric || n_extra > 0 || route_rows <= 0 || (int64_t)n_route * route_rows < M || n_route > 8))
    return -5;  // routed output excludes the addend, the mirrored output and the extra destinations
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  static const int b_box_env = [] {
    const char* e = std::getenv("SEGPT_GEMM_BBOX");
    return (e != nullptr && std::atoi(e) == 128) ? 128 : 64;
  }();
  CUtensorMap ma, mb, md, mc;
  int r;
  if (a_mn_major)  // memory [K, M]
    r = make_tensor_map_3d(&ma, A, false, (uint64_t)M, (uint64_t)K, (uint64_t)batch, (uint64_t)lda, (uint64_t)bsa, 64, 64);
  else  // memory [M, K]
    r = make_tensor_map_3d(&ma, A, false, (uint64_t)K, (uint64_t)M, (uint64_t)batch, (uint64_t)lda, (uint64_t)bsa, 64, 128);
  if (r != 0) return 100 + r;
  if (b_mn_major)  // memory [K, N]
    r = make_tensor_map_3d(&mb, B, false, (uint64_t)N, (uint64_t)K, (uint64_t)batch, (uint64_t)ldb, (uint64_t)bsb, 64, 64);
  else  // memory [N, K]
    r = make_tensor_map_3d(&mb, B, false, (uint64_t)K, (uint64_t)N, (uint64_t)batch, (uint64_t)ldb, (uint64_t)bsb, 64, (uint32_t)b_box_env);
  if (r != 0) return 200 + r;

  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.alpha = alpha; p.beta = beta;
  p.C = C; p.D = D; p.ldd = ldd; p.batch_stride_d = bsd;
  p.status = status;
  p.symmetric = symmetric ? 1 : 0;
  p.n_extra = n_extra < 0 ? 0 : (n_extra > 7 ? 7 : n_extra);
  for (int i = 0; i < 7; ++i) p.D_extra[i] = i < p.n_extra ? d_extra[i] : nullptr;
  p.wait_flags = (wait_flags != nullptr && region_rows > 0 && !a_mn_major) ? wait_flags : nullptr;
  p.wait_seq = wait_seq;
  p.region_rows = region_rows > 0 ? region_rows : 1;
  p.route_rows = n_route > 0 ? route_rows : 0;
  p.route_batch_stride = route_batch_stride;
  p.route_base = route_base;
  for (int i = 0; i < 8; ++i) p.D_route[i] = (n_route > 0) ? d_route[i < n_route ? i : n_route - 1] : nullptr;
  p.wait_limit = wait_limit;
  // extents for the debug build's index checks: last element the epilogue may touch, plus one
  p.d_extent = (int64_t)(batch - 1) * bsd + (int64_t)(M - 1) * ldd + N;
  p.route_extent = n_route > 0 ? route_base + (int64_t)(batch - 1) * route_batch_stride + (int64_t)(route_rows - 1) * ldd + N : 0;
  if (gemm_debug_extent_cap_value() > 0 && p.d_extent > gemm_debug_extent_cap_value()) p.d_extent = gemm_debug_extent_cap_value();
  p.reduce = 0;
  p.swiglu_f = 0;
  p.ws = reinterpret_cast<uint4*>(workspace);
  p.ws_flags = ws_flags;
  p.b_box_rows = b_box_env;
  static const int backoff_env = [] {
    const char* e = std::getenv("SEGPT_GEMM_EPI_BACKOFF_NS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  p.epi_backoff_ns = backoff_env;
  pair_choose_split(M, N, K, batch, p.symmetric, sm_count / 2, split_k != 0 && workspace != nullptr && ws_flags != nullptr && p.wait_flags == nullptr,
                    p.n_static, p.splits);
  const PairSched sched = make_pair_sched(M, N, K, batch, p.symmetric, p.n_static, p.splits);
  const int pairs = sched.n_items < sm_count / 2 ? sched.n_items : sm_count / 2;

  // The TMA epilogue serves plain outputs: no routing, mirroring or extra destinations, and either no addend or an fp32
  // output that accumulates into itself (D += alpha * A op(B)), which becomes a TMA reduction.
  const size_t esz = out_f32 ? 4 : 2;
  const bool accumulate = C != nullptr && C == D && beta == 1.0f && out_f32;
  const bool aligned = (reinterpret_cast<uintptr_t>(D) % 16 == 0) && ((ldd * esz) % 16 == 0) && (batch == 1 || (bsd * esz) % 16 == 0);
  bool extra_ok = true;  // further destinations go through the TMA epilogues when they are laid out and aligned like D
  for (int i = 0; i < p.n_extra; ++i) extra_ok = extra_ok && (reinterpret_cast<uintptr_t>(p.D_extra[i]) % 16 == 0);
  const bool plain = n_route == 0 && extra_ok && !(p.n_extra > 0 && accumulate) && !symmetric && aligned && D != nullptr;
  const bool tma_epi = plain && (C == nullptr || accumulate);
  const bool tma_c_epi = plain && !tma_epi && !out_f32 && (reinterpret_cast<uintptr_t>(C) % 16 == 0);
  md = ma;  // placeholders when unused
  mc = ma;
  if (tma_epi || tma_c_epi) {
    r = make_tensor_map_3d(&md, D, out_f32, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldd, (uint64_t)bsd, out_f32 ? 32 : 64, 32);
    if (r != 0) return 300 + r;
    p.reduce = (tma_epi && accumulate) ? 1 : 0;
  }
  if (tma_c_epi) {
    r = make_tensor_map_3d(&mc, C, false, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldd, (uint64_t)bsd, 64, 32);
    if (r != 0) return 400 + r;
  }
  PairExtraMaps extra_maps;
  const bool with_extra = (tma_epi || tma_c_epi) && p.n_extra > 0;
  if (with_extra) {
    for (int i = 0; i < 7; ++i) {
      r = make_tensor_map_3d(&extra_maps.m[i], i < p.n_extra ? p.D_extra[i] : D, out_f32, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldd,
                             (uint64_t)bsd, out_f32 ? 32 : 64, 32);
      if (r != 0) return 500 + r;
    }
  }
  const PairExtraMaps* extra_ptr = with_extra ? &extra_maps : nullptr;
#define SEG_PAIR(AM, BM_)                                                                                             \
  (tma_c_epi ? launch_pair<AM, BM_, __nv_bfloat16, kEpiTmaC>(ma, mb, md, mc, p, pairs, st, extra_ptr)                 \
   : tma_epi ? (out_f32 ? launch_pair<AM, BM_, float, kEpiTma>(ma, mb, md, mc, p, pairs, st, extra_ptr)               \
                        : launch_pair<AM, BM_, __nv_bfloat16, kEpiTma>(ma, mb, md, mc, p, pairs, st, extra_ptr))      \
             : (out_f32 ? launch_pair<AM, BM_, float, kEpiGeneric>(ma, mb, md, mc, p, pairs, st)                      \
                        : launch_pair<AM, BM_, __nv_bfloat16, kEpiGeneric>(ma, mb, md, mc, p, pairs, st)))
  if (!a_mn_major && !b_mn_major) return SEG_PAIR(false, false);
  if (!a_mn_major && b_mn_major) return SEG_PAIR(false, true);
  if (a_mn_major && b_mn_major) return SEG_PAIR(true, true);
  return SEG_PAIR(true, false);
#undef SEG_PAIR
}

// u[:, :F] | u[:, F:] = x W^T (W = [gate rows | up rows], [2F, K]) and f = silu(u[:, :F]) * u[:, F:] in one launch
// (the feed-forward of transformer/core.py:86-89 of the reference up to its down projection).
int gemm_swiglu_pair(const void* X, const void* W, void* U, void* Fout, int M, int F, int K, int64_t ldx, int64_t ldw, int64_t ldu,
                     int64_t ldf, int* status, int sm_count, cudaStream_t st, long long wait_limit) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if (F % 128 != 0 || K % 8 != 0) return -7;
  for (const void* ptr : {X, W, (const void*)U, (const void*)Fout})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return -8;
  if (ldx % 8 != 0 || ldw % 8 != 0 || ldu % 8 != 0 || ldf % 8 != 0) return -8;
  CUtensorMap ma, mb, md, mc;
  int r = make_tensor_map_3d(&ma, X, false, (uint64_t)K, (uint64_t)M, 1, (uint64_t)ldx, (uint64_t)M * ldx, 64, 128);
  if (r != 0) return 100 + r;
  r = make_tensor_map_3d(&mb, W, false, (uint64_t)K, (uint64_t)2 * F, 1, (uint64_t)ldw, (uint64_t)2 * F * ldw, 64, 64);
  if (r != 0) return 200 + r;
  r = make_tensor_map_3d(&md, U, false, (uint64_t)2 * F, (uint64_t)M, 1, (uint64_t)ldu, (uint64_t)M * ldu, 64, 32);
  if (r != 0) return 300 + r;
  r = make_tensor_map_3d(&mc, Fout, false, (uint64_t)F, (uint64_t)M, 1, (uint64_t)ldf, (uint64_t)M * ldf, 64, 32);
  if (r != 0) return 400 + r;
  GemmParams p;
  p.M = M; p.N = 2 * F; p.K = K; p.batch = 1;
  p.alpha = 1.f; p.beta = 0.f;
  p.C = nullptr; p.D = U; p.ldd = ldu; p.batch_stride_d = (int64_t)M * ldu;
  p.status = status;
  p.symmetric = 0;
  p.n_extra = 0;
  for (int i = 0; i < 7; ++i) p.D_extra[i] = nullptr;
  p.wait_flags = nullptr; p.wait_seq = 0; p.region_rows = 1;
  p.route_rows = 0; p.route_batch_stride = 0; p.route_base = 0;
  for (int i = 0; i < 8; ++i) p.D_route[i] = nullptr;
  p.wait_limit = wait_limit;
  p.d_extent = (int64_t)(M - 1) * ldu + 2 * F;
  p.route_extent = 0;
  p.reduce = 0;
  p.ws = nullptr; p.ws_flags = nullptr;
  p.b_box_rows = 64;
  p.epi_backoff_ns = 0;
  p.swiglu_f = F;
  pair_choose_split(M, 2 * F, K, 1, 0, sm_count / 2, false, p.n_static, p.splits);  // whole tiles only
  const PairSched sched = make_pair_sched(M, 2 * F, K, 1, 0, p.n_static, p.splits);
  const int pairs = sched.n_items < sm_count / 2 ? sched.n_items : sm_count / 2;
  return launch_pair<false, false, __nv_bfloat16, kEpiSwiglu>(ma, mb, md, mc, p, pairs, st);
}

// DU [M, 2F] = gradient of (gate | up) for f = silu(gate) * up, given dY [M, K], W [K, F] (df = dY W never reaches memory)
// and U [M, 2F] = (gate | up).
int gemm_swiglu_bwd_pair(const void* dY, const void* W, const void* U, void* DU, int M, int F, int K, int64_t ldy, int64_t ldw,
                         int64_t ldu, int64_t lddu, int* status, int sm_count, cudaStream_t st, long long wait_limit) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if (F % 256 != 0 || K % 8 != 0) return -7;
  for (const void* ptr : {dY, W, U, (const void*)DU})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return -8;
  if (ldy % 8 != 0 || ldw % 8 != 0 || ldu % 8 != 0 || lddu % 8 != 0) return -8;
  CUtensorMap ma, mb, md, mc;
  int r = make_tensor_map_3d(&ma, dY, false, (uint64_t)K, (uint64_t)M, 1, (uint64_t)ldy, (uint64_t)M * ldy, 64, 128);
  if (r != 0) return 100 + r;
  r = make_tensor_map_3d(&mb, W, false, (uint64_t)F, (uint64_t)K, 1, (uint64_t)ldw, (uint64_t)K * ldw, 64, 64);  // memory [K, F]
  if (r != 0) return 200 + r;
  r = make_tensor_map_3d(&md, DU, false, (uint64_t)2 * F, (uint64_t)M, 1, (uint64_t)lddu, (uint64_t)M * lddu, 64, 32);
  if (r != 0) return 300 + r;
  r = make_tensor_map_3d(&mc, U, false, (uint64_t)2 * F, (uint64_t)M, 1, (uint64_t)ldu, (uint64_t)M * ldu, 64, 32);
  if (r != 0) return 400 + r;
  GemmParams p;
  p.M = M; p.N = F; p.K = K; p.batch = 1;
  p.alpha = 1.f; p.beta = 0.f;
  p.C = U; p.D = DU; p.ldd = lddu; p.batch_stride_d = (int64_t)M * lddu;
  p.status = status;
  p.symmetric = 0;
  p.n_extra = 0;
  for (int i = 0; i < 7; ++i) p.D_extra[i] = nullptr;
  p.wait_flags = nullptr; p.wait_seq = 0; p.region_rows = 1;
  p.route_rows = 0; p.route_batch_stride = 0; p.route_base = 0;
  for (int i = 0; i < 8; ++i) p.D_route[i] = nullptr;
  p.wait_limit = wait_limit;
  p.d_extent = (int64_t)(M - 1) * lddu + 2 * F;
  p.route_extent = 0;
  p.reduce = 0;
  p.ws = nullptr; p.ws_flags = nullptr;
  p.b_box_rows = 64;
  p.epi_backoff_ns = 0;
  p.swiglu_f = F;
  pair_choose_split(M, F, K, 1, 0, sm_count / 2, false, p.n_static, p.splits);  // whole tiles only
  const PairSched sched = make_pair_sched(M, F, K, 1, 0, p.n_static, p.splits);
  const int pairs = sched.n_items < sm_count / 2 ? sched.n_items : sm_count / 2;
  return launch_pair<false, true, __nv_bfloat16, kEpiSwigluBwd>(ma, mb, md, mc, p, pairs, st);
}

}  // namespace seg
