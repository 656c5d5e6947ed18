// Persistent, warp-specialised bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[b] = alpha * A[b] * B[b]^T(or B[b]) + beta * C[b]        fp32 accumulation in tensor memory
//
// Operands are described by 3-D TMA tensor maps (inner, outer, batch) built on the host:
//   K-major operand  : memory [rows, K]  (contraction index contiguous)  -> box {64, rows_per_tile}
//   MN-major operand : memory [K, rows]  (row index contiguous)          -> boxes {64, 64}, one per 64 rows
// so that x @ W^T, dy @ W and dy^T @ x all read their inputs in place (no transposes are materialised).
//
// Structure (one CTA per SM, 320 threads):
//   warp 0   : TMA producer.  One elected lane walks the tiles of this CTA and the K blocks of each tile, waits
//              for a free stage (empty barrier) and issues the loads of the A and B tiles for that stage
//              (128-byte swizzle), completing on the stage's full barrier.
//   warp 1   : MMA issuer.  One elected lane waits for a stage, issues BK/16 tcgen05.mma instructions
//              (128 x BN x 16, accumulator in TMEM) and commits them to the stage's empty barrier; after the last
//              K block it commits to the accumulator's full barrier.  Two accumulators (2 x BN columns of TMEM)
//              let the next tile's mainloop overlap this tile's epilogue.
//   warps 2-9: epilogue.  Each warp owns the 32 TMEM lanes of its sub-partition (warp % 4) and one half of the
//              columns, reads the accumulator with tcgen05.ld 32 columns at a time, applies alpha / beta*C (C fetched
//              one chunk ahead) and stores bf16 or fp32 rows - to this GPU and, optionally, to peer GPUs' buffers.
// Every mbarrier wait is bounded (sm100.cuh): on expiry the CTA raises an abort flag, all roles unwind, TMEM is
// freed and a status word reports the failure to the host.
//
// The reference runs these products through cuBLAS (nn.Linear, torch.addmm) and Triton
// (training/optimizers/muon_triton.py:58-252, ns_line_1 / ns_line_2).
#include <cuda.h>

#include "bounds.cuh"
#include "common.cuh"
#include "gemm_params.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace seg {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStagingBytes = 8 * 32 * 32 * 4;  // one 32x32 fp32 transposition tile per epilogue warp
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;  // + alignment slack
};

// Tile enumeration shared by the three roles: tile t -> (batch, m_tile, n_tile), n fastest.
struct TileCoord {
  int b, m, n;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int m_tiles, int n_tiles) {
  TileCoord c;
  c.n = t % n_tiles;
  const int r = t / n_tiles;
  c.m = r % m_tiles;
  c.b = r / m_tiles;
  return c;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_area = smem + kStages * S::kStageBytes;
  uint8_t* bar_area = stage_area + S::kStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBM - 1) / kBM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles * p.batch;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  const AbortState ab{cta_abort, p.status, p.wait_limit > 0 ? p.wait_limit : (p.wait_flags != nullptr ? kPeerWaitCycles : kWaitCycles)};

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 8);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 0) {
    __syncwarp();  // lane 0 initialised the barriers above; the allocation needs the whole warp converged
    tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int it = 0;  // running stage counter across tiles
      bool ok = true;
      uint32_t regions_ready = 0;  // bit r: rows of source region r have been seen complete
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
        if (p.symmetric && (tc.n + 1) * BN <= tc.m * kBM) continue;  // wholly below the diagonal: mirrored from its twin
        if (!A_MN && p.wait_flags != nullptr) {
          const int r0 = (tc.m * kBM) / p.region_rows;
          const int last_row = min(tc.m * kBM + kBM, p.M) - 1;
          for (int r = r0; r <= last_row / p.region_rows && ok; ++r) {
            if (r < 32 && ((regions_ready >> r) & 1u)) continue;
            ok = wait_region_flag(p.wait_flags + r, p.wait_seq, ab, 4);
            if (r < 32) regions_ready |= 1u << r;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");  // rows written through the generic proxy, read by TMA
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, ab, 1)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, S::kStageBytes);
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) tma_load_3d(sa + j * (64 * kBK * 2), &map_a, fb, tc.m * kBM + j * 64, kb * kBK, tc.b);
          } else {
            tma_load_3d(sa, &map_a, fb, kb * kBK, tc.m * kBM, tc.b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * (64 * kBK * 2), &map_b, fb, tc.n * BN + j * 64, kb * kBK, tc.b);
          } else {
            tma_load_3d(sb, &map_b, fb, kb * kBK, tc.n * BN, tc.b);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN, B_MN);
      int it = 0, local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
        if (p.symmetric && (tc.n + 1) * BN <= tc.m * kBM) continue;
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_ph ^ 1, ab, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, ab, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // K-major: 16 elements of K are 32 bytes inside the 128-byte swizzled row.
            // MN-major: 16 K-rows of 128 bytes = two 1024-byte groups.
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 64 * kBK * 2, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 64 * kBK * 2, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[s]));  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(smem_u32(&acc_full[acc]));
        ++local_tile;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    // Warps 2-5 take the left half of the accumulator's columns, warps 6-9 the right half; warp % 4 selects the
    // TMEM sub-partition (32 lanes = 32 rows).  tcgen05.ld hands every lane one row of a 32-column chunk; the chunk
    // is transposed through a private, XOR-swizzled 4 KB staging tile so that global accesses are coalesced: in the
    // store phase 8 consecutive lanes cover one row (4 fp32 values each), 4 rows per instruction, full sectors.
    // The addend C is read in that same layout, one chunk ahead of its use.
    const int sub = warp & 3;
    const int ep = warp - 2;
    const int half = ep >> 2;
    constexpr int kHalfCols = BN / 2;
    constexpr int kChunks = kHalfCols / 32;
    float* stage = reinterpret_cast<float*>(stage_area) + ep * (32 * 32);
    const int q = lane & 7, rsub = lane >> 3;  // store phase: this lane holds columns [4q, 4q+4) of rows rsub + 4i
    OutT* D = reinterpret_cast<OutT*>(p.D);
    const OutT* C = reinterpret_cast<const OutT*>(p.C);
    bool vec_ok = (p.ldd % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                  (p.C == nullptr || (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.batch_stride_d % 8 == 0);
    for (int d = 0; d < p.n_extra; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.D_extra[d]) & 15) == 0);
    if (p.route_rows > 0) {
      vec_ok = (p.ldd % 8 == 0) && ((p.route_base * sizeof(OutT)) % 16 == 0) && ((p.route_batch_stride * sizeof(OutT)) % 16 == 0);
      for (int d = 0; d < 8; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.D_route[d]) & 15) == 0);
    }
    int local_tile = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
      if (p.symmetric && (tc.n + 1) * BN <= tc.m * kBM) continue;
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_ph, ab, 4)) { ok = false; break; }
      tc_fence_after();
      const int row0 = tc.m * kBM + sub * 32;  // first row of this warp's 32-row band
      const int64_t boff = (int64_t)tc.b * p.batch_stride_d;
      // routed output: destination buffer and row offset of the 8 rows this lane stores (rows row0 + rsub + 4 i)
      OutT* rbase[8];
      if (p.route_rows > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = row0 + rsub + 4 * i;
          const int reg = r / p.route_rows;
          rbase[i] = reinterpret_cast<OutT*>(p.D_route[reg < 8 ? reg : 7]) + p.route_base + (int64_t)tc.b * p.route_batch_stride +
                     (int64_t)(r - reg * p.route_rows) * p.ldd;
        }
      }
      float4 cnext[8];
      bool have_next = false;
      auto fetch_c = [&](int col, float4* dst) {  // coalesced read of C[row0 + rsub + 4i, col + 4q .. +4)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = row0 + rsub + 4 * i;
          dst[i] = (r < p.M) ? load4<OutT>(C + boff + (int64_t)r * p.ldd + col + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
      {
        const int col = tc.n * BN + half * kHalfCols;
        if (C != nullptr && vec_ok && col + 32 <= p.N) {
          fetch_c(col, cnext);
          have_next = true;
        }
      }
#pragma unroll 1
      for (int ci = 0; ci < kChunks; ++ci) {
        const int c0 = half * kHalfCols + ci * 32;
        const int col = tc.n * BN + c0;
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(sub * 32) << 16) + acc * BN + c0, v);
        float4 ccur[8];
        const bool have_cur = have_next;
        if (have_cur) {
#pragma unroll
          for (int i = 0; i < 8; ++i) ccur[i] = cnext[i];
        }
        have_next = false;
        if (ci + 1 < kChunks && C != nullptr && vec_ok && col + 64 <= p.N) {
          fetch_c(col + 32, cnext);
          have_next = true;
        }
        tmem_ld_wait();
        if (col < p.N) {  // warp-uniform
          const int ncols = (p.N - col) < 32 ? (p.N - col) : 32;
          const bool fast = vec_ok && ncols == 32 && (C == nullptr || have_cur);
          // 1. row-per-lane registers -> staging tile (piece j of row `lane` lives at slot j ^ (lane & 7))
#pragma unroll
          for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(stage + lane * 32)[j ^ (lane & 7)] =
                make_float4(p.alpha * __uint_as_float(v[4 * j]), p.alpha * __uint_as_float(v[4 * j + 1]),
                            p.alpha * __uint_as_float(v[4 * j + 2]), p.alpha * __uint_as_float(v[4 * j + 3]));
          __syncwarp();
          // 2. transposed read, addend, coalesced stores
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
                  const int64_t roff = p.route_base + (int64_t)tc.b * p.route_batch_stride + (int64_t)(r - reg * p.route_rows) * p.ldd + col + 4 * q;
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
                      const int64_t roff = p.route_base + (int64_t)tc.b * p.route_batch_stride + (int64_t)(r - reg * p.route_rows) * p.ldd + col + 4 * q + e;
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
            // keep the final values in the staging tile for the mirror pass
            if (p.symmetric) reinterpret_cast<float4*>(stage + rl * 32)[q ^ (rl & 7)] = f;
          }
          // 3. symmetric outputs: the twin tile (this chunk's columns as rows) is skipped by the schedule, so its
          //    elements are written from here, column by column, with consecutive lanes on consecutive addresses
          const int row = row0 + lane;
          const bool mirror = p.symmetric && ((row0 / BN) + 1) * BN <= (col / kBM) * kBM;
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
      ++local_tile;
    }
  }

  // ------------------------------------------------------------------ teardown (also reached after an abort)
  if (*cta_abort != 0) {
    // give loads that may still be in flight time to land before the CTA's shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------------------------------------ host side
static int64_t g_debug_extent_cap = 0;
void gemm_debug_extent_cap(int64_t elements) { g_debug_extent_cap = elements > 0 ? elements : 0; }
int64_t gemm_debug_extent_cap_value() { return g_debug_extent_cap; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int make_tensor_map_3d(CUtensorMap* map, const void* base, bool f32, uint64_t inner, uint64_t outer, uint64_t batch,
                       uint64_t outer_stride_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  const uint64_t esz = f32 ? 4 : 2;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {outer_stride_elems * esz, (batch > 1 ? batch_stride_elems : outer_stride_elems * outer) * esz};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t batch,
                                uint64_t outer_stride_elems, uint64_t batch_stride_elems, uint32_t box_outer) {
  return make_tensor_map_3d(map, base, false, inner, outer, batch, outer_stride_elems, batch_stride_elems, 64, box_outer);
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sm_count, cudaStream_t st) {
  using S = GemmSmem<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -2;
    configured = true;
  }
  const int m_tiles = (p.M + kBM - 1) / kBM, n_tiles = (p.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles * p.batch;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, kGemmThreads, S::kTotal, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int gemm_bf16(const void* A, const void* B, const void* C, void* D, int M, int N, int K, int batch, int64_t lda, int64_t ldb,
              int64_t ldd, int64_t bsa, int64_t bsb, int64_t bsd, bool a_mn_major, bool b_mn_major, bool out_f32, float alpha,
              float beta, bool symmetric, void* const* d_extra, int n_extra, int* status, int sm_count, cudaStream_t st,
              const uint32_t* wait_flags, uint32_t wait_seq, int region_rows, void* const* d_route, int n_route, int route_rows,
              int64_t route_batch_stride, int64_t route_base, long long wait_limit, int impl, void* workspace, uint32_t* ws_flags,
              int split_k) {
  if (impl != 0)
    return gemm_bf16_pair(A, B, C, D, M, N, K, batch, lda, ldb, ldd, bsa, bsb, bsd, a_mn_major, b_mn_major, out_f32, alpha, beta, symmetric,
                          d_extra, n_extra, status, sm_count, st, wait_flags, wait_seq, region_rows, d_route, n_route, route_rows,
                          route_batch_stride, route_base, wait_limit, workspace, ws_flags, split_k);
  const int BN = (N <= 128) ? 128 : 256;
  if (n_route > 0 && (C != nullptr || symmetric || n_extra > 0 || route_rows <= 0 || (int64_t)n_route * route_rows < M || n_route > 8))
    return -5;  // routed output excludes the addend, the mirrored output and the extra destinations
  CUtensorMap ma, mb;
  int r;
  if (a_mn_major)  // memory [K, M]
    r = make_tensor_map_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)batch, (uint64_t)lda, (uint64_t)bsa, 64);
  else  // memory [M, K]
    r = make_tensor_map_bf16(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, (uint64_t)lda, (uint64_t)bsa, kBM);
  if (r != 0) return 100 + r;
  if (b_mn_major)  // memory [K, N]
    r = make_tensor_map_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, (uint64_t)ldb, (uint64_t)bsb, 64);
  else  // memory [N, K]
    r = make_tensor_map_bf16(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)batch, (uint64_t)ldb, (uint64_t)bsb, (uint32_t)BN);
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
  p.wait_limit = wait_limit;
  // extents for the debug build's index checks: last element the epilogue may touch, plus one
  p.d_extent = (int64_t)(batch - 1) * bsd + (int64_t)(M - 1) * ldd + N;
  p.route_extent = n_route > 0 ? route_base + (int64_t)(batch - 1) * route_batch_stride + (int64_t)(route_rows - 1) * ldd + N : 0;
  if (g_debug_extent_cap > 0 && p.d_extent > g_debug_extent_cap) p.d_extent = g_debug_extent_cap;
  p.reduce = 0;
  p.n_static = 0;
  p.splits = 1;
  p.b_box_rows = 64;
  p.epi_backoff_ns = 0;
  p.ws = nullptr;
  p.ws_flags = nullptr;
  for (int i = 0; i < 8; ++i) p.D_route[i] = (n_route > 0) ? d_route[i < n_route ? i : n_route - 1] : nullptr;
#define SEG_GEMM(BNv, AM, BM_)                                                                      \
  (out_f32 ? launch_gemm<BNv, AM, BM_, float>(ma, mb, p, sm_count, st)                              \
           : launch_gemm<BNv, AM, BM_, __nv_bfloat16>(ma, mb, p, sm_count, st))
  if (BN == 256) {
    if (!a_mn_major && !b_mn_major) return SEG_GEMM(256, false, false);
    if (!a_mn_major && b_mn_major) return SEG_GEMM(256, false, true);
    if (a_mn_major && b_mn_major) return SEG_GEMM(256, true, true);
    return SEG_GEMM(256, true, false);
  }
  if (!a_mn_major && !b_mn_major) return SEG_GEMM(128, false, false);
  if (!a_mn_major && b_mn_major) return SEG_GEMM(128, false, true);
  if (a_mn_major && b_mn_major) return SEG_GEMM(128, true, true);
  return SEG_GEMM(128, true, false);
#undef SEG_GEMM
}

}  // namespace seg
