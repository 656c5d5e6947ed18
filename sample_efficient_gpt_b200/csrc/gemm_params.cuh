// Parameter block and host helpers shared by the two tcgen05 GEMM kernels (gemm.cu: one CTA per tile,
// gemm_pair.cu: one CTA pair per tile with cta_group::2 instructions).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100.cuh"

namespace seg {

struct GemmParams {
  int M, N, K, batch;
  float alpha, beta;
  const void* C;  // optional addend, same layout and dtype as D
  void* D;
  int64_t ldd;  // row stride of D and C in elements
  int64_t batch_stride_d;
  int* status;
  int symmetric;     // 1: D is symmetric (A == B, square): tiles wholly below the diagonal are skipped and mirrored
  void* D_extra[7];  // further destinations with D's layout (peer-mapped buffers of other ranks): every tile is
  int n_extra;       // stored to all of them, which turns the epilogue into the all-gather of the result
  // Rows of A arrive from other ranks (expert-parallel dispatch): rows [r * region_rows, (r + 1) * region_rows) of every
  // batch entry are complete once wait_flags[r] >= wait_seq (written by rank r with a system-scope release after its
  // stores).  The producer waits, bounded, for the regions a tile touches before it issues the tile's first load.
  const uint32_t* wait_flags;
  uint32_t wait_seq;
  int region_rows;
  // Routed output (expert-parallel combine): instead of D, rows [r * route_rows, (r + 1) * route_rows) of every batch entry
  // are stored into D_route[r] (peer-mapped buffer of rank r) at element offset
  //   route_base + batch * route_batch_stride + (row - r * route_rows) * ldd + column.
  void* D_route[8];
  int route_rows;  // 0: plain output
  int64_t route_batch_stride, route_base;
  long long wait_limit;  // cycles a wait may stand still before it gives up; 0: the defaults of sm100.cuh
  // elements that D (and every extra destination) / every routed destination holds from its base: read by the index checks
  // of the debug build only (bounds.cuh)
  int64_t d_extent, route_extent;
  // pair kernel only
  int reduce;          // TMA epilogue: 1 = add the tile into D (cp.reduce.async.bulk ... add), 0 = store it
  int n_static, splits;  // schedule (gemm_pair_sched.h): tiles computed whole; ranges of the contraction for the others
  int b_box_rows;        // rows of the K-major B operand's TMA box (64 or 128)
  int epi_backoff_ns;    // sleep between the epilogue warps' polls of the accumulator barrier (0: none)
  uint4* ws;             // workspace slots for the parts of tiles that are cut along the contraction
  uint32_t* ws_flags;    // one word per (slot, rank, epilogue warp), zero between launches
  int swiglu_f;          // SwiGLU epilogue: hidden width F (B holds F gate rows, then F up rows); 0 otherwise
};

// Gives up after half the limit of the barrier waits: the roles that wait (through the ring) for what this producer loads
// then still have time left, and the status word names the flag, not one of its consequences.
__device__ __forceinline__ bool wait_region_flag(const uint32_t* flag, uint32_t seq, const sm100::AbortState& ab, int code) {
  uint32_t v;
  const long long t0 = clock64();
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - seq) >= 0) return true;
    if (*ab.cta_abort != 0) return false;
    if (clock64() - t0 > ab.limit / 2) {
      *ab.cta_abort = 1;
      atomicCAS(ab.global_status, 0, code);
      return false;
    }
    __nanosleep(100);
  }
}

// 3-D tensor map {inner, outer, batch} with a {box_inner, box_outer, 1} box and 128-byte swizzle (box_inner * element size
// must be 128 bytes).  Strides in elements.  Returns 0 or the driver's error code.
int make_tensor_map_3d(CUtensorMap* map, const void* base, bool f32, uint64_t inner, uint64_t outer, uint64_t batch,
                       uint64_t outer_stride_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_outer);

// The pair kernel's launcher (gemm_pair.cu); same contract as gemm_bf16.  `workspace` / `ws_flags`: device buffers of
// gemm_pair_workspace_bytes() bytes and gemm_pair_flag_words() zeroed 32-bit words that launches on one stream share;
// without them (or with split_k == 0) every tile is computed by one pair from start to end.
// (gemm_pair_workspace_bytes / gemm_pair_flag_words are declared in kernels.h.)
int gemm_bf16_pair(const void* A, const void* B, const void* C, void* D, int M, int N, int K, int batch, int64_t lda, int64_t ldb,
                   int64_t ldd, int64_t bsa, int64_t bsb, int64_t bsd, bool a_mn_major, bool b_mn_major, bool out_f32, float alpha,
                   float beta, bool symmetric, void* const* d_extra, int n_extra, int* status, int sm_count, cudaStream_t st,
                   const uint32_t* wait_flags, uint32_t wait_seq, int region_rows, void* const* d_route, int n_route,
                   int route_rows, int64_t route_batch_stride, int64_t route_base, long long wait_limit, void* workspace,
                   uint32_t* ws_flags, int split_k);

}  // namespace seg
