// Index checking for the debug build of the extension (compiled with -DSEG_DEBUG_BOUNDS into _C_dbg.so by
// `python -m sample_efficient_gpt_b200.csrc.build --debug-bounds`, selected at run time with SEGPT_DEBUG_BOUNDS=1).
//
// Kernels that store through computed indices - above all into other ranks' memory - wrap the store in
//     if (SEG_IN_BOUNDS(status, code, first_element, n_elements, extent)) { store }
// In the debug build an access outside [0, extent) is skipped and the first one is recorded in the kernel's status word
// (kBoundsBase + code; the host reads it like any other status).  Nothing traps and nothing is asserted: a wrong index
// costs a missing store and a non-zero status, never a fault.  In the release build the macro is the constant `true`
// and the extents are not even read.  Stores issued by TMA are clipped by the tensor map in hardware and need no check.
#pragma once
#include <cuda_runtime.h>

namespace seg {

constexpr int kBoundsBase = 9000;
// codes: 1 GEMM output, 2 GEMM extra destination, 3 GEMM routed output, 4 GEMM mirrored element, 5 GEMM workspace slot,
//        11 comm wire buffer (own), 12 comm wire buffer (peer), 13 comm gradient bucket,
//        21 MoE expert / slot index, 22 MoE dispatch row, 23 MoE combine output,
//        31 attention output row, 32 attention log-sum-exp, 33 attention key / value gradient

__device__ __forceinline__ bool bounds_check(int* status, int code, long long first, long long n, long long extent) {
  if (first >= 0 && first + n <= extent) return true;
  if (status != nullptr) atomicCAS(status, 0, kBoundsBase + code);
  return false;
}

}  // namespace seg

#ifdef SEG_DEBUG_BOUNDS
#define SEG_IN_BOUNDS(status, code, first, n, extent) \
  seg::bounds_check((status), (code), (long long)(first), (long long)(n), (long long)(extent))
#else
#define SEG_IN_BOUNDS(status, code, first, n, extent) true
#endif
