// Allocation-free C entry point (this file has no counterpart in the reference, which has no native code at all).
//
// Who needs it: code that drives this library from a place where device memory cannot be requested - a host
// application that hands out one fixed arena at start-up and forbids later cudaMalloc calls, a real-time or
// safety-certified loop with a "no allocation after initialisation" rule, or a plugin that runs inside another
// framework's stream callback where calling the allocator would deadlock or break that framework's accounting.
// The regular Python bindings obtain their scratch space from the PyTorch caching allocator; those callers cannot.
//
// What it is: the backward of the fused residual-add + RMSNorm (csrc/norm.cu), with the per-CTA partial sums of
// the gain gradient kept in a fixed array that lives inside the loaded library image instead of in allocated
// scratch memory.  Inputs and outputs are still the caller's buffers.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch array can serve.  The array holds SEGPT_NOALLOC_MAX_PARTIAL_ROWS x
// SEGPT_NOALLOC_MAX_D floats (4.6 MiB) and every GPU that loads the library keeps it until the process exits.
#define SEGPT_NOALLOC_MAX_D 2048
#define SEGPT_NOALLOC_MAX_PARTIAL_ROWS 592

// dres = dres_in + d(rmsnorm)/dx, dres_lp = the same in the activation type, dgain = sum_rows dy * x * rstd * scale.
//   dy, dres_lp : [T, d] bf16 (bf16 != 0) or fp32;  dres_in (may be null), x, dres : [T, d] fp32;
//   gain, dgain : [d] fp32;  rstd : [T] fp32;  all device pointers, 16-byte aligned, d a multiple of 4.
//   stream      : a cudaStream_t (null = default stream).
// Returns 0 on success, a negative code otherwise (segpt_noalloc_last_error() describes it).  Problems with
// d > SEGPT_NOALLOC_MAX_D are rejected; the row count T is not limited (the kernel's grid is capped at
// SEGPT_NOALLOC_MAX_PARTIAL_ROWS blocks).
//
// The first call on each device looks up the device address of the scratch array (one cudaGetSymbolAddress with
// that device current); make that first call outside any stream capture.  No call allocates or frees device memory.
// All calls on a device share the one scratch array and it keeps whatever the last call left in it; the kernel
// overwrites every entry it later reads, so nothing has to be cleared between calls, but two calls that overlap
// on the GPU (different streams, no ordering between them) would race on it - serialise them.
int segpt_add_rmsnorm_bwd_noalloc(const void* dy, const float* dres_in, const float* x, const float* gain, const float* rstd,
                                  float* dres, void* dres_lp, float* dgain, int T, int d, float scale, int bf16, void* stream);

const char* segpt_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
