// Gradient-bucket all-reduce and all-gather over NVLink peer memory, written as single kernels that fuse the
// collective with the bf16 <-> fp32 casts around it.  One process per GPU; every rank launches the same kernel on
// its own device; ranks meet at flag barriers that live in symmetric (peer-mapped) memory.
//
// all-reduce of a bucket (fp32 gradients G[n] in place, bf16 on the wire, W = this rank's wire buffer):
//   A  pack    : W_me[s, b] = bf16(G[s, b])                       for every slice s != me, sub-slice b = blockIdx.x
//      barrier : block b of every rank has packed
//   B  reduce  : slice me, sub-slice b: sum over ranks p (fixed order) of W_p[me, b] in fp32 -> G (fp32, final)
//                and the bf16 result is stored into W_p[me, b] of every peer p           (reduce-scatter + push)
//                NVLS variant: one multimem.ld_reduce on the multicast address replaces the w loads, one
//                multimem.st replaces the w stores (the switch reduces and broadcasts).
//      barrier : block b of every rank has pushed
//   C  unpack  : G[s, b] = fp32(W_me[s, b]) for the slices owned by other ranks          (all-gather landing + cast)
// Block b only ever touches sub-slice b, on every rank, so per-block barriers suffice and no grid-wide sync is needed.
// Flags are monotonically increasing sequence numbers (never reset), one word per (block, source rank).
// Every wait is bounded: after the wait limit (a kernel argument, kCommWaitCycles by default) without the peer's flag the
// block records the failure in a status word and stops touching remote memory; the host raises an error after the step.
//
// The reference reduces each bucket with an NCCL all-reduce of a bf16 copy and casts back on the host side
// (training/distributed/ddp_bucket.py:91-104,118-134).
#include "bounds.cuh"
#include "common.cuh"
#include "kernels.h"

namespace seg {

constexpr long long kCommWaitCycles = 20000000000LL;  // ~10 s: ranks may be skewed by a checkpoint write

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct CommPeers {
  void* buf[kMaxRanks];       // wire buffers of every rank (peer-mapped)
  uint32_t* flags[kMaxRanks];  // flag arrays of every rank: [blocks][kMaxRanks]
};

// All threads of the block call this.  Returns false when a peer did not show up in time.
// Ordering: the block's stores happen before the CTA barrier, the flag is written after it with a system-scope release by
// the threads that passed the barrier - release is cumulative, so a peer that acquires the flag sees every store of the
// block.  (One release per peer instead of a system fence in each of the 512 threads: the fences were the larger part of
// a small bucket's time.)
__device__ __forceinline__ bool block_barrier(const CommPeers& pe, int rank, int world, uint32_t seq, int* status, long long limit) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    st_release_sys(pe.flags[peer] + (size_t)blockIdx.x * kMaxRanks + rank, seq);
    const uint32_t* mine = pe.flags[rank] + (size_t)blockIdx.x * kMaxRanks + peer;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - seq) < 0) {
      if (clock64() - t0 > limit) {
        atomicCAS(status, 0, 1000 + peer);
        ok_s = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ void multimem_ld_reduce_bf16x8(const void* mc_ptr, uint32_t* r) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "l"(mc_ptr)
               : "memory");
}
__device__ __forceinline__ void multimem_st_bf16x8(void* mc_ptr, const uint32_t* r) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3])
               : "memory");
}

// n is padded by the host so that n % (world * 8) == 0; slice = n / world elements.
// sq_out (optional): += sum of squares of the reduced values of this rank's slice (the gradient norm then needs only a
// sum of one scalar per rank instead of a pass over every gradient tensor).
__global__ void __launch_bounds__(512) allreduce_bucket_kernel(float* __restrict__ grads, CommPeers pe, void* mc_base,
                                                             int64_t wire_off, int64_t n, int rank, int world, uint32_t seq,
                                                             int* status, float* __restrict__ sq_out, long long limit,
                                                             int64_t wire_elems) {
  const int64_t slice = n / world;
  const int nb = gridDim.x;
  // sub-slice b of a slice, in units of 8 elements
  const int64_t vecs = slice / 8;
  const int64_t v0 = vecs * blockIdx.x / nb, v1 = vecs * (blockIdx.x + 1) / nb;
  __nv_bfloat16* w_me = reinterpret_cast<__nv_bfloat16*>(pe.buf[rank]) + wire_off;

  // A: pack the slices owned by other ranks (this rank's own slice is read as fp32 in phase B)
  constexpr int kUnroll = 4;
  for (int s = 0; s < world; ++s) {
    if (s == rank && mc_base == nullptr) continue;  // the multicast reduction reads every rank's copy from the wire buffers
    const int64_t base = (int64_t)s * slice;
    for (int64_t v = v0 + threadIdx.x; v < v1; v += (int64_t)blockDim.x * kUnroll) {
      float f[kUnroll][8];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v + (int64_t)u * blockDim.x < v1) load8<float>(grads + base + (v + (int64_t)u * blockDim.x) * 8, f[u]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v + (int64_t)u * blockDim.x < v1 && SEG_IN_BOUNDS(status, 11, wire_off + base + (v + (int64_t)u * blockDim.x) * 8, 8, wire_elems))
          store8<__nv_bfloat16>(w_me + base + (v + (int64_t)u * blockDim.x) * 8, f[u]);
    }
  }
  if (!block_barrier(pe, rank, world, seq, status, limit)) return;

  // B: reduce my slice, push the result to everyone
  float sq = 0.f;
  {
    const int64_t base = (int64_t)rank * slice;
    if (mc_base != nullptr) {
      __nv_bfloat16* mc = reinterpret_cast<__nv_bfloat16*>(mc_base) + wire_off;
      for (int64_t v = v0 + threadIdx.x; v < v1; v += (int64_t)blockDim.x * kUnroll) {
        uint32_t r[kUnroll][4];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (v + (int64_t)u * blockDim.x < v1) multimem_ld_reduce_bf16x8(mc + base + (v + (int64_t)u * blockDim.x) * 8, r[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (v + (int64_t)u * blockDim.x < v1) {
            const int64_t vv = v + (int64_t)u * blockDim.x;
            multimem_st_bf16x8(mc + base + vv * 8, r[u]);
            float f[8];
            unpack8(*reinterpret_cast<const bf16x8*>(r[u]), f);
            store8<float>(grads + base + vv * 8, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) sq = fmaf(f[j], f[j], sq);
          }
      }
    } else {
      // kPeerUnroll vectors per thread and trip: (world - 1) * kPeerUnroll independent 16-byte peer loads are in flight before
      // the first is used, which is what hides the NVLink round trip at small world sizes
      constexpr int kPeerUnroll = 2;
      for (int64_t v = v0 + threadIdx.x; v < v1; v += (int64_t)blockDim.x * kPeerUnroll) {
        bf16x8 in[kPeerUnroll][kMaxRanks];
        float own[kPeerUnroll][8];
#pragma unroll
        for (int u = 0; u < kPeerUnroll; ++u) {
          const int64_t vv = v + (int64_t)u * blockDim.x;
          if (vv < v1) {
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
              if (p < world && p != rank)
                in[u][p] = *reinterpret_cast<const bf16x8*>(reinterpret_cast<const __nv_bfloat16*>(pe.buf[p]) + wire_off + base + vv * 8);
            load8<float>(grads + base + vv * 8, own[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < kPeerUnroll; ++u) {
          const int64_t vv = v + (int64_t)u * blockDim.x;
          if (vv >= v1) continue;
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)  // fixed order of summation on every rank; each term is bf16-rounded
            if (p < world) {
              float f[8];
              unpack8(p == rank ? pack8(own[u]) : in[u][p], f);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] += f[j];
            }
          const bf16x8 out = pack8(acc);
          float fin[8];
          unpack8(out, fin);  // every rank ends with the same bf16-rounded value
          if (SEG_IN_BOUNDS(status, 13, base + vv * 8, 8, n)) store8<float>(grads + base + vv * 8, fin);
#pragma unroll
          for (int j = 0; j < 8; ++j) sq = fmaf(fin[j], fin[j], sq);
          if (SEG_IN_BOUNDS(status, 12, wire_off + base + vv * 8, 8, wire_elems)) {
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
              if (p < world && p != rank)
                *reinterpret_cast<bf16x8*>(reinterpret_cast<__nv_bfloat16*>(pe.buf[p]) + wire_off + base + vv * 8) = out;
          }
        }
      }
    }
  }
  if (sq_out != nullptr) {
    __shared__ float red_s[32];
    const float total = block_sum(sq, red_s);
    if (threadIdx.x == 0) atomicAdd(sq_out, total);
  }
  if (!block_barrier(pe, rank, world, seq + 1, status, limit)) return;

  // C: unpack the other owners' slices
  for (int s = 0; s < world; ++s) {
    if (s == rank) continue;
    const int64_t base = (int64_t)s * slice;
    for (int64_t v = v0 + threadIdx.x; v < v1; v += (int64_t)blockDim.x * kUnroll) {
      float f[kUnroll][8];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v + (int64_t)u * blockDim.x < v1) load8<__nv_bfloat16>(w_me + base + (v + (int64_t)u * blockDim.x) * 8, f[u]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v + (int64_t)u * blockDim.x < v1 && SEG_IN_BOUNDS(status, 13, base + (v + (int64_t)u * blockDim.x) * 8, 8, n))
          store8<float>(grads + base + (v + (int64_t)u * blockDim.x) * 8, f[u]);
    }
  }
}

// All-gather in place: `buf` (symmetric, 16-byte elements view) holds world chunks of chunk_bytes; rank r's chunk r is
// valid on entry, all chunks are valid on exit.  Pull model: every rank copies the peers' chunks from their memory.
__global__ void __launch_bounds__(512) allgather_kernel(CommPeers pe, int64_t off_bytes, int64_t chunk_bytes, int rank, int world,
                                                      uint32_t seq, int* status, long long limit) {
  if (!block_barrier(pe, rank, world, seq, status, limit)) return;
  const int nb = gridDim.x;
  const int64_t vecs = chunk_bytes / 16;
  const int64_t v0 = vecs * blockIdx.x / nb, v1 = vecs * (blockIdx.x + 1) / nb;
  uint4* mine = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pe.buf[rank]) + off_bytes);
  for (int step = 1; step < world; ++step) {
    const int p = (rank + step) % world;  // start with different peers on different ranks
    const uint4* theirs = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(pe.buf[p]) + off_bytes) + (int64_t)p * vecs;
    uint4* dst = mine + (int64_t)p * vecs;
    for (int64_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) dst[v] = theirs[v];
  }
  // nobody may overwrite its chunk (next step) before every peer has read it
  block_barrier(pe, rank, world, seq + 1, status, limit);
}

static CommPeers make_peers(void* const* bufs, uint32_t* const* flags, int world) {
  CommPeers pe;
  for (int i = 0; i < kMaxRanks; ++i) {
    pe.buf[i] = i < world ? bufs[i] : nullptr;
    pe.flags[i] = i < world ? flags[i] : nullptr;
  }
  return pe;
}

void comm_allreduce_bucket(float* grads, void* const* wire_bufs, uint32_t* const* flags, void* mc_base, int64_t wire_off,
                           int64_t n, int rank, int world, uint32_t seq, int blocks, int* status, cudaStream_t st, float* sq_out,
                           long long wait_cycles, int64_t wire_elems) {
  if (wire_elems <= 0) wire_elems = wire_off + n;  // callers that do not say how long the wire buffers are: this bucket's end
  allreduce_bucket_kernel<<<blocks, 512, 0, st>>>(grads, make_peers(wire_bufs, flags, world), mc_base, wire_off, n, rank, world, seq,
                                                  status, sq_out, wait_cycles > 0 ? wait_cycles : kCommWaitCycles, wire_elems);
}

void comm_allgather(void* const* bufs, uint32_t* const* flags, int64_t off_bytes, int64_t chunk_bytes, int rank, int world,
                    uint32_t seq, int blocks, int* status, cudaStream_t st, long long wait_cycles) {
  allgather_kernel<<<blocks, 512, 0, st>>>(make_peers(bufs, flags, world), off_bytes, chunk_bytes, rank, world, seq, status,
                                           wait_cycles > 0 ? wait_cycles : kCommWaitCycles);
}

}  // namespace seg
