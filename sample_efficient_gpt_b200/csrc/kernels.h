// Host-callable launchers of the sm_100a kernels (raw pointers + stream; no framework types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace seg {

// ---- norm.cu
constexpr int kNormBwdMaxGrid = 148 * 4;  // CTAs of the backward kernel == rows of its dgain scratch
void add_rmsnorm_fwd(const float* res, const void* delta, const float* gain, float* x_out, void* y, float* rstd, float* kurt,
                     int T, int d, float scale, float eps, bool bf16, cudaStream_t st);
int add_rmsnorm_bwd_grid(int T);
// scratch: fp32 [add_rmsnorm_bwd_grid(T), d]
void add_rmsnorm_bwd(const void* dy, const float* dres_in, const float* x, const float* gain, const float* rstd, float* dres,
                     void* dres_lp, float* dgain, float* scratch, int T, int d, float scale, bool bf16, cudaStream_t st);

// ---- elementwise.cu
void swiglu_fwd(const void* u, void* f, int64_t T, int F, bool bf16, cudaStream_t st);
void swiglu_bwd(const void* df, const void* u, void* du, int64_t T, int F, bool bf16, cudaStream_t st);
// z and dz are addressed as [token * stride + head] (stride in elements; 0 = H, i.e. compact [T, H]).
void gate_fwd(const void* o, const void* z, void* g, int64_t T, int H, int hd, bool bf16, cudaStream_t st, int64_t z_stride = 0);
void gate_bwd(const void* dg, const void* o, const void* z, void* dout, void* dz, int64_t T, int H, int hd, bool bf16, cudaStream_t st,
              int64_t z_stride = 0, int64_t dz_stride = 0);

// ---- qkv_post.cu
constexpr int kQkvPostMaxGrid = 148 * 8;  // CTAs of the kernels == rows of the backward's scalar scratch
int qkv_post_bwd_grid(int64_t T, int nslots, int hd);
struct QkvPostParams {
  int B, S, H, Hkv, hd;
  bool qknorm;
  const float* cos;  // [>=S, hd/2]
  const float* sin;
  const float* qgain;   // [1]
  const float* alpha1;  // [1]
  const float* alpha2;  // [1]
  const float* vscale;  // [1]
  int64_t qkv_stride;   // row stride (elements) of qkv and dqkv: (H + 2 Hkv) * hd, or more when the projection is wider
  const int* pos;       // optional device scalar added to every token's position (decode: S == 1, position = cache length)
  bool dv1_accumulate = false;  // backward: add the value-residual gradient to dv1_out instead of overwriting it
  int* status = nullptr;        // device word for the bounded waits of the shared-memory variant (nullptr: that variant is not used)
};
// Shared-memory variants (qkv_post_tile.cu; bf16, head_dim 64, S a multiple of the token tile).  They return false / 0 when the
// call is not theirs and nothing was launched.
bool qkv_post_fwd_tile(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st);
int qkv_post_bwd_tile(const void* dq, const void* dk, const void* dv, const void* qkv, const void* v1, void* dqkv, float* dv1_out,
                      float* partial, int partial_rows, const QkvPostParams& p, bool bf16, cudaStream_t st);
void qkv_post_fwd(const void* qkv, const void* v1, void* q, void* k, void* v, const QkvPostParams& p, bool bf16, cudaStream_t st);
// dv_is_f32: dv is fp32 (first block, after the v1 gradients were added); dv1_out fp32 [T,Hkv,hd] or nullptr;
// scalars: fp32[4] = {dqgain, dalpha1, dalpha2, dvscale}; partial: scratch fp32 [qkv_post_bwd_grid(...), 4].
void qkv_post_bwd(const void* dq, const void* dk, const void* dv, bool dv_is_f32, const void* qkv, const void* v1, void* dqkv,
                  float* dv1_out, float* scalars, float* partial, const QkvPostParams& p, bool bf16, cudaStream_t st);

// ---- cross_entropy.cu
// In place over a chunk of logits [rows, V] (bf16): writes per-row loss, z and lse, and overwrites the
// logits with grad_scale * (softmax * (1 + 2 s lse) - onehot) (zero rows for ignored targets) when
// write_grad.  logit_scale multiplies the raw logits first (and the gradient once more).
void ce_chunk_fwd_bwd(void* logits, const int64_t* targets, float* loss, float* z, float* lse, int rows, int V,
                      float lse_square_scale, int64_t ignore_index, float grad_scale, float logit_scale, bool write_grad,
                      cudaStream_t st);

// ---- multi_tensor.cu
void adamw_multi(float** p, const float** g, float** m, float** v, void** shadow, const int64_t* sizes, const int32_t* chunk_tensor,
                 const int64_t* chunk_offset, int n_chunks, int chunk_elems, float lr, float wd, float b1, float b2, float eps,
                 float step_size, cudaStream_t st);
void ema_multi(float** ema, const float** src, const int64_t* sizes, const int32_t* chunk_tensor, const int64_t* chunk_offset,
               int n_chunks, int chunk_elems, float decay, cudaStream_t st);
void cast_multi(void** dst_bf16, const float** src, const int64_t* sizes, const int32_t* chunk_tensor, const int64_t* chunk_offset,
                int n_chunks, int chunk_elems, cudaStream_t st);

// ---- muon.cu
int muon_chunks_per_matrix(int64_t numel);
// momentum [slots, numel] fp32 and xout [slots, numel] bf16 are indexed through slot_of[i]; grads[i] are fp32 pointers.
// partial: scratch fp32 [n_mats * muon_chunks_per_matrix(numel)].  numel must be a multiple of 8.
void muon_momentum(const float* const* grads, const int32_t* slot_of, float* momentum, void* xout, float* partial, int n_mats,
                   int64_t numel, float mu, float eps, cudaStream_t st);
// v [slots, R, C] bf16; second / sq / mult fp32 [n_mats, R] (R >= C) or [n_mats, C]; params[i] fp32, shadows[i] bf16 or null
// array; sq_sum_out accumulates sum ||v_i||_F^2.  mode: 0 none, 1 plain decay, 2 cautious decay.  C % 8 == 0.
void muon_tail(const void* v, const int32_t* slot_of, float* second, float* sq, float* mult, float* const* params,
               void* const* shadows, float* sq_sum_out, int n_mats, int R, int C, float beta2, int normalize, float lr_eff,
               float decay, int mode, cudaStream_t st);

// ---- comm.cu (NVLink peer-memory collectives; one process per GPU)
constexpr int kMaxRanks = 8;
constexpr int kCommMaxBlocks = 128;  // flag words per rank = kCommMaxBlocks * kMaxRanks
// grads: this rank's fp32 bucket (n elements, n % (world*8) == 0), reduced in place across ranks with bf16 on the wire.
// wire_bufs[p] / flags[p]: peer-mapped wire buffer and flag array of rank p; wire_off: element offset of the bucket in the
// wire buffers; mc_base: NVLS multicast address of the wire buffer or null; seq: first of two consecutive barrier numbers.
// sq_out (optional, fp32 scalar): += sum of squares of the reduced slice this rank owns.
void comm_allreduce_bucket(float* grads, void* const* wire_bufs, uint32_t* const* flags, void* mc_base, int64_t wire_off,
                           int64_t n, int rank, int world, uint32_t seq, int blocks, int* status, cudaStream_t st,
                           float* sq_out = nullptr, long long wait_cycles = 0, int64_t wire_elems = 0);
// wire_elems: bf16 elements every wire buffer holds (index checks of the debug build; 0: wire_off + n).
// wait_cycles (both collectives): how long a block waits for a peer's flag before it gives up and sets *status to
// 1000 + peer (0: about ten seconds).
// bufs[p] + off_bytes holds `world` chunks of chunk_bytes (multiple of 16); chunk `rank` is valid on entry, all on exit.
void comm_allgather(void* const* bufs, uint32_t* const* flags, int64_t off_bytes, int64_t chunk_bytes, int rank, int world,
                    uint32_t seq, int blocks, int* status, cudaStream_t st, long long wait_cycles = 0);

// ---- moe.cu (router, slot assignment, expert-parallel push / pull over peer memory)
constexpr int kMoeMaxExperts = 32;
constexpr int kMoeMaxTopK = 4;
constexpr int kMoeTokensPerBlock = 32;  // granularity of the (token, choice)-ordered slot scan
constexpr int kMoeTailBlocks = 4;       // zero-filling CTAs per expert in the push kernel
// x [T, d] bf16, wr [E, d] fp32 -> probs [T, E] fp32, idx [T, k] int32, w [T, k] fp32 (renormalised top-k weights);
// block_counts / block_off: int32 scratch [ceil(T / kMoeTokensPerBlock), E]; totals [E] assignments per expert.
// Returns non-zero when E, k or d is out of range (E <= 32, k <= min(4, E), d % 8 == 0).
int moe_route(const void* x, const float* wr, int T, int d, int E, int k, float* probs, int* idx, float* w, int* block_counts,
              int* block_off, int* totals, cudaStream_t st);
// slot [T, k]: position of the assignment inside its expert (token-major order), -1 when >= cap.
void moe_slots(const int* idx, const int* block_off, int T, int E, int k, int cap, int* slot, cudaStream_t st);
// dst[r]: rank r's buffer [E / world][world][cap][d] bf16 (peer-mapped).  Row (e_local, rank, slot) <- w * x[t] for every kept
// assignment (w == nullptr: unscaled); rows [min(totals[e], cap), cap) of this rank's regions are zero-filled.
// flags (optional): flags[r] is rank r's flag array; after all rows are stored, flags[r][rank] = seq is written with a
// system-scope release (consumed by gemm_bf16's wait_flags).  done_counter: a zero-initialised device word.
void moe_push(const void* x, const int* idx, const int* slot, const float* w, const int* totals, void* const* dst, int T, int d,
              int E, int k, int cap, int world, int rank, cudaStream_t st, uint32_t* const* flags = nullptr,
              uint32_t* done_counter = nullptr, uint32_t seq = 0, int* status = nullptr);
// status (optional): receives the code of the debug build's index checks (bounds.cuh).
// out[t] = sum over kept assignments of w * src[owner](e_local, rank, slot) (w == nullptr: 1); with dots != nullptr also
// dots[t, c] = <g[t], src2[owner] row> (0 for dropped assignments).  out is bf16 or fp32.
void moe_pull(void* const* src, void* const* src2, const int* idx, const int* slot, const float* w, const void* g, void* out,
              bool out_f32, float* dots, int T, int d, int E, int k, int cap, int world, int rank, cudaStream_t st);
// dlogits [T, E] from the gradient of the renormalised weights dw [T, k] and a per-expert additive term aux_vec [E] on
// d(probs) (load-balance loss), through the softmax.
void moe_route_bwd(const float* probs, const int* idx, const float* dw, const float* aux_vec, int T, int E, int k, float* dlogits,
                   cudaStream_t st);

// ---- gemm.cu (tcgen05 / TMEM / TMA)
// D[b] = alpha * A[b] * op(B[b]) + beta * C[b], bf16 inputs, fp32 accumulation, D and C bf16 or fp32.
//   a_mn_major = false: A is [M, K] row-major (lda = row stride);  true: A is stored [K, M].
//   b_mn_major = false: B is [N, K] row-major (the product is A * B^T); true: B is stored [K, N].
//   symmetric: A == B and D square: only tiles on or above the diagonal are computed, the rest is mirrored.
// d_extra[0..n_extra): up to 7 further destination buffers with D's layout (peer memory of other ranks).
// Strides are in elements; bases and row strides must be 16-byte aligned.  Returns 0 when the launch was issued.
// `status` is a device int that stays 0 unless a bounded wait inside the kernel gave up.
// wait_flags (optional, A row-major only): rows [r * region_rows, (r+1) * region_rows) of A are written by another rank and
// are complete once wait_flags[r] >= wait_seq; the kernel waits (bounded) per tile instead of the host ordering the launch.
int gemm_bf16(const void* A, const void* B, const void* C, void* D, int M, int N, int K, int batch, int64_t lda, int64_t ldb,
              int64_t ldd, int64_t bsa, int64_t bsb, int64_t bsd, bool a_mn_major, bool b_mn_major, bool out_f32, float alpha,
              float beta, bool symmetric, void* const* d_extra, int n_extra, int* status, int sm_count, cudaStream_t st,
              const uint32_t* wait_flags = nullptr, uint32_t wait_seq = 0, int region_rows = 0, void* const* d_route = nullptr,
              int n_route = 0, int route_rows = 0, int64_t route_batch_stride = 0, int64_t route_base = 0, long long wait_limit = 0,
              int impl = 1, void* workspace = nullptr, uint32_t* ws_flags = nullptr, int split_k = 1);
// wait_limit: cycles a wait inside the kernel may stand still before it gives up (0: about one second, ten with wait_flags).
// impl: 1 = CTA-pair kernel (cta_group::2, 256-row tiles), 0 = one CTA per 128-row tile.  workspace / ws_flags / split_k:
// the pair kernel's buffers for tiles cut along the contraction (sizes: gemm_pair_workspace_bytes / gemm_pair_flag_words) and
// the switch for cutting.
// Up projection of a SwiGLU feed-forward with the activation in the epilogue (CTA-pair kernel): U [M, 2F] = X W^T for
// W = [F gate rows | F up rows] and Fout [M, F] = silu(U[:, :F]) * U[:, F:], formed from the bf16-rounded U.  bf16, row-major,
// F a multiple of 128, K a multiple of 8, 16-byte aligned bases and row strides.
int gemm_swiglu_pair(const void* X, const void* W, void* U, void* Fout, int M, int F, int K, int64_t ldx, int64_t ldw, int64_t ldu,
                     int64_t ldf, int* status, int sm_count, cudaStream_t st, long long wait_limit = 0);
// Data gradient of the down projection with the SwiGLU backward in the epilogue: DU [M, 2F] = (d gate | d up) from dY [M, K],
// W [K, F] (row-major: the down projection's weight), U [M, 2F] = (gate | up); df = dY W is rounded to bf16 on chip, as a
// stored df would be, and never written.  bf16, F a multiple of 256.
int gemm_swiglu_bwd_pair(const void* dY, const void* W, const void* U, void* DU, int M, int F, int K, int64_t ldy, int64_t ldw,
                         int64_t ldu, int64_t lddu, int* status, int sm_count, cudaStream_t st, long long wait_limit = 0);
// Debug build only (no effect otherwise): every GEMM launched afterwards pretends that its output holds at most `elements`
// elements (0: off), so that a test can watch the index checks refuse in-range stores - and only those - without any fault.
void gemm_debug_extent_cap(int64_t elements);
int64_t gemm_debug_extent_cap_value();
size_t gemm_pair_workspace_bytes();
size_t gemm_pair_flag_words();
// d_route (optional): routed output - rows [r * route_rows, (r+1) * route_rows) of every batch entry go to d_route[r] (a buffer of
// rank r, peer-mapped) at element offset route_base + batch * route_batch_stride + (row - r * route_rows) * ldd + column; D is
// not written.  Not combinable with C, symmetric or d_extra.

// ---- attn_bwd.cu (tcgen05 flash attention, backward)
// q, o, d_o, dq [B,S,H,hd]; k, v, dk, dv [B,S,Hkv,hd] bf16; lse [B,H,S] fp32 from the forward.  Scratch: dq_acc fp32 like q
// (zeroed here), dsum and lse2 fp32 [B,H,S].  Causal; hd == 64, S % 128 == 0.  Returns 0 when launched.
// prof (both kernels, optional): 16 int64 on the device that receive per-stage cycle counts of one CTA.
int attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
             float* dq_acc, float* dsum, float* lse2, int B, int S, int H, int Hkv, int hd, int* status, cudaStream_t st,
             long long* prof = nullptr);

// ---- attn_fwd.cu (tcgen05 flash attention, forward)
// q [B,S,H,hd], k/v [B,S,Hkv,hd] bf16, o like q, lse fp32 [B,H,S]; causal; hd == 64, any S >= 1.
// Returns 0 when launched, a negative code for unsupported shapes.
int attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int H, int Hkv, int hd, int* status,
             cudaStream_t st, long long* prof = nullptr);

}  // namespace seg
