// Schedule of the CTA-pair GEMM (gemm_pair.cu): plain C++ that compiles for the host and the device, so the same
// functions place the work in the kernel, size the grid on the host and can be checked exhaustively on a CPU.
//
// Tiles are 256 rows x (256 | last-column remainder) columns.  Order: column index fastest (the narrower last-column tile
// closes its row of tiles, so that the pairs that run narrow tiles - which move more operand bytes per FLOP - are always
// a minority), then row tile, then batch; a symmetric output lists only tiles on or above the diagonal.
// Work items are dealt round-robin to the pairs, so that the pairs running at the same time work on neighbouring tiles
// and walk the contraction in step - operand panels shared between tiles are then fetched from HBM once and served from
// L2 to the others.  The first n_static tiles are whole-tile items.  The remaining R tiles (the last, partly filled wave,
// or everything when there are fewer tiles than pairs) are cut into `splits` ranges of the contraction, range index
// outermost: the item of range ks adds the running sum that range ks-1 left in its workspace slot to its own raw fp32
// accumulator and leaves the new sum in its own slot; the item of the last range owns the tile and runs the epilogue on
// the total.  The order of the additions is fixed, so results are reproducible, and the slot an item reads always
// belongs to an item with a lower index, which its pair reaches no later than this one is reached.
#pragma once
#if !defined(__CUDACC__)
#define __host__
#define __device__
#endif

namespace seg {

constexpr int kPairM = 256;  // rows of a pair tile, 128 per CTA
constexpr int kPairN = 256;  // widest tile
constexpr int kPairK = 64;   // contraction elements per stage (one k-block)
constexpr int kPairMaxSlots = 384;                  // workspace slots (parts in flight) per stream
constexpr int kPairSlotPieces = 2 * 8 * 4 * 8 * 32;  // 16-byte pieces per slot: (rank, epilogue warp, chunk, quad, lane)
constexpr int kPairMaxSplits = 12;

struct PairSched {
  int m_tiles, n_full, tail_nt, batch, kb_total, symmetric;
  int per_batch, total;  // tiles per batch entry, tiles in all
  int n_static, splits, kb_per, rem_tiles, n_items;
};

__host__ __device__ inline PairSched make_pair_sched(int M, int N, int K, int batch, int symmetric, int n_static, int splits) {
  PairSched s;
  s.m_tiles = (M + kPairM - 1) / kPairM;
  s.n_full = N / kPairN;
  const int rem = N - s.n_full * kPairN;
  s.tail_nt = rem > 0 ? ((rem + 31) / 32) * 32 : 0;
  s.batch = batch;
  s.kb_total = (K + kPairK - 1) / kPairK;
  s.symmetric = symmetric;
  const int n_cols = s.n_full + (rem > 0 ? 1 : 0);
  // symmetric: row m holds column tiles m .. n_cols - 1
  s.per_batch = symmetric ? n_cols * (n_cols + 1) / 2 - (n_cols - s.m_tiles) * (n_cols - s.m_tiles + 1) / 2 : s.m_tiles * n_cols;
  s.total = batch * s.per_batch;
  s.splits = splits < 1 ? 1 : splits;
  s.n_static = (s.splits == 1 || n_static > s.total) ? s.total : (n_static < 0 ? 0 : n_static);
  s.rem_tiles = s.total - s.n_static;
  s.kb_per = (s.kb_total + s.splits - 1) / s.splits;
  s.n_items = s.n_static + s.rem_tiles * s.splits;
  return s;
}

struct PairItem {
  int t, b, m, n, nt, kb0, kb1;
  int ks;  // range of the contraction this item covers, -1 for a whole tile
};

__host__ __device__ inline void pair_tile_coords(const PairSched& s, int t, PairItem& c) {
  const int n_cols = s.n_full + (s.tail_nt > 0 ? 1 : 0);
  c.b = t / s.per_batch;
  int idx = t - c.b * s.per_batch;
  if (s.symmetric) {
    int m = 0, row = n_cols;
    while (idx >= row) {
      idx -= row;
      --row;
      ++m;
    }
    c.m = m;
    c.n = m + idx;
  } else {
    c.m = idx / n_cols;
    c.n = idx - c.m * n_cols;
  }
  c.nt = c.n < s.n_full ? kPairN : s.tail_nt;
}

__host__ __device__ inline PairItem pair_item(const PairSched& s, int i) {
  PairItem it;
  if (i < s.n_static) {
    it.t = i;
    it.ks = -1;
    it.kb0 = 0;
    it.kb1 = s.kb_total;
  } else {
    const int j = i - s.n_static;
    it.ks = j / s.rem_tiles;
    it.t = s.n_static + (j - it.ks * s.rem_tiles);
    it.kb0 = it.ks * s.kb_per;
    it.kb1 = it.kb0 + s.kb_per < s.kb_total ? it.kb0 + s.kb_per : s.kb_total;
  }
  pair_tile_coords(s, it.t, it);
  return it;
}
// An item of ranges 0 .. splits-2 writes slot pair_slot(); the item of range splits-1 (or a whole-tile item) owns the tile.
__host__ __device__ inline bool pair_item_owns(const PairSched& s, const PairItem& it) { return it.ks < 0 || it.ks == s.splits - 1; }
__host__ __device__ inline int pair_slot(const PairSched& s, int ks, int t) { return ks * s.rem_tiles + (t - s.n_static); }

// ---------------------------------------------------------------------------------------------------------- host model
// Makespan, in k-blocks of a full-width tile, of dealing a schedule round-robin to `pairs` pairs.  Each item costs its
// k-blocks scaled by its width plus a fixed overhead (pipeline fill, accumulator hand-over, epilogue); an item of a cut tile also
// pays for reading and writing the running sum.  Only evaluated for problems of a few waves (pair_choose_split).
inline double pair_makespan(const PairSched& s, int pairs) {
  const double kItemOverhead = 5.0, kPartRead = 2.0, kPartWrite = 1.0;
  const int P = s.n_items < pairs ? s.n_items : pairs;
  if (P <= 0) return 0.0;
  double load[256];
  if (P > 256) return 0.0;
  for (int i = 0; i < P; ++i) load[i] = 0.0;
  for (int i = 0; i < s.n_items; ++i) {
    const PairItem it = pair_item(s, i);
    double c = (it.nt / 256.0) * (it.kb1 - it.kb0) + kItemOverhead;
    if (it.ks >= 0) c += (it.ks > 0 ? kPartRead : 0.0) + (it.ks < s.splits - 1 ? kPartWrite : 0.0);
    load[i % P] += c;
  }
  double m = 0.0;
  for (int i = 0; i < P; ++i) m = load[i] > m ? load[i] : m;
  return m;
}

// Chooses how many trailing tiles to cut along the contraction, and into how many ranges.
inline void pair_choose_split(int M, int N, int K, int batch, int symmetric, int pairs, bool allow, int& n_static, int& splits) {
  const PairSched whole = make_pair_sched(M, N, K, batch, symmetric, 0, 1);
  n_static = whole.total;
  splits = 1;
  if (!allow || whole.total >= 4 * pairs || whole.kb_total < 16) return;
  double best = pair_makespan(whole, pairs);
  const int waves = whole.total / pairs;
  for (int keep = waves; keep >= 0 && keep >= waves - 1; --keep) {
    const int ns = keep * pairs;
    const int R = whole.total - ns;
    if (R <= 0) continue;
    for (int sp = 2; sp <= kPairMaxSplits; ++sp) {
      if (whole.kb_total / sp < 8 || (long long)(sp - 1) * R > kPairMaxSlots) break;
      const PairSched cand = make_pair_sched(M, N, K, batch, symmetric, ns, sp);
      if ((sp - 1) * cand.kb_per >= cand.kb_total) continue;  // an empty last range
      const double c = pair_makespan(cand, pairs);
      if (c < 0.97 * best) {
        best = c;
        n_static = ns;
        splits = sp;
      }
    }
  }
}

}  // namespace seg
