// Schedule of the CTA-pair GEMM (gemm_pair.cu): plain C++ that compiles for the host and the device, so the same
// functions place the work in the kernel, size the grid on the host and can be checked exhaustively on a CPU.
//
// Tiles are 256 rows x (256 | last-column remainder) columns.  Order: all full-width tiles (column index fastest, then row
// tile, then batch), then the narrower last-column tiles; a symmetric output lists only tiles on or above the diagonal.
// Work items are dealt round-robin to the pairs, so that the pairs running at the same time work on neighbouring tiles
// and walk the contraction in step - operand panels shared between tiles are then fetched from HBM once and served from
// L2 to the others.  The first n_static tiles are whole-tile items.  The remaining R tiles (the last, partly filled wave,
// or everything when there are fewer tiles than pairs) are cut into `splits` ranges of the contraction, range index
// outermost: items of ranges 0 .. splits-2 leave their raw fp32 accumulator in a workspace slot, the item of the last
// range owns the tile, adds the parts in range order (deterministic) and runs the epilogue.  An owner's parts always
// belong to items with a lower index, which their pairs reach no later than the owner reaches its own.
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
  int full_per_batch, tail_per_batch, full_count, total;
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
  s.full_per_batch = symmetric ? s.n_full * (s.n_full + 1) / 2 : s.m_tiles * s.n_full;
  s.tail_per_batch = rem > 0 ? s.m_tiles : 0;
  s.full_count = batch * s.full_per_batch;
  s.total = s.full_count + batch * s.tail_per_batch;
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
  if (t < s.full_count) {
    c.b = t / s.full_per_batch;
    int idx = t - c.b * s.full_per_batch;
    if (s.symmetric) {  // rows of the upper triangle: row m holds tiles n = m .. n_full - 1
      int m = 0, row = s.n_full;
      while (idx >= row) {
        idx -= row;
        --row;
        ++m;
      }
      c.m = m;
      c.n = m + idx;
    } else {
      c.m = idx / s.n_full;
      c.n = idx - c.m * s.n_full;
    }
    c.nt = kPairN;
  } else {
    const int idx = t - s.full_count;
    c.b = idx / s.tail_per_batch;
    c.m = idx - c.b * s.tail_per_batch;
    c.n = s.n_full;
    c.nt = s.tail_nt;
  }
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
// k-blocks scaled by its width plus a fixed overhead (pipeline fill, accumulator hand-over, epilogue); an owner pays for
// reading the parts.  Items come in at most four runs of equal cost (static full, static narrow, then per range: split
// full, split narrow), which round-robin spreads evenly, so the load of a pair follows from counting.
struct PairRun {
  long long count;
  double cost;
};
inline double pair_makespan(const PairSched& s, int pairs) {
  const double kItemOverhead = 5.0, kPartRead = 3.0;
  const double wt = s.tail_nt / 256.0;
  PairRun runs[2 + 2 * kPairMaxSplits];
  int n = 0;
  const long long sf = s.n_static < s.full_count ? s.n_static : s.full_count;  // static full-width tiles
  const long long st = s.n_static - sf;                                         // static narrow tiles
  if (sf > 0) runs[n++] = {sf, s.kb_total + kItemOverhead};
  if (st > 0) runs[n++] = {st, wt * s.kb_total + kItemOverhead};
  const long long rf = s.full_count - sf, rt = s.rem_tiles - rf;  // split tiles of either width
  for (int ks = 0; ks < s.splits && s.rem_tiles > 0; ++ks) {
    const int kb0 = ks * s.kb_per, kb1 = kb0 + s.kb_per < s.kb_total ? kb0 + s.kb_per : s.kb_total;
    const double extra = kItemOverhead + (ks == s.splits - 1 ? kPartRead * (s.splits - 1) : 1.0);
    if (rf > 0) runs[n++] = {rf, (double)(kb1 - kb0) + extra};
    if (rt > 0) runs[n++] = {rt, wt * (kb1 - kb0) + extra};
  }
  const int P = s.n_items < pairs ? s.n_items : pairs;
  if (P <= 0) return 0.0;
  // load of pair p = sum over runs of (items of the run that land on p) * cost; evaluate at the breakpoints only
  double best = 0.0;
  long long start = 0;
  long long marks[2 * (2 + 2 * kPairMaxSplits) + 1];
  int nm = 0;
  marks[nm++] = 0;
  for (int r = 0; r < n; ++r) {
    marks[nm++] = start % P;
    start += runs[r].count;
    marks[nm++] = start % P;
  }
  for (int mi = 0; mi < nm; ++mi) {
    const long long p = marks[mi];
    double load = 0.0;
    long long s0 = 0;
    for (int r = 0; r < n; ++r) {
      // items s0 .. s0 + count - 1 go to pairs (index % P): how many land on p
      const long long first = s0 + ((p - s0 % P) + P) % P;
      if (first < s0 + runs[r].count) load += (double)((s0 + runs[r].count - 1 - first) / P + 1) * runs[r].cost;
      s0 += runs[r].count;
    }
    best = load > best ? load : best;
  }
  return best;
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
