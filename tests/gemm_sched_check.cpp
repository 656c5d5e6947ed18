// Host check of the CTA-pair GEMM's schedule: for a list of shapes, every k-block of every tile is covered exactly once,
// every tile has exactly one owning item, the running sum an item reads was written by the item of the range before it, which has a lower index (so the
// pair that holds it reaches it no later than the reader reaches its own item), and slots are unique and inside the workspace.  Prints "ok <cases>" or the first violation.
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <set>
#include <vector>

#include "gemm_pair_sched.h"

using namespace seg;

static int check(int M, int N, int K, int batch, int symmetric, int sm_pairs, bool allow) {
  int n_static, splits;
  pair_choose_split(M, N, K, batch, symmetric, sm_pairs, allow, n_static, splits);
  const PairSched s = make_pair_sched(M, N, K, batch, symmetric, n_static, splits);
  if (!allow && splits != 1) { std::printf("split although not allowed\n"); return 1; }
  if ((long long)(s.splits - 1) * s.rem_tiles > kPairMaxSlots) { std::printf("too many slots\n"); return 1; }
  std::vector<std::vector<int>> cover(s.total, std::vector<int>(s.kb_total, 0));
  std::vector<int> owners(s.total, 0);
  std::set<int> slots;
  for (int i = 0; i < s.n_items; ++i) {
    const PairItem it = pair_item(s, i);
    if (it.t < 0 || it.t >= s.total || it.kb0 < 0 || it.kb1 > s.kb_total || it.kb0 >= it.kb1) { std::printf("M %d N %d K %d splits %d: bad item %d (kb %d..%d)\n", M, N, K, splits, i, it.kb0, it.kb1); return 1; }
    if (it.m < 0 || it.m >= s.m_tiles || it.n < 0 || it.n > s.n_full || it.b < 0 || it.b >= batch) { std::printf("bad coords\n"); return 1; }
    if (symmetric && it.n < it.m) { std::printf("tile below the diagonal scheduled\n"); return 1; }
    if (it.nt % 32 != 0 || it.nt < 32 || it.nt > 256) { std::printf("bad width %d\n", it.nt); return 1; }
    for (int k = it.kb0; k < it.kb1; ++k) cover[it.t][k]++;
    if (it.ks > 0) {  // the running sum this item reads was written by the item of the range before it
      const int writer = s.n_static + (it.ks - 1) * s.rem_tiles + (it.t - s.n_static);
      if (writer >= i) { std::printf("running sum written by a later item\n"); return 1; }
      const PairItem w = pair_item(s, writer);
      if (w.t != it.t || w.ks != it.ks - 1 || pair_item_owns(s, w) || w.kb1 != it.kb0) { std::printf("running-sum chain broken\n"); return 1; }
    }
    if (pair_item_owns(s, it)) {
      owners[it.t]++;
    } else {
      const int slot = pair_slot(s, it.ks, it.t);
      if (slot < 0 || slot >= kPairMaxSlots || !slots.insert(slot).second) { std::printf("slot %d reused or out of range\n", slot); return 1; }
    }
  }
  for (int t = 0; t < s.total; ++t) {
    if (owners[t] != 1) { std::printf("tile %d has %d owners\n", t, owners[t]); return 1; }
    for (int k = 0; k < s.kb_total; ++k)
      if (cover[t][k] != 1) { std::printf("M %d N %d K %d b %d sym %d: tile %d k-block %d covered %d times\n", M, N, K, batch, symmetric, t, k, cover[t][k]); return 1; }
  }
  if (symmetric) {  // exactly the tiles with n >= m
    const int nc = (N + 255) / 256, mt = (M + 255) / 256;
    int want = 0;
    for (int m = 0; m < mt; ++m) want += nc - m;
    if (s.total != batch * want) { std::printf("symmetric tile count %d, expected %d\n", s.total, batch * want); return 1; }
  }
  // every tile position appears once
  std::set<long long> seen;
  for (int t = 0; t < s.total; ++t) {
    PairItem c;
    pair_tile_coords(s, t, c);
    if (!seen.insert(((long long)c.b << 40) | ((long long)c.m << 20) | c.n).second) { std::printf("tile listed twice\n"); return 1; }
    if ((c.n < s.n_full) != (c.nt == 256) && s.tail_nt != 256) { std::printf("width of tile\n"); return 1; }
  }
  return 0;
}

int main(int argc, char** argv) {
  if (argc == 5) {  // report the choice for one shape: M N K batch
    int ns, sp;
    const int M = std::atoi(argv[1]), N = std::atoi(argv[2]), K = std::atoi(argv[3]), b = std::atoi(argv[4]);
    pair_choose_split(M, N, K, b, 0, 74, true, ns, sp);
    const PairSched s = make_pair_sched(M, N, K, b, 0, ns, sp), w = make_pair_sched(M, N, K, b, 0, 0, 1);
    std::printf("tiles %d n_static %d splits %d makespan %.1f (whole tiles %.1f)\n", s.total, s.n_static, s.splits, pair_makespan(s, 74), pair_makespan(w, 74));
    return 0;
  }
  const int shapes[][3] = {{32768, 1944, 1152}, {32768, 1152, 1152}, {32768, 6144, 1152}, {32768, 1152, 3072}, {1944, 1152, 32768},
                           {1152, 1152, 32768}, {6144, 1152, 32768}, {1152, 3072, 32768}, {8192, 49152, 1152}, {128, 128, 64},
                           {24, 40, 64}, {300, 1944, 200}, {1300, 776, 1152}, {18, 1152, 32768}, {256, 256, 262144}, {200, 72, 1024},
                           {4096, 256, 128}, {1, 8, 8}, {2048, 2048, 2048}, {777, 999, 4097}, {49152, 1152, 8192}};
  int cases = 0;
  for (auto& sh : shapes)
    for (int batch : {1, 3, 30})
      for (int pairs : {74, 66, 8, 1})
        for (int allow : {1, 0}) {
          if ((long long)sh[0] * sh[1] * batch > (1LL << 31)) continue;
          if (check(sh[0], sh[1], sh[2], batch, 0, pairs, allow != 0)) return 1;
          ++cases;
        }
  for (int n : {256, 384, 1152, 3072, 640, 72})
    for (int k : {1152, 3072, 6144, 64})
      for (int batch : {1, 30})
        for (int allow : {1, 0}) {
          if (check(n, n, k, batch, 1, 74, allow != 0)) return 1;
          ++cases;
        }
  std::printf("ok %d\n", cases);
  return 0;
}
