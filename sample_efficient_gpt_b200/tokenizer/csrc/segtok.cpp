// Native tokenizer tools (C++17 + pybind11): a pre-tokenisation splitter/counter and an incremental BPE trainer.
//
// Splitter  - counterpart of the reference's Rust `fastsplit` crate (fastsplit/src/lib.rs:14-116): split text on one
//             special token, cut every piece into pre-tokens with the GPT-4 style pattern
//               (?i:'s|'t|'re|'ve|'m|'ll|'d) | [^\r\n\p{L}\p{N}]?\p{L}+ | \p{N}{1,3} | ?[^\s\p{L}\p{N}]+[\r\n]* |
//               \s*[\r\n]+ | \s+(?!\S) | \s+
//             and count them.  The pattern is implemented as a hand-written scanner over UTF-8 (no regex engine):
//             each alternative is tried in order at the current position, with the backtracking behaviour of the two
//             whitespace alternatives written out.  Invalid UTF-8 is replaced by U+FFFD per maximal ill-formed
//             subsequence.  The GIL is released while scanning.
// BpeTrainer - counterpart of the Rust `rustbpe` crate (rustbpe/src/lib.rs:96-318): words = unique pre-token byte
//             strings with counts, pair counts with a max-heap and lazy refresh of stale entries, merges recorded in
//             order.  Ties between equally frequent pairs go to the pair whose (left bytes, right bytes) tuple is
//             largest, which is the rule of the Python trainer (tokenizer/train_bpe.py:54-74).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <cstdint>
#include <cstdio>
#include <queue>
#include <stdexcept>
#include <string>
#include <string_view>
#include <thread>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "unicode_tables.h"

namespace py = pybind11;

namespace {

// ------------------------------------------------------------------------------------------------ unicode classes
bool in_ranges(const CpRange* r, int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < r[mid].lo) hi = mid - 1;
    else if (cp > r[mid].hi) lo = mid + 1;
    else return true;
  }
  return false;
}

enum : uint8_t { kLetter = 1, kNumber = 2, kSpace = 4 };

struct AsciiClass {
  uint8_t t[128];
  AsciiClass() {
    for (uint32_t c = 0; c < 128; ++c) {
      t[c] = (in_ranges(kLetterRanges, kLetterRanges_count, c) ? kLetter : 0) |
             (in_ranges(kNumberRanges, kNumberRanges_count, c) ? kNumber : 0) |
             (in_ranges(kSpaceRanges, kSpaceRanges_count, c) ? kSpace : 0);
    }
  }
};
const AsciiClass kAscii;

inline uint8_t classify(uint32_t cp) {
  if (cp < 128) return kAscii.t[cp];
  if (in_ranges(kLetterRanges, kLetterRanges_count, cp)) return kLetter;
  if (in_ranges(kNumberRanges, kNumberRanges_count, cp)) return kNumber;
  if (in_ranges(kSpaceRanges, kSpaceRanges_count, cp)) return kSpace;
  return 0;
}

// Decode one code point of valid UTF-8 at s[i]; *len receives its byte length.
inline uint32_t decode(const uint8_t* s, size_t i, size_t n, int* len) {
  const uint8_t b = s[i];
  if (b < 0x80) { *len = 1; return b; }
  if (b < 0xE0 && i + 1 < n) { *len = 2; return ((b & 0x1Fu) << 6) | (s[i + 1] & 0x3Fu); }
  if (b < 0xF0 && i + 2 < n) { *len = 3; return ((b & 0x0Fu) << 12) | ((s[i + 1] & 0x3Fu) << 6) | (s[i + 2] & 0x3Fu); }
  if (i + 3 < n) {
    *len = 4;
    return ((b & 0x07u) << 18) | ((s[i + 1] & 0x3Fu) << 12) | ((s[i + 2] & 0x3Fu) << 6) | (s[i + 3] & 0x3Fu);
  }
  *len = 1;
  return 0xFFFD;
}

// Valid UTF-8 copy of the input: every maximal ill-formed subsequence becomes U+FFFD.
std::string sanitize_utf8(const uint8_t* s, size_t n) {
  std::string out;
  out.reserve(n);
  size_t i = 0;
  auto bad = [&]() { out += "\xEF\xBF\xBD"; };
  while (i < n) {
    const uint8_t b = s[i];
    if (b < 0x80) { out.push_back((char)b); ++i; continue; }
    int need;
    uint8_t lo = 0x80, hi = 0xBF;
    if (b >= 0xC2 && b <= 0xDF) need = 1;
    else if (b == 0xE0) { need = 2; lo = 0xA0; }
    else if ((b >= 0xE1 && b <= 0xEC) || b == 0xEE || b == 0xEF) need = 2;
    else if (b == 0xED) { need = 2; hi = 0x9F; }
    else if (b == 0xF0) { need = 3; lo = 0x90; }
    else if (b >= 0xF1 && b <= 0xF3) need = 3;
    else if (b == 0xF4) { need = 3; hi = 0x8F; }
    else { bad(); ++i; continue; }
    size_t j = i + 1;
    int got = 0;
    while (got < need && j < n) {
      const uint8_t c = s[j];
      const uint8_t l = (got == 0) ? lo : 0x80, h = (got == 0) ? hi : 0xBF;
      if (c < l || c > h) break;
      ++j;
      ++got;
    }
    if (got == need) out.append((const char*)s + i, j - i);
    else bad();
    i = j;
  }
  return out;
}

bool is_valid_utf8(const uint8_t* s, size_t n) {
  size_t i = 0;
  while (i < n) {
    const uint8_t b = s[i];
    if (b < 0x80) { ++i; continue; }
    int need;
    uint8_t lo = 0x80, hi = 0xBF;
    if (b >= 0xC2 && b <= 0xDF) need = 1;
    else if (b == 0xE0) { need = 2; lo = 0xA0; }
    else if ((b >= 0xE1 && b <= 0xEC) || b == 0xEE || b == 0xEF) need = 2;
    else if (b == 0xED) { need = 2; hi = 0x9F; }
    else if (b == 0xF0) { need = 3; lo = 0x90; }
    else if (b >= 0xF1 && b <= 0xF3) need = 3;
    else if (b == 0xF4) { need = 3; hi = 0x8F; }
    else return false;
    for (int k = 1; k <= need; ++k) {
      if (i + k >= n) return false;
      const uint8_t c = s[i + k];
      const uint8_t l = (k == 1) ? lo : 0x80, h = (k == 1) ? hi : 0xBF;
      if (c < l || c > h) return false;
    }
    i += need + 1;
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ the scanner
inline bool is_newline(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// Case-insensitive match of an ASCII letter, including the Unicode simple case folds that land on it
// (U+017F LATIN SMALL LETTER LONG S folds to 's', U+212A KELVIN SIGN folds to 'k').
inline bool ci_eq(uint32_t cp, char lower) {
  if (cp == (uint32_t)lower || cp == (uint32_t)(lower - 32)) return true;
  return lower == 's' && cp == 0x17F;
}

// End (exclusive) of the pre-token that starts at byte i of s[0..n); always > i.
size_t match_at(const uint8_t* s, size_t i, size_t n) {
  int l0;
  const uint32_t c0 = decode(s, i, n, &l0);
  // 1. contractions
  if (c0 == '\'' && i + 1 < n) {
    int l1;
    const uint32_t c1 = decode(s, i + 1, n, &l1);
    if (ci_eq(c1, 's') || ci_eq(c1, 't') || ci_eq(c1, 'm') || ci_eq(c1, 'd')) return i + 1 + l1;
    if (i + 1 + l1 < n) {
      int l2;
      const uint32_t c2 = decode(s, i + 1 + l1, n, &l2);
      if ((ci_eq(c1, 'r') && ci_eq(c2, 'e')) || (ci_eq(c1, 'v') && ci_eq(c2, 'e')) || (ci_eq(c1, 'l') && ci_eq(c2, 'l')))
        return i + 1 + l1 + l2;
    }
  }
  const uint8_t k0 = classify(c0);
  // 2. optional single non-letter/number/newline character, then letters
  {
    size_t p = i;
    bool ok = false;
    if (k0 & kLetter) ok = true;
    else if (!(k0 & kNumber) && !is_newline(c0) && i + l0 < n) {
      int l1;
      const uint32_t c1 = decode(s, i + l0, n, &l1);
      if (classify(c1) & kLetter) { ok = true; p = i + l0; }
    }
    if (ok) {
      while (p < n) {
        int l;
        const uint32_t c = decode(s, p, n, &l);
        if (!(classify(c) & kLetter)) break;
        p += l;
      }
      return p;
    }
  }
  // 3. one to three numbers
  if (k0 & kNumber) {
    size_t p = i + l0;
    for (int cnt = 1; cnt < 3 && p < n; ++cnt) {
      int l;
      const uint32_t c = decode(s, p, n, &l);
      if (!(classify(c) & kNumber)) break;
      p += l;
    }
    return p;
  }
  // 4. optional space, run of other characters, trailing newlines
  {
    size_t p = i;
    bool ok = false;
    if (k0 == 0) ok = true;
    else if (c0 == ' ' && i + 1 < n) {
      int l1;
      const uint32_t c1 = decode(s, i + 1, n, &l1);
      if (classify(c1) == 0) { ok = true; p = i + 1; }
    }
    if (ok) {
      while (p < n) {
        int l;
        const uint32_t c = decode(s, p, n, &l);
        if (classify(c) != 0) break;
        p += l;
      }
      while (p < n && (s[p] == '\r' || s[p] == '\n')) ++p;
      return p;
    }
  }
  // 5-7. white space: measure the run once
  size_t p = i, last_nl_end = 0, last_char_start = i;
  int chars = 0;
  while (p < n) {
    int l;
    const uint32_t c = decode(s, p, n, &l);
    if (!(classify(c) & kSpace)) break;
    last_char_start = p;
    p += l;
    ++chars;
    if (is_newline(c)) last_nl_end = p;
  }
  if (chars == 0) return i + l0;      // unreachable for classified input; keeps the scanner total
  if (last_nl_end != 0) return last_nl_end;  // \s*[\r\n]+ : up to the last newline of the run
  if (p == n) return p;                      // \s+(?!\S) at the end of the piece
  if (chars >= 2) return last_char_start;    // \s+(?!\S) : all but the last white-space character
  return p;                                  // \s+
}

using Counts = std::unordered_map<std::string, uint64_t>;

void count_piece(const uint8_t* s, size_t n, Counts& counts) {
  size_t i = 0;
  while (i < n) {
    const size_t j = match_at(s, i, n);
    counts[std::string((const char*)s + i, j - i)] += 1;
    i = j;
  }
}

void pieces_of(const uint8_t* s, size_t n, size_t b, size_t e, std::vector<std::string>& out) {
  size_t i = b;
  (void)n;
  while (i < e) {
    const size_t j = match_at(s + b, i - b, e - b) + b;
    out.emplace_back((const char*)s + i, j - i);
    i = j;
  }
}

class Splitter {
 public:
  explicit Splitter(std::string special) : special_(std::move(special)) {}

  Counts split_counts(const std::string& text) const {
    Counts counts;
    counts.reserve(text.size() / 8 + 16);
    const uint8_t* s = (const uint8_t*)text.data();
    size_t start = 0;
    if (!special_.empty()) {
      size_t pos;
      while ((pos = text.find(special_, start)) != std::string::npos) {
        if (pos > start) count_piece(s + start, pos - start, counts);
        start = pos + special_.size();
      }
    }
    if (start < text.size()) count_piece(s + start, text.size() - start, counts);
    return counts;
  }

  // text given as bytes (decoded leniently) or str
  py::dict split(py::object chunk) const {
    std::string text;
    if (py::isinstance<py::bytes>(chunk)) {
      std::string raw = chunk.cast<std::string>();
      text = is_valid_utf8((const uint8_t*)raw.data(), raw.size()) ? std::move(raw) : sanitize_utf8((const uint8_t*)raw.data(), raw.size());
    } else if (py::isinstance<py::str>(chunk)) {
      text = chunk.cast<std::string>();
    } else {
      throw py::type_error("Expected bytes or str");
    }
    Counts counts;
    {
      py::gil_scoped_release nogil;
      counts = split_counts(text);
    }
    return to_dict(counts);
  }

  py::dict seek_and_split(const std::string& path, uint64_t start, uint64_t end) const {
    if (end < start) throw py::value_error("end < start");
    Counts counts;
    std::string err;
    {
      py::gil_scoped_release nogil;
      FILE* f = std::fopen(path.c_str(), "rb");
      if (!f) err = "cannot open " + path;
      else {
        std::string raw(end - start, '\0');
        if (std::fseek(f, (long)start, SEEK_SET) != 0 || std::fread(raw.data(), 1, raw.size(), f) != raw.size()) err = "short read from " + path;
        std::fclose(f);
        if (err.empty()) {
          const std::string text = is_valid_utf8((const uint8_t*)raw.data(), raw.size()) ? std::move(raw)
                                                                                         : sanitize_utf8((const uint8_t*)raw.data(), raw.size());
          counts = split_counts(text);
        }
      }
    }
    if (!err.empty()) throw std::runtime_error(err);
    return to_dict(counts);
  }

  // Pre-token counts of a whole file on `threads` native threads: the file is mapped, cut at document separators into
  // about four pieces per thread, the pieces are counted in parallel (work taken from a shared counter) and the per-thread
  // tables are merged before a single conversion to a dict - no Python work and no GIL between the pieces.
  py::dict count_file(const std::string& path, int threads) const {
    Counts total;
    std::string err;
    {
      py::gil_scoped_release nogil;
      const int fd = ::open(path.c_str(), O_RDONLY);
      if (fd < 0) err = "cannot open " + path;
      struct stat st {};
      if (err.empty() && ::fstat(fd, &st) != 0) err = "cannot stat " + path;
      const size_t n = err.empty() ? (size_t)st.st_size : 0;
      const uint8_t* base = nullptr;
      if (err.empty() && n > 0) {
        void* m = ::mmap(nullptr, n, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m == MAP_FAILED) err = "cannot map " + path;
        else base = (const uint8_t*)m;
      }
      if (fd >= 0) ::close(fd);
      if (err.empty() && n > 0) {
        const unsigned nt = (unsigned)std::max(1, std::min(threads, 64));
        // piece boundaries: the first separator at or after every n / pieces bytes (none: the piece grows)
        std::vector<size_t> cuts{0};
        const size_t pieces = (size_t)nt * 4;
        if (!special_.empty()) {
          for (size_t i = 1; i < pieces; ++i) {
            size_t from = std::max(n / pieces * i, cuts.back());
            if (from >= n) break;
            const void* hit = ::memmem(base + from, n - from, special_.data(), special_.size());
            if (hit == nullptr) break;
            const size_t pos = (const uint8_t*)hit - base;
            if (pos > cuts.back()) cuts.push_back(pos);
          }
        }
        cuts.push_back(n);
        std::vector<Counts> part(nt);
        std::atomic<size_t> next{0};
        auto work = [&](unsigned t) {
          for (size_t i = next.fetch_add(1); i + 1 < cuts.size(); i = next.fetch_add(1)) {
            const uint8_t* b = base + cuts[i];
            const size_t len = cuts[i + 1] - cuts[i];
            const std::string text = is_valid_utf8(b, len) ? std::string((const char*)b, len) : sanitize_utf8(b, len);
            for (auto& kv : split_counts(text)) part[t][kv.first] += kv.second;
          }
        };
        std::vector<std::thread> th;
        for (unsigned t = 1; t < nt; ++t) th.emplace_back(work, t);
        work(0);
        for (auto& x : th) x.join();
        total = std::move(part[0]);
        for (unsigned t = 1; t < nt; ++t)
          for (auto& kv : part[t]) total[kv.first] += kv.second;
        ::munmap((void*)base, n);
      }
    }
    if (!err.empty()) throw std::runtime_error(err);
    return to_dict(total);
  }

  // ordered pre-tokens of a str (used by encoders and tests)
  std::vector<std::string> pretokens(const std::string& text) const {
    std::vector<std::string> out;
    const uint8_t* s = (const uint8_t*)text.data();
    size_t start = 0;
    if (!special_.empty()) {
      size_t pos;
      while ((pos = text.find(special_, start)) != std::string::npos) {
        if (pos > start) pieces_of(s, text.size(), start, pos, out);
        start = pos + special_.size();
      }
    }
    if (start < text.size()) pieces_of(s, text.size(), start, text.size(), out);
    return out;
  }

 private:
  static py::dict to_dict(const Counts& counts) {
    py::dict d;
    for (const auto& kv : counts) d[py::str(kv.first)] = kv.second;
    return d;
  }
  std::string special_;
};

// ------------------------------------------------------------------------------------------------ BPE trainer
using Pair = uint64_t;
inline Pair mk(uint32_t a, uint32_t b) { return ((uint64_t)a << 32) | b; }
inline uint32_t left_of(Pair p) { return (uint32_t)(p >> 32); }
inline uint32_t right_of(Pair p) { return (uint32_t)p; }

struct PairHash {
  size_t operator()(Pair p) const noexcept {
    uint64_t x = p * 0x9E3779B97F4A7C15ull;
    return (size_t)(x ^ (x >> 29));
  }
};

class BpeTrainer {
 public:
  BpeTrainer() { reset(); }

  void train_from_pretokens(const std::vector<std::pair<py::bytes, int64_t>>& pre_tokens, uint32_t target_vocab_no_specials) {
    if (target_vocab_no_specials < 256) throw py::value_error("vocab_size must be at least 256");
    reset();
    std::vector<std::vector<uint32_t>> words;
    std::vector<int64_t> counts;
    words.reserve(pre_tokens.size());
    for (const auto& pc : pre_tokens) {
      const std::string b = pc.first;
      std::vector<uint32_t> ids(b.size());
      for (size_t i = 0; i < b.size(); ++i) ids[i] = (uint8_t)b[i];
      words.push_back(std::move(ids));
      counts.push_back(pc.second);
    }
    py::gil_scoped_release nogil;
    train_core(words, counts, target_vocab_no_specials - 256);
  }

  std::vector<std::pair<py::bytes, py::bytes>> export_merges_bytes() const {
    std::vector<std::pair<py::bytes, py::bytes>> out;
    for (const auto& m : merges_order_) out.emplace_back(py::bytes(token_bytes_[m.first]), py::bytes(token_bytes_[m.second]));
    return out;
  }
  std::vector<std::pair<uint32_t, py::bytes>> export_vocab_bytes() const {
    std::vector<std::pair<uint32_t, py::bytes>> out;
    for (uint32_t i = 0; i < token_bytes_.size(); ++i) out.emplace_back(i, py::bytes(token_bytes_[i]));
    return out;
  }
  std::vector<std::pair<py::bytes, uint32_t>> get_mergeable_ranks() const {
    std::vector<std::pair<py::bytes, uint32_t>> out;
    for (uint32_t i = 0; i < token_bytes_.size(); ++i) out.emplace_back(py::bytes(token_bytes_[i]), i);
    return out;
  }
  std::string get_pattern() const {
    return "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}{1,3}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+";
  }

  // lowest-rank-first merging of each pre-token of `text`
  std::vector<uint32_t> encode(const std::string& text) const {
    std::vector<uint32_t> all;
    Splitter sp("");
    for (const std::string& piece : sp.pretokens(text)) {
      std::vector<uint32_t> ids(piece.size());
      for (size_t i = 0; i < piece.size(); ++i) ids[i] = (uint8_t)piece[i];
      while (ids.size() >= 2) {
        uint32_t best_id = UINT32_MAX;
        size_t best_i = 0;
        for (size_t i = 0; i + 1 < ids.size(); ++i) {
          auto it = merges_.find(mk(ids[i], ids[i + 1]));
          if (it != merges_.end() && it->second < best_id) { best_id = it->second; best_i = i; }
        }
        if (best_id == UINT32_MAX) break;
        ids[best_i] = best_id;
        ids.erase(ids.begin() + best_i + 1);
      }
      all.insert(all.end(), ids.begin(), ids.end());
    }
    return all;
  }

 private:
  struct Job {
    int64_t count;
    Pair pair;
  };

  void reset() {
    merges_.clear();
    merges_order_.clear();
    token_bytes_.clear();
    for (int b = 0; b < 256; ++b) token_bytes_.push_back(std::string(1, (char)b));
  }

  // heap order: higher count first; ties: larger (left bytes, right bytes) first
  bool job_less(const Job& a, const Job& b) const {
    if (a.count != b.count) return a.count < b.count;
    const std::string& al = token_bytes_[left_of(a.pair)];
    const std::string& bl = token_bytes_[left_of(b.pair)];
    if (al != bl) return al < bl;
    return token_bytes_[right_of(a.pair)] < token_bytes_[right_of(b.pair)];
  }

  void train_core(std::vector<std::vector<uint32_t>>& words, const std::vector<int64_t>& counts, uint32_t num_merges) {
    using CountMap = std::unordered_map<Pair, int64_t, PairHash>;
    using WhereMap = std::unordered_map<Pair, std::vector<uint32_t>, PairHash>;
    CountMap pair_counts;
    WhereMap where;
    // initial counts: one local map per thread, merged afterwards
    const unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 16u));
    std::vector<CountMap> lc(nt);
    std::vector<WhereMap> lw(nt);
    std::vector<std::thread> th;
    const size_t W = words.size();
    for (unsigned t = 0; t < nt; ++t) {
      th.emplace_back([&, t]() {
        const size_t b = W * t / nt, e = W * (t + 1) / nt;
        for (size_t i = b; i < e; ++i) {
          const auto& ids = words[i];
          if (ids.size() < 2 || counts[i] == 0) continue;
          for (size_t k = 0; k + 1 < ids.size(); ++k) {
            const Pair p = mk(ids[k], ids[k + 1]);
            lc[t][p] += counts[i];
            auto& v = lw[t][p];
            if (v.empty() || v.back() != (uint32_t)i) v.push_back((uint32_t)i);
          }
        }
      });
    }
    for (auto& x : th) x.join();
    for (unsigned t = 0; t < nt; ++t) {
      for (auto& kv : lc[t]) pair_counts[kv.first] += kv.second;
      for (auto& kv : lw[t]) {
        auto& dst = where[kv.first];
        dst.insert(dst.end(), kv.second.begin(), kv.second.end());
      }
    }
    auto cmp = [this](const Job& a, const Job& b) { return job_less(a, b); };
    std::priority_queue<Job, std::vector<Job>, decltype(cmp)> heap(cmp);
    for (const auto& kv : pair_counts)
      if (kv.second > 0) heap.push(Job{kv.second, kv.first});

    uint32_t done = 0;
    std::vector<std::pair<Pair, int64_t>> deltas;
    while (done < num_merges && !heap.empty()) {
      Job top = heap.top();
      heap.pop();
      auto itc = pair_counts.find(top.pair);
      const int64_t current = itc == pair_counts.end() ? 0 : itc->second;
      if (top.count != current) {  // stale entry: refresh lazily
        if (current > 0) heap.push(Job{current, top.pair});
        continue;
      }
      if (current <= 0) break;
      const uint32_t a = left_of(top.pair), b = right_of(top.pair);
      const uint32_t new_id = (uint32_t)token_bytes_.size();
      token_bytes_.push_back(token_bytes_[a] + token_bytes_[b]);
      merges_[top.pair] = new_id;
      merges_order_.emplace_back(a, b);
      std::vector<uint32_t> touched;
      touched.swap(where[top.pair]);
      std::vector<Pair> created;
      for (uint32_t wi : touched) {
        auto& ids = words[wi];
        const size_t n = ids.size();
        if (n < 2) continue;
        std::vector<uint32_t> out;
        out.reserve(n);
        deltas.clear();
        size_t i = 0;
        while (i < n) {
          if (i + 1 < n && ids[i] == a && ids[i + 1] == b) {
            if (!out.empty()) {
              deltas.emplace_back(mk(out.back(), a), -1);
              deltas.emplace_back(mk(out.back(), new_id), +1);
            }
            deltas.emplace_back(top.pair, -1);
            if (i + 2 < n) {
              deltas.emplace_back(mk(b, ids[i + 2]), -1);
              deltas.emplace_back(mk(new_id, ids[i + 2]), +1);
            }
            out.push_back(new_id);
            i += 2;
          } else {
            out.push_back(ids[i]);
            i += 1;
          }
        }
        ids.swap(out);
        for (const auto& d : deltas) {
          const int64_t tot = d.second * counts[wi];
          if (tot == 0) continue;
          pair_counts[d.first] += tot;
          if (d.second > 0) {
            auto& v = where[d.first];
            if (v.empty() || v.back() != wi) v.push_back(wi);
            created.push_back(d.first);
          }
        }
      }
      std::sort(created.begin(), created.end());
      created.erase(std::unique(created.begin(), created.end()), created.end());
      for (Pair p : created) {
        const int64_t c = pair_counts[p];
        if (c > 0) heap.push(Job{c, p});
      }
      ++done;
    }
  }

  std::unordered_map<Pair, uint32_t, PairHash> merges_;
  std::vector<std::pair<uint32_t, uint32_t>> merges_order_;
  std::vector<std::string> token_bytes_;
};

// ------------------------------------------------------------------------------------------------ BPE encoder
// Encodes text with a given vocabulary: byte -> id table, merges as (left id, right id, new id, rank).  A pre-token is
// merged lowest-rank-first, every occurrence of the chosen pair left to right per round (the statement of
// tokenizer/tokenizer.py:104-351 of the reference); an optional second stage of merges runs over the whole piece, across
// pre-token boundaries.  Pieces must not contain special tokens (the caller splits on them).
class Encoder {
 public:
  using Merge = std::tuple<uint32_t, uint32_t, uint32_t, uint32_t>;
  Encoder(std::vector<uint32_t> lut256, const std::vector<Merge>& first, const std::vector<Merge>& second) : lut_(std::move(lut256)) {
    if (lut_.size() != 256) throw py::value_error("the byte table needs 256 entries");
    for (const auto& m : first) first_[mk(std::get<0>(m), std::get<1>(m))] = {std::get<3>(m), std::get<2>(m)};
    for (const auto& m : second) second_[mk(std::get<0>(m), std::get<1>(m))] = {std::get<3>(m), std::get<2>(m)};
  }

  // Holds the GIL: the instance's pre-token cache is shared by all callers.
  std::vector<uint32_t> encode_ordinary(const std::string& text) { return encode_with(text, cache_); }

  // Many pieces at once on native threads; every thread keeps its own pre-token cache.
  std::vector<std::vector<uint32_t>> encode_batch(const std::vector<std::string>& texts, int threads) const {
    std::vector<std::vector<uint32_t>> out(texts.size());
    py::gil_scoped_release nogil;
    const unsigned nt = (unsigned)std::max(1, std::min<int>(threads, 64));
    std::atomic<size_t> next{0};
    auto work = [&]() {
      Cache cache;
      for (size_t i = next.fetch_add(1); i < texts.size(); i = next.fetch_add(1)) out[i] = encode_with(texts[i], cache);
    };
    std::vector<std::thread> th;
    for (unsigned t = 1; t < nt; ++t) th.emplace_back(work);
    work();
    for (auto& x : th) x.join();
    return out;
  }

 private:
  struct RankId {
    uint32_t rank, id;
  };
  using Table = std::unordered_map<Pair, RankId, PairHash>;
  using Cache = std::unordered_map<std::string, std::vector<uint32_t>>;

  static void merge_by_rank(std::vector<uint32_t>& ids, const Table& table) {
    std::vector<uint32_t> out;
    while (ids.size() >= 2) {
      uint32_t best = UINT32_MAX, new_id = 0;
      Pair best_pair = 0;
      for (size_t i = 0; i + 1 < ids.size(); ++i) {
        const auto it = table.find(mk(ids[i], ids[i + 1]));
        if (it != table.end() && it->second.rank < best) {
          best = it->second.rank;
          new_id = it->second.id;
          best_pair = it->first;
        }
      }
      if (best == UINT32_MAX) break;
      out.clear();
      for (size_t i = 0; i < ids.size();) {
        if (i + 1 < ids.size() && mk(ids[i], ids[i + 1]) == best_pair) {
          out.push_back(new_id);
          i += 2;
        } else {
          out.push_back(ids[i]);
          i += 1;
        }
      }
      ids.swap(out);
    }
  }

  std::vector<uint32_t> encode_with(const std::string& text, Cache& cache) const {
    std::vector<uint32_t> all;
    const uint8_t* s = (const uint8_t*)text.data();
    const size_t n = text.size();
    size_t i = 0;
    std::string key;
    while (i < n) {
      const size_t j = match_at(s, i, n);
      key.assign((const char*)s + i, j - i);
      auto it = cache.find(key);
      if (it == cache.end()) {
        std::vector<uint32_t> ids(key.size());
        for (size_t k = 0; k < key.size(); ++k) ids[k] = lut_[(uint8_t)key[k]];
        merge_by_rank(ids, first_);
        if (cache.size() >= (size_t)2000000) cache.clear();
        it = cache.emplace(key, std::move(ids)).first;
      }
      all.insert(all.end(), it->second.begin(), it->second.end());
      i = j;
    }
    if (!second_.empty()) merge_by_rank(all, second_);
    return all;
  }

  std::vector<uint32_t> lut_;
  Table first_, second_;
  Cache cache_;
};

}  // namespace

PYBIND11_MODULE(_segtok, m) {
  m.doc() = "native pre-tokeniser and BPE trainer";
  py::class_<Splitter>(m, "Splitter")
      .def(py::init<std::string>(), py::arg("special_token"))
      .def("split", &Splitter::split, py::arg("chunk"))
      .def("seek_and_split", &Splitter::seek_and_split, py::arg("filepath"), py::arg("start"), py::arg("end"))
      .def("count_file", &Splitter::count_file, py::arg("filepath"), py::arg("threads") = 8)
      .def("pretokens", &Splitter::pretokens, py::arg("text"));
  py::class_<BpeTrainer>(m, "Tokenizer")
      .def(py::init<>())
      .def("train_from_pretokens", &BpeTrainer::train_from_pretokens, py::arg("pre_tokens"), py::arg("target_vocab_no_specials"))
      .def("export_merges_bytes", &BpeTrainer::export_merges_bytes)
      .def("export_vocab_bytes", &BpeTrainer::export_vocab_bytes)
      .def("get_pattern", &BpeTrainer::get_pattern)
      .def("get_mergeable_ranks", &BpeTrainer::get_mergeable_ranks)
      .def("encode", &BpeTrainer::encode, py::arg("text"));
  py::class_<Encoder>(m, "Encoder")
      .def(py::init<std::vector<uint32_t>, const std::vector<Encoder::Merge>&, const std::vector<Encoder::Merge>&>(), py::arg("lut256"),
           py::arg("merges"), py::arg("second_stage") = std::vector<Encoder::Merge>())
      .def("encode_ordinary", &Encoder::encode_ordinary, py::arg("text"))
      .def("encode_batch", &Encoder::encode_batch, py::arg("texts"), py::arg("threads") = 8);
}
