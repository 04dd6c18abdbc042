// BPE trainer: learns merges from chunk frequencies (see text.hpp).  The learned vocabulary is a pure function of the
// chunk counts: the most frequent pair merges first, ties go to the smaller (left id, right id), a merge whose token
// would exceed max_token_bytes is discarded together with its statistics, and training stops at the vocabulary size
// or when the best pair is rarer than min_frequency (tokenizer/bpe_trainer.cpp:90-271 in the reference).
#include <algorithm>
#include <fstream>
#include <queue>

#include "text.hpp"

namespace gbh {

void BpeTrainer::add_chunk_counts(const std::string& chunk, u64 count) {
  if (chunk.empty() || count == 0) return;
  const std::string norm = normalize(cfg_.normalizer, chunk);
  bool any = false;
  for (const Chunk& c : pre_tokenize(norm)) {
    if (c.text.empty()) continue;
    counts_[c.text] += count;
    total_ += count;
    any = true;
  }
  if (!any && !norm.empty()) {
    counts_[norm] += count;
    total_ += count;
  }
}

void BpeTrainer::add_text(const std::string& text) {
  for (const Chunk& c : pre_tokenize(normalize(cfg_.normalizer, text))) {
    if (c.text.empty()) continue;
    ++counts_[c.text];
    ++total_;
  }
}

void BpeTrainer::add_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  GBH_CHECK(f.good(), "cannot open corpus file: " + path);
  std::string line;
  while (std::getline(f, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    add_text(line);
  }
}

namespace {

inline u64 pair_of(i32 a, i32 b) { return (static_cast<u64>(static_cast<u32>(a)) << 32) | static_cast<u32>(b); }

struct PairHash {
  size_t operator()(u64 k) const { return static_cast<size_t>(splitmix64(k)); }
};

struct PairStat {
  i64 count = 0;
  std::vector<u32> words;   // words that contained the pair at some point (may be stale or repeated)
};

struct Best {
  i64 count;
  u64 pair;
};
struct BestOrder {   // max-heap on count; among equal counts the numerically smaller pair comes out first
  bool operator()(const Best& x, const Best& y) const { return x.count != y.count ? x.count < y.count : x.pair > y.pair; }
};

}  // namespace

Tokenizer BpeTrainer::train() {
  GBH_CHECK(!counts_.empty(), "BPE trainer has no data");
  const int reserved = special::COUNT + 256;
  GBH_CHECK(cfg_.vocab_size > reserved + 100, "vocab_size too small");

  std::vector<std::string> vocab = special_token_strings();
  vocab.reserve(static_cast<size_t>(cfg_.vocab_size));
  for (int b = 0; b < 256; ++b) vocab.emplace_back(1, static_cast<char>(b));

  // one symbol sequence per distinct chunk, weighted by its frequency
  std::vector<std::vector<i32>> words;
  std::vector<i64> freq;
  for (const auto& kv : counts_) {
    if (kv.second < static_cast<u64>(cfg_.min_frequency) || kv.first.size() < 2) continue;
    std::vector<i32> w(kv.first.size());
    for (size_t i = 0; i < w.size(); ++i) w[i] = special::COUNT + static_cast<i32>(static_cast<u8>(kv.first[i]));
    words.push_back(std::move(w));
    freq.push_back(static_cast<i64>(kv.second));
  }

  std::unordered_map<u64, PairStat, PairHash> stats;
  stats.reserve(1u << 20);
  for (u32 wi = 0; wi < words.size(); ++wi) {
    const auto& w = words[wi];
    for (size_t i = 0; i + 1 < w.size(); ++i) {
      PairStat& st = stats[pair_of(w[i], w[i + 1])];
      st.count += freq[wi];
      if (st.words.empty() || st.words.back() != wi) st.words.push_back(wi);
    }
  }
  std::priority_queue<Best, std::vector<Best>, BestOrder> heap;
  for (const auto& kv : stats) heap.push(Best{kv.second.count, kv.first});

  std::vector<std::pair<std::string, std::string>> merges;
  const int want = cfg_.vocab_size - reserved;
  int done = 0;
  std::vector<u64> touched;
  std::vector<i32> rebuilt;
  while (done < want && !heap.empty()) {
    const Best top = heap.top();
    heap.pop();
    const auto cur = stats.find(top.pair);
    if (cur == stats.end() || cur->second.count != top.count) continue;   // stale heap entry
    if (top.count < static_cast<i64>(cfg_.min_frequency)) break;
    const i32 a = static_cast<i32>(top.pair >> 32), b = static_cast<i32>(top.pair & 0xFFFFFFFFu);
    std::string merged = vocab[static_cast<size_t>(a)] + vocab[static_cast<size_t>(b)];
    if (static_cast<int>(merged.size()) > cfg_.max_token_bytes) {
      stats.erase(cur);   // never merge this pair; occurrences created later start a fresh count
      continue;
    }
    const i32 fresh = static_cast<i32>(vocab.size());
    merges.emplace_back(vocab[static_cast<size_t>(a)], vocab[static_cast<size_t>(b)]);
    vocab.push_back(std::move(merged));
    ++done;

    std::vector<u32> affected = std::move(cur->second.words);
    stats.erase(cur);
    touched.clear();
    auto bump = [&](i32 l, i32 r, i64 delta, u32 wi) {
      const u64 k = pair_of(l, r);
      PairStat& st = stats[k];
      st.count += delta;
      if (delta > 0 && (st.words.empty() || st.words.back() != wi)) st.words.push_back(wi);
      touched.push_back(k);
    };
    for (u32 wi : affected) {
      std::vector<i32>& w = words[wi];
      const i64 f = freq[wi];
      rebuilt.clear();
      bool changed = false;
      for (size_t i = 0; i < w.size();) {
        if (i + 1 < w.size() && w[i] == a && w[i + 1] == b) {
          // left neighbour as it stands after the merges already made in this word; right neighbour unmerged
          if (!rebuilt.empty()) {
            bump(rebuilt.back(), a, -f, wi);
            bump(rebuilt.back(), fresh, +f, wi);
          }
          if (i + 2 < w.size()) {
            bump(b, w[i + 2], -f, wi);
            bump(fresh, w[i + 2], +f, wi);
          }
          rebuilt.push_back(fresh);
          i += 2;
          changed = true;
        } else {
          rebuilt.push_back(w[i++]);
        }
      }
      if (changed) w = rebuilt;
    }
    std::sort(touched.begin(), touched.end());
    touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
    for (u64 k : touched) {
      const auto it = stats.find(k);
      if (it == stats.end()) continue;
      if (it->second.count <= 0) stats.erase(it);
      else heap.push(Best{it->second.count, k});
    }
  }
  merges_done_ = done;
  // a corpus too small for the requested size leaves placeholder slots that never encode
  for (int i = 0; static_cast<int>(vocab.size()) < cfg_.vocab_size; ++i) vocab.push_back("<|unused" + std::to_string(i) + "|>");

  Tokenizer tk;
  tk.build(std::move(vocab), merges, cfg_.normalizer);
  return tk;
}

}  // namespace gbh
