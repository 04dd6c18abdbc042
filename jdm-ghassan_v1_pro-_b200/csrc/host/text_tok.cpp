// Byte-level BPE tokenizer, its .gtok file and the streaming detokeniser (see text.hpp for the contract).
#include <algorithm>
#include <atomic>
#include <fstream>
#include <functional>
#include <queue>
#include <thread>
#include <unordered_set>

#include "text.hpp"

namespace gbh {

const std::vector<std::string>& special_token_strings() {
  static const std::vector<std::string> names = {
      "<pad>",  "<s>",    "</s>",   "<unk>",      "<|system|>", "<|user|>", "<|assistant|>", "<|end|>",
      "<|nl|>", "<|fr|>", "<|ar|>", "<|darija|>", "<|latin|>",  "<|tool|>", "<|mask|>",      "<|reserved|>"};
  return names;
}

namespace {
constexpr u32 kGtokMagic = 0x4B4F5447u;   // "GTOK"
constexpr u32 kGtokVersion = 1u;
constexpr u32 kMaxEntries = 10000000u;
constexpr u32 kMaxTokenBytes = 1024u;
inline u64 pair_key(i32 l, i32 r) { return (static_cast<u64>(static_cast<u32>(l)) << 32) | static_cast<u32>(r); }
bool is_unused_slot(const std::string& t) { return t.size() > 8 && t.compare(0, 8, "<|unused") == 0; }
}  // namespace

Tokenizer::Tokenizer() : cache_(std::make_shared<std::vector<CacheShard>>(kCacheShards)) {}

void Tokenizer::index_vocab() {
  ids_.clear();
  ids_.reserve(vocab_.size() * 2);
  for (size_t i = 0; i < vocab_.size(); ++i) ids_[vocab_[i]] = static_cast<i32>(i);   // a duplicate keeps the last id
  for (auto& sh : *cache_) {
    std::lock_guard<std::mutex> lk(sh.mu);
    sh.map.clear();
  }
}

void Tokenizer::init_empty(const NormalizerConfig& ncfg) {
  vocab_ = special_token_strings();
  for (int b = 0; b < 256; ++b) vocab_.emplace_back(1, static_cast<char>(b));
  merges_.clear();
  ncfg_ = ncfg;
  index_vocab();
}

void Tokenizer::build(std::vector<std::string> vocab, const std::vector<std::pair<std::string, std::string>>& merges,
                      const NormalizerConfig& ncfg) {
  vocab_ = std::move(vocab);
  ncfg_ = ncfg;
  index_vocab();
  merges_.clear();
  merges_.reserve(merges.size() * 2);
  std::unordered_set<i32> produced;
  for (size_t rank = 0; rank < merges.size(); ++rank) {
    const auto l = ids_.find(merges[rank].first), r = ids_.find(merges[rank].second);
    if (l == ids_.end() || r == ids_.end()) continue;
    const auto m = ids_.find(merges[rank].first + merges[rank].second);
    if (m == ids_.end()) continue;
    merges_[pair_key(l->second, r->second)] = Rule{static_cast<i32>(rank), m->second};
    produced.insert(m->second);
  }
  // padding slots ("<|unusedN|>") exist only to reach the configured vocabulary size: text that happens to spell
  // one must not encode to it, so they leave the lookup table unless a merge really produces them
  for (size_t i = 0; i < vocab_.size(); ++i)
    if (is_unused_slot(vocab_[i]) && !produced.count(static_cast<i32>(i))) ids_.erase(vocab_[i]);
}

std::vector<std::pair<std::string, std::string>> Tokenizer::merges_in_rank_order() const {
  std::vector<std::pair<i32, u64>> order;
  order.reserve(merges_.size());
  for (const auto& kv : merges_) order.emplace_back(kv.second.rank, kv.first);
  std::sort(order.begin(), order.end());
  std::vector<std::pair<std::string, std::string>> out;
  out.reserve(order.size());
  for (const auto& e : order) {
    const u32 l = static_cast<u32>(e.second >> 32), r = static_cast<u32>(e.second);
    if (l < vocab_.size() && r < vocab_.size()) out.emplace_back(vocab_[l], vocab_[r]);
  }
  return out;
}

// Applies merges to `sym` until none is left: always the pair of lowest rank, leftmost among equals.
void Tokenizer::merge_symbols(std::vector<i32>& sym) const {
  const size_t n = sym.size();
  if (n < 2 || merges_.empty()) return;
  if (n <= 24) {
    // short pieces (almost every word): rescan for the best pair after each merge
    size_t len = n;
    while (len > 1) {
      i32 best_rank = INT32_MAX, best_to = 0;
      size_t best_at = 0;
      for (size_t i = 0; i + 1 < len; ++i) {
        const auto it = merges_.find(pair_key(sym[i], sym[i + 1]));
        if (it != merges_.end() && it->second.rank < best_rank) {
          best_rank = it->second.rank;
          best_to = it->second.merged;
          best_at = i;
        }
      }
      if (best_rank == INT32_MAX) break;
      sym[best_at] = best_to;
      sym.erase(sym.begin() + static_cast<long>(best_at) + 1);
      --len;
    }
    return;
  }
  // long pieces: linked list over the symbols + a heap of candidate pairs, stale entries dropped on pop
  struct Cand {
    i32 rank;
    int at;
    i32 left, right, to;
  };
  auto worse = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.at > b.at; };
  std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
  std::vector<int> nxt(n), prv(n);
  std::vector<char> live(n, 1);
  for (size_t i = 0; i < n; ++i) {
    prv[i] = static_cast<int>(i) - 1;
    nxt[i] = i + 1 < n ? static_cast<int>(i) + 1 : -1;
  }
  auto offer = [&](int l) {
    if (l < 0 || nxt[l] < 0) return;
    const auto it = merges_.find(pair_key(sym[l], sym[nxt[l]]));
    if (it != merges_.end()) heap.push(Cand{it->second.rank, l, sym[l], sym[nxt[l]], it->second.merged});
  };
  for (size_t i = 0; i + 1 < n; ++i) offer(static_cast<int>(i));
  while (!heap.empty()) {
    const Cand c = heap.top();
    heap.pop();
    if (!live[c.at] || sym[c.at] != c.left) continue;
    const int r = nxt[c.at];
    if (r < 0 || !live[r] || sym[r] != c.right) continue;
    sym[c.at] = c.to;
    live[r] = 0;
    nxt[c.at] = nxt[r];
    if (nxt[r] >= 0) prv[nxt[r]] = c.at;
    offer(prv[c.at]);
    offer(c.at);
  }
  std::vector<i32> out;
  out.reserve(n);
  for (int i = 0; i >= 0; i = nxt[i]) out.push_back(sym[i]);
  sym.swap(out);
}

void Tokenizer::encode_piece(const std::string& piece, std::vector<i32>& out) const {
  if (piece.empty()) return;
  const auto whole = ids_.find(piece);
  if (whole != ids_.end() && whole->second >= special::COUNT) {   // the piece is itself a token (never a special)
    out.push_back(whole->second);
    return;
  }
  CacheShard& sh = (*cache_)[std::hash<std::string>{}(piece) % kCacheShards];
  {
    std::lock_guard<std::mutex> lk(sh.mu);
    const auto hit = sh.map.find(piece);
    if (hit != sh.map.end()) {
      out.insert(out.end(), hit->second.begin(), hit->second.end());
      return;
    }
  }
  std::vector<i32> sym(piece.size());
  for (size_t i = 0; i < piece.size(); ++i) sym[i] = special::COUNT + static_cast<i32>(static_cast<u8>(piece[i]));
  merge_symbols(sym);
  out.insert(out.end(), sym.begin(), sym.end());
  std::lock_guard<std::mutex> lk(sh.mu);
  if (sh.map.size() >= cache_limit_per_shard_) sh.map.clear();   // a memo, not a contract: start over when full
  sh.map.emplace(piece, std::move(sym));
}

void Tokenizer::encode_normalized_into(const std::string& raw, std::vector<i32>& out) const {
  for (const Chunk& c : pre_tokenize(normalize(ncfg_, raw))) encode_piece(c.text, out);
}

std::vector<i32> Tokenizer::encode(const std::string& text, bool add_bos, bool add_eos) const {
  std::vector<i32> out;
  out.reserve(text.size() / 3 + 2);
  if (add_bos) out.push_back(special::BOS);
  encode_normalized_into(text, out);
  if (add_eos) out.push_back(special::EOS);
  return out;
}

std::vector<i32> Tokenizer::encode_with_specials(const std::string& text) const {
  const auto& names = special_token_strings();
  std::vector<i32> out;
  std::string plain;
  auto flush_plain = [&] {
    if (!plain.empty()) encode_normalized_into(plain, out);
    plain.clear();
  };
  size_t i = 0;
  while (i < text.size()) {
    int hit = -1;
    if (text[i] == '<') {
      size_t hit_len = 0;
      for (size_t s = 0; s < names.size(); ++s)   // longest literal special at this position
        if (names[s].size() > hit_len && text.compare(i, names[s].size(), names[s]) == 0) {
          hit = static_cast<int>(s);
          hit_len = names[s].size();
        }
    }
    if (hit >= 0) {
      flush_plain();
      out.push_back(hit);
      i += names[static_cast<size_t>(hit)].size();
    } else {
      plain.push_back(text[i++]);
    }
  }
  flush_plain();
  return out;
}

std::vector<std::vector<i32>> Tokenizer::encode_batch(const std::vector<std::string>& texts, bool add_bos, bool add_eos,
                                                      int threads) const {
  std::vector<std::vector<i32>> out(texts.size());
  int nt = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  nt = std::max(1, std::min<int>(nt, static_cast<int>((texts.size() + 15) / 16)));
  std::atomic<size_t> cursor{0};
  auto work = [&] {
    for (;;) {
      const size_t lo = cursor.fetch_add(16);
      if (lo >= texts.size()) break;
      for (size_t k = lo; k < std::min(texts.size(), lo + 16); ++k) out[k] = encode(texts[k], add_bos, add_eos);
    }
  };
  if (nt == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& t : pool) t.join();
  }
  return out;
}

const std::string& Tokenizer::token_text(i32 id) const {
  static const std::string none;
  return id >= 0 && id < vocab_size() ? vocab_[static_cast<size_t>(id)] : none;
}

i32 Tokenizer::token_to_id(const std::string& tok) const {
  const auto it = ids_.find(tok);
  return it == ids_.end() ? -1 : it->second;
}

std::string Tokenizer::decode(const std::vector<i32>& ids, bool skip_special) const {
  std::string out;
  out.reserve(ids.size() * 3);
  for (i32 id : ids)
    if (!(skip_special && is_special(id))) out += token_text(id);
  return out;
}

std::string Tokenizer::Stream::push(i32 id) {
  held_ += tk_->token_text(id);
  // longest prefix made of complete sequences; a malformed byte is passed through on its own
  size_t done = 0;
  while (done < held_.size()) {
    const int len = uni::seq_len(static_cast<u8>(held_[done]));
    if (len == 0 || done + static_cast<size_t>(len) > held_.size()) break;
    bool well_formed = true;
    for (int k = 1; k < len && well_formed; ++k) well_formed = (static_cast<u8>(held_[done + k]) & 0xC0) == 0x80;
    done += well_formed ? static_cast<size_t>(len) : 1;
  }
  std::string ready = held_.substr(0, done);
  held_.erase(0, done);
  return ready;
}

std::string Tokenizer::Stream::flush() {
  if (held_.empty()) return {};
  std::string tail = uni::complete(held_) ? held_ : std::string("\xEF\xBF\xBD");
  held_.clear();
  return tail;
}

// ------------------------------------------------------------------ .gtok
// u32 magic, u32 version, u32 normaliser bits, u32 n_vocab, n_vocab x {u32 len, bytes}, u32 n_merges,
// n_merges x {u32 left id, u32 right id} in rank order.  Little-endian.
std::string Tokenizer::to_bytes() const {
  ByteWriter w;
  w.put<u32>(kGtokMagic);
  w.put<u32>(kGtokVersion);
  w.put<u32>(ncfg_.pack());
  w.put<u32>(static_cast<u32>(vocab_.size()));
  for (const auto& t : vocab_) {
    w.put_str32(t);
  }
  std::vector<std::pair<i32, u64>> order;
  order.reserve(merges_.size());
  for (const auto& kv : merges_) order.emplace_back(kv.second.rank, kv.first);
  std::sort(order.begin(), order.end());
  w.put<u32>(static_cast<u32>(order.size()));
  for (const auto& e : order) {
    w.put<u32>(static_cast<u32>(e.second >> 32));
    w.put<u32>(static_cast<u32>(e.second));
  }
  return std::string(w.buf.begin(), w.buf.end());
}

void Tokenizer::save(const std::string& path) const {
  const std::string blob = to_bytes();
  std::ofstream f(path, std::ios::binary);
  GBH_CHECK(f.good(), "cannot write tokenizer: " + path);
  f.write(blob.data(), static_cast<std::streamsize>(blob.size()));
  GBH_CHECK(f.good(), "tokenizer write failed: " + path);
}

bool Tokenizer::parse(const u8* p, size_t n) {
  std::vector<std::string> vocab;
  std::vector<std::pair<u32, u32>> pairs;
  u32 bits = 0, nv = 0;
  try {   // the reader throws when the data ends early
    ByteReader r(p, n);
    if (r.get<u32>() != kGtokMagic || r.get<u32>() != kGtokVersion) return false;
    bits = r.get<u32>();
    nv = r.get<u32>();
    if (nv == 0 || nv > kMaxEntries) return false;
    vocab.reserve(nv);
    for (u32 i = 0; i < nv; ++i) {
      const u32 len = r.get<u32>();
      if (len > kMaxTokenBytes) return false;
      const u8* b = r.take(len);
      vocab.emplace_back(reinterpret_cast<const char*>(b), len);
    }
    // ids 0..15 must be the specials and 16..271 the 256 single bytes, in order
    if (vocab.size() < static_cast<size_t>(special::COUNT) + 256) return false;
    const auto& names = special_token_strings();
    for (int s = 0; s < special::COUNT; ++s)
      if (vocab[static_cast<size_t>(s)] != names[static_cast<size_t>(s)]) return false;
    for (int b = 0; b < 256; ++b) {
      const std::string& t = vocab[static_cast<size_t>(special::COUNT + b)];
      if (t.size() != 1 || static_cast<u8>(t[0]) != b) return false;
    }
    const u32 nm = r.get<u32>();
    if (nm > kMaxEntries) return false;
    pairs.resize(nm);
    for (auto& pr : pairs) {
      pr.first = r.get<u32>();
      pr.second = r.get<u32>();
      if (pr.first >= nv || pr.second >= nv) return false;
    }
  } catch (const Error&) {
    return false;
  }
  vocab_ = std::move(vocab);
  ncfg_ = NormalizerConfig::unpack(bits);
  index_vocab();
  merges_.clear();
  merges_.reserve(pairs.size() * 2);
  for (size_t rank = 0; rank < pairs.size(); ++rank) {
    const auto m = ids_.find(vocab_[pairs[rank].first] + vocab_[pairs[rank].second]);
    if (m == ids_.end()) continue;   // a rule whose product is not in the vocabulary can never fire
    merges_[pair_key(static_cast<i32>(pairs[rank].first), static_cast<i32>(pairs[rank].second))] =
        Rule{static_cast<i32>(rank), m->second};
  }
  return true;
}

bool Tokenizer::load_bytes(const std::string& blob) { return parse(reinterpret_cast<const u8*>(blob.data()), blob.size()); }

bool Tokenizer::load(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f.good()) return false;
  const std::string blob((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  return load_bytes(blob);
}

Tokenizer::Fertility Tokenizer::measure(const std::vector<std::string>& lines) const {
  Fertility f;
  for (const auto& line : lines) {
    if (line.empty()) continue;
    f.tokens += encode(line).size();
    f.bytes += line.size();
    bool in_word = false;
    for (size_t i = 0; i < line.size();) {
      const bool ws = uni::is_whitespace(uni::decode(line, i));
      if (!ws && !in_word) ++f.words;
      in_word = !ws;
    }
  }
  f.tokens_per_word = f.words ? static_cast<double>(f.tokens) / static_cast<double>(f.words) : 0.0;
  f.bytes_per_token = f.tokens ? static_cast<double>(f.bytes) / static_cast<double>(f.tokens) : 0.0;
  return f;
}

}  // namespace gbh
