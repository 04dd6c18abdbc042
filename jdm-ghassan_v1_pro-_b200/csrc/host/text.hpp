// Text stack: Arabic-aware normaliser, script-aware pre-tokeniser, byte-level BPE tokenizer with its .gtok file,
// streaming detokeniser and the BPE trainer.  Token ids are a data contract (shards and checkpoints are only valid
// for the tokenizer that produced them), so the normalisation order, the chunking rules, the merge priority
// (lowest rank first, leftmost on ties) and the .gtok layout follow the reference (tokenizer/normalizer.cpp:40-234,
// tokenizer/tokenizer.cpp:25-360, tokenizer/bpe_trainer.cpp:90-271).
#pragma once
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "core.hpp"
#include "unicode.hpp"

namespace gbh {

// ------------------------------------------------------------------ normaliser
struct NormalizerConfig {
  bool strip_diacritics = true;      // bit 0
  bool strip_tatweel = true;         // bit 1
  bool unify_presentation = true;    // bit 2
  bool arabic_digits_ascii = true;   // bit 3
  bool fold_letters = false;         // bit 4
  bool lowercase_latin = true;       // bit 5
  bool collapse_whitespace = true;   // bit 6
  bool strip_control = true;         // bit 7
  bool strip_zero_width = true;      // bit 8
  bool collapse_repeats = false;     // bit 9
  bool fold_fullwidth = true;        // bit 10
  int max_repeat = 3;                // bits 16..19 (0 reads back as 3)

  u32 pack() const;
  static NormalizerConfig unpack(u32 bits);
};

std::string normalize(const NormalizerConfig& cfg, const std::string& text);
// Aggressive form used for comparisons (dedup keys, retrieval): defaults + letter folding + repeat collapsing.
std::string canonical_text(const std::string& text);

enum class ChunkKind : u8 { Arabic = 0, Latin = 1, Number = 2, Punct = 3, Space = 4, Emoji = 5, Other = 6 };
struct Chunk {
  std::string text;
  ChunkKind kind = ChunkKind::Other;
};
std::vector<Chunk> pre_tokenize(const std::string& normalized);

// ------------------------------------------------------------------ tokenizer
namespace special {
constexpr i32 PAD = 0, BOS = 1, EOS = 2, UNK = 3, SYSTEM = 4, USER = 5, ASSISTANT = 6, END = 7, NL = 8, FR = 9, AR = 10,
              DARIJA = 11, LATIN = 12, TOOL = 13, MASK = 14, RESERVED = 15, COUNT = 16;
}
const std::vector<std::string>& special_token_strings();

class Tokenizer {
 public:
  Tokenizer();
  // 16 specials + 256 byte tokens, no merges
  void init_empty(const NormalizerConfig& ncfg);
  // full vocabulary (specials, bytes, merged tokens in creation order) + the merge list in rank order
  void build(std::vector<std::string> vocab, const std::vector<std::pair<std::string, std::string>>& merges,
             const NormalizerConfig& ncfg);
  bool load(const std::string& path);
  bool load_bytes(const std::string& blob);
  void save(const std::string& path) const;
  std::string to_bytes() const;

  std::vector<i32> encode(const std::string& text, bool add_bos = false, bool add_eos = false) const;
  // text that may contain literal special-token strings ("<|user|>...") which map to their ids
  std::vector<i32> encode_with_specials(const std::string& text) const;
  // many texts at once on `threads` worker threads (0 = hardware concurrency)
  std::vector<std::vector<i32>> encode_batch(const std::vector<std::string>& texts, bool add_bos, bool add_eos,
                                             int threads) const;
  std::string decode(const std::vector<i32>& ids, bool skip_special = false) const;

  int vocab_size() const { return static_cast<int>(vocab_.size()); }
  const std::string& token_text(i32 id) const;
  i32 token_to_id(const std::string& tok) const;
  const std::vector<std::string>& vocab() const { return vocab_; }
  std::vector<std::pair<std::string, std::string>> merges_in_rank_order() const;
  size_t merge_count() const { return merges_.size(); }
  bool is_special(i32 id) const { return id >= 0 && id < special::COUNT; }
  const NormalizerConfig& normalizer_config() const { return ncfg_; }

  struct Fertility {
    double tokens_per_word = 0, bytes_per_token = 0;
    u64 tokens = 0, words = 0, bytes = 0;
  };
  Fertility measure(const std::vector<std::string>& lines) const;

  // Incremental detokeniser: emits only complete UTF-8 sequences, holds back a split multi-byte character.
  class Stream {
   public:
    explicit Stream(const Tokenizer& tk) : tk_(&tk) {}
    std::string push(i32 id);
    std::string flush();

   private:
    const Tokenizer* tk_;
    std::string held_;
  };

 private:
  struct Rule {
    i32 rank;
    i32 merged;
  };
  void index_vocab();
  void encode_piece(const std::string& piece, std::vector<i32>& out) const;
  void merge_symbols(std::vector<i32>& sym) const;
  void encode_normalized_into(const std::string& raw, std::vector<i32>& out) const;
  bool parse(const u8* p, size_t n);

  std::vector<std::string> vocab_;
  std::unordered_map<std::string, i32> ids_;
  std::unordered_map<u64, Rule> merges_;   // (left id << 32 | right id) -> rank, merged id
  NormalizerConfig ncfg_;
  // memo of already-merged pieces; sharded so that encode_batch threads rarely contend
  static constexpr int kCacheShards = 16;
  struct CacheShard {
    std::mutex mu;
    std::unordered_map<std::string, std::vector<i32>> map;
  };
  std::shared_ptr<std::vector<CacheShard>> cache_;
  size_t cache_limit_per_shard_ = 200000 / kCacheShards;
};

// ------------------------------------------------------------------ BPE trainer
struct BpeTrainerConfig {
  int vocab_size = 32000;
  int min_frequency = 2;
  int max_token_bytes = 32;
  NormalizerConfig normalizer{};
};

class BpeTrainer {
 public:
  explicit BpeTrainer(BpeTrainerConfig cfg) : cfg_(std::move(cfg)) {}
  void add_text(const std::string& text);
  void add_file(const std::string& path);
  void add_chunk_counts(const std::string& chunk, u64 count);
  Tokenizer train();
  u64 unique_chunks() const { return counts_.size(); }
  u64 total_chunks() const { return total_; }
  int merges_done() const { return merges_done_; }

 private:
  BpeTrainerConfig cfg_;
  std::unordered_map<std::string, u64> counts_;
  u64 total_ = 0;
  int merges_done_ = 0;
};

}  // namespace gbh
