// Token shards (.gbin v1) and the stochastic batch sampler.
//
// File layout (little endian): u32 magic 0x4E494247 | u32 version 1 | u32 dtype (0 = u16 ids,
// 1 = u32 ids) | u32 flags (bit 0 = loss mask present) | u64 n_tokens | u64 n_docs | token ids |
// u64 doc_start[n_docs] | u8 mask[n_tokens] (only when flagged).  The size must match exactly.
// Same format and the same random stream as the reference (training/dataloader.h:11-22,
// training/dataloader.cpp:117-153, 475-756), so a (seed, batch index) pair names the same batch in
// both engines and checkpoints carry over.
#pragma once
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "core.hpp"

namespace gbh {

constexpr u32 kShardMagic = 0x4E494247u;

class ShardWriter {
 public:
  ShardWriter(std::string path, int vocab_size, bool with_mask);
  // tokens must lie in [0, vocab); mask (optional, 0/1 per token) defaults to all ones
  void add_document(const i32* tokens, size_t n, const u8* mask);
  void close();
  u64 token_count() const { return tokens_.size(); }
  u64 doc_count() const { return doc_starts_.size(); }

 private:
  std::string path_;
  int vocab_;
  bool with_mask_;
  bool closed_ = false;
  std::vector<u32> tokens_;
  std::vector<u8> mask_;
  std::vector<u64> doc_starts_;
};

// Read-only memory-mapped shard.
class ShardFile {
 public:
  ShardFile() = default;
  ~ShardFile();
  ShardFile(ShardFile&&) noexcept;
  ShardFile& operator=(ShardFile&&) noexcept;
  ShardFile(const ShardFile&) = delete;
  ShardFile& operator=(const ShardFile&) = delete;

  // false (with *why set) when the file is missing, truncated, oversized or internally inconsistent
  bool open(const std::string& path, std::string* why = nullptr);
  const std::string& path() const { return path_; }
  u64 n_tokens() const { return n_tokens_; }
  u64 n_docs() const { return n_docs_; }
  bool has_mask() const { return mask_ != nullptr; }
  i32 token(u64 i) const { return wide_ ? static_cast<i32>(tok32_[i]) : static_cast<i32>(tok16_[i]); }
  u8 mask(u64 i) const { return mask_ ? mask_[i] : 1; }
  u64 doc_start(u64 d) const { return d < n_docs_ ? doc_at(d) : 0; }
  // first document boundary strictly after position i (n_tokens when i is in the last document)
  u64 doc_end_after(u64 i) const;

 private:
  void reset();
  std::string path_;
  void* map_ = nullptr;
  size_t map_len_ = 0;
  u64 n_tokens_ = 0, n_docs_ = 0;
  bool wide_ = false;
  const u16* tok16_ = nullptr;
  const u32* tok32_ = nullptr;
  // the offsets follow the token array, so they sit on a 2- or 4-byte boundary: read them byte-wise
  u64 doc_at(u64 d) const {
    u64 v;
    std::memcpy(&v, docs_ + d * 8, 8);
    return v;
  }
  const u8* docs_ = nullptr;
  const u8* mask_ = nullptr;
};

std::vector<std::string> list_shards(const std::string& dir, const std::string& prefix);

struct SamplerState {
  u64 rng[4] = {0, 0, 0, 0};
  i64 batches = 0;
  float rng_spare = 0.f;
  i32 rng_has_spare = 0;
};

struct BatchOut {
  i32* ids;       // [B*T]
  i32* targets;   // [B*T], -100 = unsupervised
  i32* segments;  // [B*T]
  i64 supervised = 0;
};

// Sampling with replacement: a row picks a shard with probability proportional to its token count
// (or a domain by mix weight, then a shard), then either a random in-document window (best of up to
// four starts) or, when packing, whole random documents back to back with increasing segment ids.
class BatchSampler {
 public:
  bool open(const std::vector<std::string>& paths, int batch, int seq, bool pack, u64 seed);
  bool open_glob(const std::string& dir, const std::string& prefix, int batch, int seq, bool pack, u64 seed);
  bool open_mix(const std::string& dir, const std::map<std::string, double>& mix, int batch, int seq, bool pack,
                u64 seed);
  void set_vocab(int v) { vocab_ = v; }
  void next(BatchOut& out);
  // advance the stream by n batches without touching token data
  void fast_forward(i64 n);
  void reseed(u64 seed);
  SamplerState state() const { return committed_; }
  void set_state(const SamplerState& s);
  u64 total_tokens() const { return total_tokens_; }
  int num_shards() const;
  i64 batches_seen() const { return batches_; }
  bool using_mix() const { return !groups_.empty(); }
  bool all_have_mask() const;
  std::string mix_report() const;
  int batch() const { return B_; }
  int seq() const { return T_; }

 private:
  struct Group {
    std::string domain;
    double weight = 0;
    u64 tokens = 0;
    std::vector<std::unique_ptr<ShardFile>> shards;
  };
  struct Window {  // one contiguous run to copy into a row
    u64 start = 0, want = 0, doc_end = 0;
  };
  const ShardFile& draw_shard();
  bool draw_window(const ShardFile& sh, Window& w);              // unpacked
  bool draw_packed_doc(const ShardFile& sh, int pos, Window& w, bool& retry); // packed
  void fill_row(const ShardFile& sh, BatchOut& out, int b);
  void plan_row(const ShardFile& sh);                             // RNG draws only
  void commit();
  void start(int batch, int seq, bool pack, u64 seed);
  bool admit(std::unique_ptr<ShardFile>& s, const std::string& path);

  std::vector<std::unique_ptr<ShardFile>> shards_;
  std::vector<Group> groups_;
  Rng rng_;
  int B_ = 0, T_ = 0, vocab_ = 0;
  bool pack_ = false;
  u64 total_tokens_ = 0;
  i64 batches_ = 0;
  SamplerState committed_{};
};

}  // namespace gbh
