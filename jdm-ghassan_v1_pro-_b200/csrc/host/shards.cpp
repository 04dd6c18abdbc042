#include "shards.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdarg>
#include <filesystem>
#include <fstream>

namespace fs = std::filesystem;

namespace gbh {

std::string sfmt(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  va_list ap2;
  va_copy(ap2, ap);
  const int n = std::vsnprintf(nullptr, 0, fmt, ap);
  va_end(ap);
  std::string out;
  if (n > 0) {
    out.resize(static_cast<size_t>(n) + 1);
    std::vsnprintf(out.data(), out.size(), fmt, ap2);
    out.resize(static_cast<size_t>(n));
  }
  va_end(ap2);
  return out;
}

u64 fingerprint_file(const std::string& path) {
  std::FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) return 0;
  u64 h = kFnvOffset;
  std::vector<u8> buf(1 << 16);
  size_t got;
  while ((got = std::fread(buf.data(), 1, buf.size(), f)) > 0) h = fnv1a64(buf.data(), got, h);
  std::fclose(f);
  return h ? h : 1ULL;
}

std::string fingerprint_hex(u64 fp) {
  if (!fp) return "unknown";
  return sfmt("%016llx", static_cast<unsigned long long>(fp));
}

std::vector<u8> read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  GBH_CHECK(f.good(), "cannot open file: " + path);
  const std::streamoff n = f.tellg();
  std::vector<u8> out(static_cast<size_t>(n));
  f.seekg(0);
  if (n) f.read(reinterpret_cast<char*>(out.data()), n);
  GBH_CHECK(f.good() || n == 0, "short read: " + path);
  return out;
}

void write_file_atomic(const std::string& path, const void* data, size_t n) {
  const std::string tmp = path + ".tmp";
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    GBH_CHECK(f.good(), "cannot write file: " + tmp);
    f.write(static_cast<const char*>(data), static_cast<std::streamsize>(n));
    f.flush();
    GBH_CHECK(f.good(), "write failed: " + tmp);
  }
  std::error_code ec;
  fs::rename(tmp, path, ec);
  GBH_CHECK(!ec, "rename failed: " + tmp + " -> " + path);
}

// ============================================================================ writer
ShardWriter::ShardWriter(std::string path, int vocab_size, bool with_mask)
    : path_(std::move(path)), vocab_(vocab_size), with_mask_(with_mask) {
  GBH_CHECK(vocab_size > 0, "shard writer needs a positive vocabulary size");
}

void ShardWriter::add_document(const i32* tokens, size_t n, const u8* mask) {
  GBH_CHECK(!closed_, "shard already closed: " + path_);
  if (n == 0) return;
  GBH_CHECK(with_mask_ || !mask, "loss mask supplied to a shard writer created without a mask");
  for (size_t i = 0; i < n; ++i) {
    GBH_CHECK(tokens[i] >= 0 && tokens[i] < vocab_,
              sfmt("token id %d out of writing-vocab range [0,%d)", tokens[i], vocab_));
    if (mask) GBH_CHECK(mask[i] <= 1, sfmt("loss mask must be 0/1, got %u at position %zu", unsigned(mask[i]), i));
  }
  doc_starts_.push_back(tokens_.size());
  tokens_.insert(tokens_.end(), tokens, tokens + n);
  if (with_mask_) {
    if (mask) mask_.insert(mask_.end(), mask, mask + n);
    else mask_.insert(mask_.end(), n, u8(1));
  }
}

void ShardWriter::close() {
  if (closed_) return;
  fs::path p(path_);
  if (p.has_parent_path()) fs::create_directories(p.parent_path());
  ByteWriter w;
  const bool narrow = vocab_ <= 65535;
  w.put<u32>(kShardMagic);
  w.put<u32>(1);
  w.put<u32>(narrow ? 0u : 1u);
  w.put<u32>(with_mask_ ? 1u : 0u);
  w.put<u64>(tokens_.size());
  w.put<u64>(doc_starts_.size());
  if (narrow) {
    for (u32 t : tokens_) w.put<u16>(static_cast<u16>(t));
  } else {
    w.put_bytes(tokens_.data(), tokens_.size() * 4);
  }
  w.put_bytes(doc_starts_.data(), doc_starts_.size() * 8);
  if (with_mask_) w.put_bytes(mask_.data(), mask_.size());
  std::ofstream f(path_, std::ios::binary | std::ios::trunc);
  GBH_CHECK(f.good(), "cannot write shard: " + path_);
  f.write(reinterpret_cast<const char*>(w.buf.data()), static_cast<std::streamsize>(w.buf.size()));
  f.flush();
  GBH_CHECK(f.good(), "shard write failed: " + path_);
  closed_ = true;
}

// ============================================================================ reader
ShardFile::~ShardFile() { reset(); }
void ShardFile::reset() {
  if (map_) munmap(map_, map_len_);
  map_ = nullptr;
  map_len_ = 0;
  tok16_ = nullptr;
  tok32_ = nullptr;
  docs_ = nullptr;
  mask_ = nullptr;
  n_tokens_ = n_docs_ = 0;
}
ShardFile::ShardFile(ShardFile&& o) noexcept { *this = std::move(o); }
ShardFile& ShardFile::operator=(ShardFile&& o) noexcept {
  if (this != &o) {
    reset();
    path_ = std::move(o.path_);
    map_ = o.map_; map_len_ = o.map_len_;
    n_tokens_ = o.n_tokens_; n_docs_ = o.n_docs_; wide_ = o.wide_;
    tok16_ = o.tok16_; tok32_ = o.tok32_; docs_ = o.docs_; mask_ = o.mask_;
    o.map_ = nullptr; o.map_len_ = 0;
    o.reset();
  }
  return *this;
}

bool ShardFile::open(const std::string& path, std::string* why) {
  auto bad = [&](const char* m) {
    if (why) *why = m;
    reset();
    return false;
  };
  reset();
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return bad("cannot open");
  struct stat st {};
  if (fstat(fd, &st) != 0 || st.st_size < 32) {
    ::close(fd);
    return bad("shorter than a shard header");
  }
  map_len_ = static_cast<size_t>(st.st_size);
  map_ = mmap(nullptr, map_len_, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (map_ == MAP_FAILED) {
    map_ = nullptr;
    return bad("mmap failed");
  }
  const u8* base = static_cast<const u8*>(map_);
  ByteReader r(base, 32);
  const u32 magic = r.get<u32>(), ver = r.get<u32>(), dtype = r.get<u32>(), flags = r.get<u32>();
  const u64 nt = r.get<u64>(), nd = r.get<u64>();
  if (magic != kShardMagic || ver != 1) return bad("bad magic or version");
  if (dtype > 1 || (flags & ~1u) || nd > nt) return bad("bad header fields");
  if (nt > (8ull << 30) / 2 || nd > (1ull << 30)) return bad("header counts out of range");
  const u64 tok_bytes = nt * (dtype ? 4 : 2);
  const u64 need = 32 + tok_bytes + nd * 8 + ((flags & 1u) ? nt : 0);
  if (need != map_len_) return bad("file size does not match the header");
  wide_ = dtype == 1;
  if (wide_) tok32_ = reinterpret_cast<const u32*>(base + 32);
  else tok16_ = reinterpret_cast<const u16*>(base + 32);
  docs_ = base + 32 + tok_bytes;
  if (flags & 1u) mask_ = base + 32 + tok_bytes + nd * 8;
  n_tokens_ = nt;
  n_docs_ = nd;
  // document starts: first is 0, strictly increasing, all inside the token range
  if (nd == 0) {
    if (nt != 0) { /* a shard without document table is one long document */ }
  } else {
    u64 prev = 0;
    for (u64 d = 0; d < nd; ++d) {
      u64 v;
      std::memcpy(&v, docs_ + d * 8, 8);
      if ((d == 0 && v != 0) || (d > 0 && v <= prev) || v >= nt) return bad("bad document offsets");
      prev = v;
    }
  }
  if (mask_) {
    for (u64 i = 0; i < nt; ++i)
      if (mask_[i] > 1) return bad("loss mask is not binary");
  }
  if (nd == 0 && nt == 0) return bad("empty shard");
  path_ = path;
  return true;
}

u64 ShardFile::doc_end_after(u64 i) const {
  if (n_docs_ == 0) return n_tokens_;
  u64 lo = 0, hi = n_docs_;                  // first document whose start is > i
  while (lo < hi) {
    const u64 mid = lo + (hi - lo) / 2;
    if (doc_at(mid) <= i) lo = mid + 1;
    else hi = mid;
  }
  return lo == n_docs_ ? n_tokens_ : doc_at(lo);
}

std::vector<std::string> list_shards(const std::string& dir, const std::string& prefix) {
  std::vector<std::string> out;
  std::error_code ec;
  if (!fs::exists(dir, ec)) return out;
  for (const auto& e : fs::directory_iterator(dir, ec)) {
    if (ec) break;
    std::error_code fec;
    if (!e.is_regular_file(fec) || fec) continue;
    const std::string name = e.path().filename().string();
    if (name.size() < 5 || name.compare(name.size() - 5, 5, ".gbin") != 0) continue;
    if (!prefix.empty() && name.compare(0, prefix.size(), prefix) != 0) continue;
    out.push_back(e.path().string());
  }
  std::sort(out.begin(), out.end());
  return out;
}

// ============================================================================ sampler
void BatchSampler::start(int batch, int seq, bool pack, u64 seed) {
  B_ = batch;
  T_ = seq;
  pack_ = pack;
  rng_.reseed(seed);
  shards_.clear();
  groups_.clear();
  total_tokens_ = 0;
  batches_ = 0;
  commit();
}

void BatchSampler::commit() {
  const RngState& st = rng_.state();
  for (int i = 0; i < 4; ++i) committed_.rng[i] = st.s[i];
  committed_.rng_spare = st.spare;
  committed_.rng_has_spare = st.has_spare ? 1 : 0;
  committed_.batches = batches_;
}

bool BatchSampler::admit(std::unique_ptr<ShardFile>& s, const std::string& path) {
  s = std::make_unique<ShardFile>();
  std::string why;
  if (!s->open(path, &why)) return false;
  const u64 min_tokens = pack_ ? 2u : static_cast<u64>(T_) + 1u;
  return s->n_tokens() >= min_tokens;
}

bool BatchSampler::open(const std::vector<std::string>& paths, int batch, int seq, bool pack, u64 seed) {
  if (batch <= 0 || seq <= 0) return false;
  start(batch, seq, pack, seed);
  for (const auto& p : paths) {
    std::unique_ptr<ShardFile> s;
    if (!admit(s, p)) continue;
    total_tokens_ += s->n_tokens();
    shards_.push_back(std::move(s));
  }
  return !shards_.empty();
}

bool BatchSampler::open_glob(const std::string& dir, const std::string& prefix, int batch, int seq, bool pack,
                             u64 seed) {
  return open(list_shards(dir, prefix), batch, seq, pack, seed);
}

bool BatchSampler::open_mix(const std::string& dir, const std::map<std::string, double>& mix, int batch, int seq,
                            bool pack, u64 seed) {
  if (batch <= 0 || seq <= 0) return false;
  start(batch, seq, pack, seed);
  double wsum = 0;
  for (const auto& [domain, w] : mix) {
    if (!std::isfinite(w) || !(w > 0.0)) continue;
    const std::string stem = "train_" + domain + "_";
    Group g;
    g.domain = domain;
    g.weight = w;
    for (const auto& p : list_shards(dir, stem)) {
      std::unique_ptr<ShardFile> s;
      if (!admit(s, p)) continue;
      g.tokens += s->n_tokens();
      g.shards.push_back(std::move(s));
    }
    if (g.shards.empty()) continue;
    wsum += w;
    total_tokens_ += g.tokens;
    groups_.push_back(std::move(g));
  }
  if (groups_.empty()) {
    total_tokens_ = 0;
    return false;
  }
  for (auto& g : groups_) g.weight /= wsum;
  return true;
}

int BatchSampler::num_shards() const {
  if (groups_.empty()) return static_cast<int>(shards_.size());
  int n = 0;
  for (const auto& g : groups_) n += static_cast<int>(g.shards.size());
  return n;
}

bool BatchSampler::all_have_mask() const {
  bool any = false;
  auto scan = [&](const std::vector<std::unique_ptr<ShardFile>>& v) {
    for (const auto& s : v) {
      any = true;
      if (!s->has_mask()) return false;
    }
    return true;
  };
  if (groups_.empty()) return scan(shards_) && any;
  for (const auto& g : groups_)
    if (!scan(g.shards)) return false;
  return any;
}

std::string BatchSampler::mix_report() const {
  if (groups_.empty()) return "";
  std::string s = "mix:";
  for (const auto& g : groups_)
    s += sfmt(" %s=%.2f(%llu tok)", g.domain.c_str(), g.weight, static_cast<unsigned long long>(g.tokens));
  return s;
}

static const ShardFile& pick_by_tokens(const std::vector<std::unique_ptr<ShardFile>>& v, u64 pick) {
  size_t i = 0;
  for (; i + 1 < v.size(); ++i) {
    if (pick < v[i]->n_tokens()) break;
    pick -= v[i]->n_tokens();
  }
  return *v[i];
}

const ShardFile& BatchSampler::draw_shard() {
  if (!groups_.empty()) {
    const double r = static_cast<double>(rng_.uniform());
    double acc = 0;
    size_t gi = groups_.size() - 1;
    for (size_t i = 0; i < groups_.size(); ++i) {
      acc += groups_[i].weight;
      if (r < acc) {
        gi = i;
        break;
      }
    }
    const Group& g = groups_[gi];
    return pick_by_tokens(g.shards, rng_.below(g.tokens));
  }
  return pick_by_tokens(shards_, rng_.below(total_tokens_));
}

// Best of up to four random starts: keep the start with the longest run to its document end,
// stop early once a full row (+1 for the last target) fits.
bool BatchSampler::draw_window(const ShardFile& sh, Window& w) {
  const u64 need = static_cast<u64>(T_) + 1;
  u64 best = 0;
  for (int attempt = 0; attempt < 4; ++attempt) {
    const u64 last = sh.n_tokens() ? sh.n_tokens() - 1 : 0;
    u64 start = last ? rng_.below(last + 1) : 0;
    u64 end = sh.doc_end_after(start);
    u64 avail = end > start ? end - start : 0;
    if (!avail) {
      start = sh.n_docs() ? sh.doc_start(rng_.below(sh.n_docs())) : 0;
      end = sh.doc_end_after(start);
      avail = end > start ? end - start : 0;
    }
    if (avail > best) {
      best = avail;
      w.start = start;
      w.doc_end = end;
      if (best >= need) break;
    }
  }
  if (!best || w.start >= sh.n_tokens()) return false;
  w.want = std::min(best, need);
  if (w.start + w.want > sh.n_tokens()) w.want = sh.n_tokens() - w.start;
  return w.want > 0;
}

// One random whole document (truncated to the space left in the row, +1 token for the last target).
// retry=true: an empty document was drawn, draw again; false return with retry=false: stop the row.
bool BatchSampler::draw_packed_doc(const ShardFile& sh, int pos, Window& w, bool& retry) {
  retry = false;
  const u64 start = sh.doc_start(rng_.below(sh.n_docs()));
  const u64 end = sh.doc_end_after(start);
  const u64 len = end > start ? end - start : 0;
  if (!len) {
    retry = true;
    return false;
  }
  u64 want = std::min<u64>(len, static_cast<u64>(T_ - pos) + 1);
  if (start + want > sh.n_tokens()) want = sh.n_tokens() - start;
  if (!want) return false;
  w.start = start;
  w.want = want;
  w.doc_end = end;
  return true;
}

static void copy_run(const ShardFile& sh, u64 start, u64 want, u64 doc_end, int room, int vocab, i32* ids, i32* tgt,
                     i32* seg, i32 segment, i64& supervised) {
  const int n = static_cast<int>(std::min<u64>(want, static_cast<u64>(room)));
  for (int i = 0; i < n; ++i) {
    const u64 at = start + static_cast<u64>(i);
    const i32 tok = sh.token(at);
    if (vocab > 0 && (tok < 0 || tok >= vocab))
      fail(sfmt("dataloader: token id %d out of range [0,%d) at shard %s pos %llu (corrupt shard or vocab mismatch)",
                tok, vocab, sh.path().c_str(), static_cast<unsigned long long>(at)));
    ids[i] = tok;
    seg[i] = segment;
    const bool has_next = static_cast<u64>(i) + 1 < want && at + 1 < doc_end;
    if (has_next && sh.mask(at + 1)) {
      const i32 nxt = sh.token(at + 1);
      if (vocab > 0 && (nxt < 0 || nxt >= vocab))
        fail(sfmt("dataloader: token id %d out of range [0,%d) at shard %s pos %llu (corrupt shard or vocab mismatch)",
                  nxt, vocab, sh.path().c_str(), static_cast<unsigned long long>(at + 1)));
      tgt[i] = nxt;
      ++supervised;
    }
  }
}

void BatchSampler::fill_row(const ShardFile& sh, BatchOut& out, int b) {
  const size_t row = static_cast<size_t>(b) * static_cast<size_t>(T_);
  if (!pack_) {
    Window w;
    if (draw_window(sh, w))
      copy_run(sh, w.start, w.want, w.doc_end, T_, vocab_, out.ids + row, out.targets + row, out.segments + row, 0,
               out.supervised);
    return;
  }
  int pos = 0;
  i32 segment = 0;
  while (pos < T_) {
    Window w;
    bool retry;
    if (!draw_packed_doc(sh, pos, w, retry)) {
      if (retry) continue;
      break;
    }
    copy_run(sh, w.start, w.want, w.doc_end, T_ - pos, vocab_, out.ids + row + pos, out.targets + row + pos,
             out.segments + row + pos, segment, out.supervised);
    pos += static_cast<int>(std::min<u64>(w.want, static_cast<u64>(T_ - pos)));
    ++segment;
  }
}

void BatchSampler::plan_row(const ShardFile& sh) {
  if (!pack_) {
    Window w;
    draw_window(sh, w);
    return;
  }
  int pos = 0;
  while (pos < T_) {
    Window w;
    bool retry;
    if (!draw_packed_doc(sh, pos, w, retry)) {
      if (retry) continue;
      break;
    }
    pos += static_cast<int>(std::min<u64>(w.want, static_cast<u64>(T_ - pos)));
  }
}

void BatchSampler::next(BatchOut& out) {
  GBH_CHECK(num_shards() > 0, "dataloader: no shards are open");
  const size_t n = static_cast<size_t>(B_) * static_cast<size_t>(T_);
  std::fill(out.ids, out.ids + n, 0);
  std::fill(out.targets, out.targets + n, -100);
  std::fill(out.segments, out.segments + n, 0);  // padding stays attention-neutral (segment 0)
  out.supervised = 0;
  for (int b = 0; b < B_; ++b) {
    const ShardFile& sh = draw_shard();
    if (pack_ && sh.n_docs() == 0)
      fail("dataloader: packed sampling needs a document table: " + sh.path());
    fill_row(sh, out, b);
  }
  ++batches_;
  commit();
}

void BatchSampler::fast_forward(i64 n) {
  if (n <= 0 || num_shards() == 0) return;
  for (i64 s = 0; s < n; ++s) {
    for (int b = 0; b < B_; ++b) {
      const ShardFile& sh = draw_shard();
      if (pack_ && sh.n_docs() == 0) continue;
      plan_row(sh);
    }
    ++batches_;
  }
  commit();
}

void BatchSampler::reseed(u64 seed) {
  rng_.reseed(seed);
  batches_ = 0;
  commit();
}

void BatchSampler::set_state(const SamplerState& s) {
  RngState st;
  for (int i = 0; i < 4; ++i) st.s[i] = s.rng[i];
  st.spare = s.rng_spare;
  st.has_spare = s.rng_has_spare != 0;
  rng_.set_state(st);
  batches_ = s.batches;
  committed_ = s;
}

}  // namespace gbh
