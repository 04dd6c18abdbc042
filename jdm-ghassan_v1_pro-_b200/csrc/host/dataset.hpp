// Text pipeline primitives: line cleaner (HTML, mojibake, PII), quality gate, toxicity lexicon, exact + MinHash
// near-duplicate filter with an evaluation blocklist, and a lexicon language identifier for Moroccan Darija in Arabic
// and Latin script, Modern Standard Arabic, French and English.  Capability map of the reference's dataset/ module
// (dataset/cleaner.h:9-84, dedup.h:11-57, langid.h:8-62); lexicons and thresholds here are this project's own.
#pragma once
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "core.hpp"
#include "text.hpp"

namespace gbh {

// ------------------------------------------------------------------ PII
struct PiiReport {
  int emails = 0, phones = 0, urls_with_creds = 0, ibans = 0, cards = 0, api_keys = 0, ids = 0, ips = 0;
  int total() const { return emails + phones + urls_with_creds + ibans + cards + api_keys + ids + ips; }
  bool any() const { return total() > 0; }
};
PiiReport scan_pii(const std::string& text);
std::string redact_pii(const std::string& text, PiiReport* report = nullptr);   // replaces hits by <EMAIL>, <PHONE>, ...

// ------------------------------------------------------------------ cleaner
std::string strip_html_tags(const std::string& s);
std::string fix_mojibake(const std::string& s);   // UTF-8 read as Latin-1 and re-encoded ("Ã©" -> "é")

struct CleanConfig {
  bool strip_html = true, fix_mojibake = true, drop_pii_lines = true, redact_instead_drop = false;
  int min_chars = 2, max_chars = 100000;
  NormalizerConfig normalizer{};
};
struct CleanStats {
  u64 lines_in = 0, lines_out = 0, dropped_empty = 0, dropped_short = 0, dropped_long = 0, dropped_pii = 0,
      dropped_encoding = 0, dropped_quality = 0, bytes_in = 0, bytes_out = 0;
};
class Cleaner {
 public:
  explicit Cleaner(CleanConfig cfg = {}) : cfg_(cfg) {}
  bool clean_line(const std::string& in, std::string& out, CleanStats& st) const;
  const CleanConfig& config() const { return cfg_; }

 private:
  CleanConfig cfg_;
};

struct QualityConfig {
  double max_symbol_ratio = 0.25, max_digit_ratio = 0.30, max_upper_ratio = 0.40, max_repeat_line = 0.15,
         max_word_repeat = 0.15, min_letter_ratio = 0.45;
  int min_words = 2, max_word_length = 60;
  bool require_arabic_or_latin = true, reject_ai_disclaimers = true, reject_placeholders = true;
};
struct QualityVerdict {
  bool accept = true;
  std::string reason;
};
QualityVerdict quality_check(const std::string& text, const QualityConfig& cfg = {});
QualityConfig english_quality_config();
// English text: the wider English limits when `cfg` is the default one, then the hard "I am a language model" phrases
QualityVerdict quality_check_english(const std::string& text, const QualityConfig& cfg = {});

struct ToxicityResult {
  bool toxic = false;
  int hits = 0;
  std::vector<std::string> categories;
};
ToxicityResult check_toxicity(const std::string& text);

// ------------------------------------------------------------------ dedup
class Deduplicator {
 public:
  struct Config {
    bool exact = true, near = true;
    int num_hashes = 128, bands = 16, shingle = 5;
    double jaccard_threshold = 0.85;
    u64 seed = 0xD1CE5EEDull;
  };
  Deduplicator() : Deduplicator(Config{}) {}
  explicit Deduplicator(const Config& cfg);
  bool add(const std::string& text);                 // true = new (kept), false = duplicate or blocked
  bool is_duplicate(const std::string& text) const;  // query only
  void add_blocklist_text(const std::string& text);  // e.g. evaluation prompts that must not leak into training
  u64 seen() const { return seen_; }
  u64 exact_dups() const { return exact_dups_; }
  u64 near_dups() const { return near_dups_; }
  u64 blocked() const { return blocked_; }

 private:
  std::vector<u64> signature(const std::string& canonical) const;
  int near_match(const std::vector<u64>& sig) const;   // index of a stored signature above the threshold, or -1
  Config cfg_;
  std::vector<u64> seeds_;
  std::unordered_set<u64> exact_, blocklist_;
  std::vector<std::unordered_map<u64, std::vector<u32>>> bands_;
  std::vector<std::vector<u64>> sigs_;
  std::vector<char> sig_blocked_;
  u64 seen_ = 0, exact_dups_ = 0, near_dups_ = 0, blocked_ = 0;
};

// ------------------------------------------------------------------ language id
enum class LangTag : u8 { DarijaArab = 0, DarijaLatn = 1, MSA = 2, French = 3, English = 4, Mixed = 5, Other = 6 };
const char* lang_name(LangTag t);
struct LangScore {
  LangTag tag = LangTag::Other;
  double confidence = 0, darija_score = 0, msa_score = 0, french_score = 0, english_score = 0, arabizi_score = 0,
         arabic_ratio = 0, latin_ratio = 0;
};
LangScore classify_language(const std::string& text);
double msa_ratio(const std::string& text);

struct StyleFlags {
  bool has_boilerplate = false, excessive_msa = false, too_many_bullets = false, too_long = false;
  int bullet_count = 0;
  double msa_ratio = 0;
  std::vector<std::string> matched_phrases;
  bool robotic() const { return has_boilerplate || excessive_msa || too_many_bullets; }
};
StyleFlags check_assistant_style(const std::string& reply, const std::string& user_msg);
bool has_hard_ai_boilerplate(const std::string& reply);

}  // namespace gbh
