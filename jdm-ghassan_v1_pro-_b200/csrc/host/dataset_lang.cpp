// Near-duplicate filter (MinHash + banded LSH) and lexicon language identification (see dataset.hpp).
#include <algorithm>
#include <cmath>
#include <sstream>

#include "dataset.hpp"

namespace gbh {

// ------------------------------------------------------------------ dedup
Deduplicator::Deduplicator(const Config& cfg) : cfg_(cfg) {
  GBH_CHECK(cfg_.num_hashes > 0 && cfg_.bands > 0 && cfg_.num_hashes % cfg_.bands == 0, "dedup: bands must divide num_hashes");
  u64 s = cfg_.seed;
  for (int i = 0; i < cfg_.num_hashes; ++i) seeds_.push_back(s = splitmix64(s));
  bands_.resize(static_cast<size_t>(cfg_.bands));
}

std::vector<u64> Deduplicator::signature(const std::string& canonical) const {
  // character shingles of `shingle` code points, hashed once, then re-mixed per permutation
  std::vector<size_t> starts;
  for (size_t i = 0; i < canonical.size();) {
    starts.push_back(i);
    uni::decode(canonical, i);
  }
  starts.push_back(canonical.size());
  std::vector<u64> sig(static_cast<size_t>(cfg_.num_hashes), ~0ull);
  const size_t k = static_cast<size_t>(cfg_.shingle);
  const size_t n_chars = starts.size() - 1;
  const size_t n_sh = n_chars >= k ? n_chars - k + 1 : 1;
  for (size_t i = 0; i < n_sh; ++i) {
    const size_t lo = starts[i], hi = starts[std::min(n_chars, i + k)];
    const u64 h = fnv1a64(canonical.data() + lo, hi - lo);
    for (size_t j = 0; j < sig.size(); ++j) sig[j] = std::min(sig[j], splitmix64(h ^ seeds_[j]));
  }
  return sig;
}

int Deduplicator::near_match(const std::vector<u64>& sig) const {
  const int rows = cfg_.num_hashes / cfg_.bands;
  for (int b = 0; b < cfg_.bands; ++b) {
    const u64 key = fnv1a64(sig.data() + b * rows, static_cast<size_t>(rows) * sizeof(u64));
    const auto it = bands_[static_cast<size_t>(b)].find(key);
    if (it == bands_[static_cast<size_t>(b)].end()) continue;
    for (u32 cand : it->second) {
      int same = 0;
      for (size_t j = 0; j < sig.size(); ++j) same += sig[j] == sigs_[cand][j];
      if (static_cast<double>(same) / sig.size() >= cfg_.jaccard_threshold) return static_cast<int>(cand);
    }
  }
  return -1;
}

void Deduplicator::add_blocklist_text(const std::string& text) {
  const std::string canon = canonical_text(text);
  if (canon.empty()) return;
  blocklist_.insert(fnv1a64(canon.data(), canon.size()));
  if (cfg_.near) {
    std::vector<u64> sig = signature(canon);
    const int rows = cfg_.num_hashes / cfg_.bands;
    const u32 id = static_cast<u32>(sigs_.size());
    for (int b = 0; b < cfg_.bands; ++b)
      bands_[static_cast<size_t>(b)][fnv1a64(sig.data() + b * rows, static_cast<size_t>(rows) * sizeof(u64))].push_back(id);
    sigs_.push_back(std::move(sig));
    sig_blocked_.push_back(1);
  }
}

bool Deduplicator::is_duplicate(const std::string& text) const {
  const std::string canon = canonical_text(text);
  const u64 h = fnv1a64(canon.data(), canon.size());
  if (blocklist_.count(h) || (cfg_.exact && exact_.count(h))) return true;
  return cfg_.near && near_match(signature(canon)) >= 0;
}

bool Deduplicator::add(const std::string& text) {
  ++seen_;
  const std::string canon = canonical_text(text);
  const u64 h = fnv1a64(canon.data(), canon.size());
  if (blocklist_.count(h)) {
    ++blocked_;
    return false;
  }
  if (cfg_.exact) {
    if (exact_.count(h)) {
      ++exact_dups_;
      return false;
    }
    exact_.insert(h);
  }
  if (cfg_.near) {
    std::vector<u64> sig = signature(canon);
    const int hit = near_match(sig);
    if (hit >= 0) {
      if (sig_blocked_[static_cast<size_t>(hit)]) ++blocked_;
      else ++near_dups_;
      return false;
    }
    const int rows = cfg_.num_hashes / cfg_.bands;
    const u32 id = static_cast<u32>(sigs_.size());
    for (int b = 0; b < cfg_.bands; ++b)
      bands_[static_cast<size_t>(b)][fnv1a64(sig.data() + b * rows, static_cast<size_t>(rows) * sizeof(u64))].push_back(id);
    sigs_.push_back(std::move(sig));
    sig_blocked_.push_back(0);
  }
  return true;
}

// ------------------------------------------------------------------ language id
namespace {

const std::unordered_set<std::string>& lexicon(int which) {
  // function words and very frequent forms; Arabic entries are in canonical (letter-folded) spelling
  static const std::unordered_set<std::string> darija_ar = {
      "واش", "بزاف", "ديال", "دابا", "كيفاش", "علاش", "شنو", "فين", "غادي", "كنت", "كاين", "ماشي", "هادشي", "هاد", "ديالي",
      "ديالك", "بغيت", "كيف", "داير", "مزيان", "خويا", "صافي", "شحال", "عافاك", "بحال", "حيت", "راه", "باش", "كاع",
      "والو", "شي", "هضر", "دير", "كندير", "كنهضر", "معاك", "ليا", "ليك", "لينا"};
  static const std::unordered_set<std::string> darija_lat = {
      "wach", "bzaf", "bzzaf", "dyal", "daba", "kifach", "3lach", "chno", "fin", "ghadi", "kayn", "machi", "hadchi", "had",
      "dyali", "dyalk", "bghit", "kidayr", "mzyan", "khoya", "safi", "ch7al", "3afak", "b7al", "7it", "rah", "bach", "ga3",
      "walo", "chi", "hder", "dir", "m3a", "m3ak", "lik", "salam", "labas", "wakha", "3la", "f", "l", "w", "ana", "nta", "nti"};
  static const std::unordered_set<std::string> msa = {
      "الذي", "التي", "الذين", "هذا", "هذه", "ذلك", "لكن", "حيث", "ليس", "سوف", "لقد", "يجب", "يمكن", "كذلك", "ايضا",
      "بينما", "عندما", "لذلك", "حتي", "اذا", "ماذا", "لماذا", "كيف", "اين", "نحن", "انتم", "هؤلاء", "تلك", "الان", "جدا"};
  static const std::unordered_set<std::string> french = {
      "le", "la", "les", "des", "une", "est", "et", "que", "qui", "dans", "pour", "pas", "sur", "avec", "vous", "nous",
      "je", "tu", "il", "elle", "mais", "ou", "donc", "car", "ce", "cette", "sont", "être", "avoir", "très", "bonjour", "merci"};
  static const std::unordered_set<std::string> english = {
      "the", "and", "is", "are", "was", "were", "of", "to", "in", "that", "it", "for", "with", "as", "this", "you", "have",
      "not", "but", "from", "they", "what", "which", "can", "will", "would", "there", "their", "about", "how", "why", "hello",
      "please", "thanks", "i", "a", "an", "be", "on", "at", "by", "we", "he", "she", "do", "does", "did"};
  switch (which) {
    case 0: return darija_ar;
    case 1: return darija_lat;
    case 2: return msa;
    case 3: return french;
    default: return english;
  }
}

std::vector<std::string> words_of(const std::string& canon) {
  std::vector<std::string> out;
  std::string cur;
  for (size_t i = 0; i < canon.size();) {
    const size_t at = i;
    const u32 c = uni::decode(canon, i);
    const bool wordish = uni::is_arabic_letter(c) || uni::is_latin_letter(c) || uni::is_ascii_digit(c) || c == '\'';
    if (wordish) cur.append(canon, at, i - at);
    else if (!cur.empty()) {
      out.push_back(std::move(cur));
      cur.clear();
    }
  }
  if (!cur.empty()) out.push_back(std::move(cur));
  return out;
}

bool arabizi_shape(const std::string& w) {   // a Latin word carrying one of the digits used as letters
  bool letter = false, digit = false;
  for (char c : w) {
    letter |= (c >= 'a' && c <= 'z');
    digit |= c == '3' || c == '7' || c == '9' || c == '5' || c == '2';
  }
  return letter && digit;
}

}  // namespace

const char* lang_name(LangTag t) {
  static const char* names[] = {"ar-MA-arab", "ar-MA-latn", "ar-MSA", "fr", "en", "mixed", "other"};
  return names[static_cast<int>(t)];
}

LangScore classify_language(const std::string& text) {
  LangScore r;
  const uni::ScriptStats st = uni::script_stats(text);
  const double letters = static_cast<double>(st.arabic + st.latin);
  if (letters < 1) return r;
  r.arabic_ratio = st.arabic / letters;
  r.latin_ratio = st.latin / letters;
  const std::vector<std::string> ws = words_of(canonical_text(text));
  if (ws.empty()) return r;
  double hit[5] = {0, 0, 0, 0, 0}, shaped = 0;
  for (const auto& w : ws) {
    for (int k = 0; k < 5; ++k) hit[k] += lexicon(k).count(w);
    shaped += arabizi_shape(w);
  }
  const double n = static_cast<double>(ws.size());
  r.darija_score = hit[0] / n;
  r.arabizi_score = (hit[1] + shaped) / n;
  r.msa_score = hit[2] / n;
  r.french_score = hit[3] / n;
  r.english_score = hit[4] / n;
  if (r.arabic_ratio >= 0.7) {
    // Arabic script: Darija unless Standard-Arabic function words clearly dominate
    const bool msa = r.msa_score > r.darija_score + 0.02 && r.msa_score >= 0.05;
    r.tag = msa ? LangTag::MSA : LangTag::DarijaArab;
    r.confidence = std::min(1.0, 0.4 + 2.0 * std::fabs(r.darija_score - r.msa_score) + (msa ? 0 : 0.1));
  } else if (r.latin_ratio >= 0.7) {
    const double best = std::max({r.arabizi_score, r.french_score, r.english_score});
    if (best < 0.04) {
      r.tag = LangTag::Other;
      r.confidence = 0.2;
    } else if (r.arabizi_score >= r.french_score && r.arabizi_score >= r.english_score * 0.8 && r.arabizi_score >= 0.08) {
      r.tag = LangTag::DarijaLatn;
      r.confidence = std::min(1.0, 0.35 + 2.0 * r.arabizi_score);
    } else if (r.english_score >= r.french_score) {
      r.tag = LangTag::English;
      r.confidence = std::min(1.0, 0.35 + 2.0 * r.english_score);
    } else {
      r.tag = LangTag::French;
      r.confidence = std::min(1.0, 0.35 + 2.0 * r.french_score);
    }
  } else {
    r.tag = LangTag::Mixed;
    r.confidence = 0.5;
  }
  return r;
}

double msa_ratio(const std::string& text) {
  const std::vector<std::string> ws = words_of(canonical_text(text));
  if (ws.empty()) return 0.0;
  double m = 0, ar = 0;
  for (const auto& w : ws) {
    size_t i = 0;
    const bool arabic_word = uni::is_arabic_letter(uni::decode(w, i));
    ar += arabic_word;
    m += lexicon(2).count(w);
  }
  return ar > 0 ? m / ar : 0.0;
}

bool has_hard_ai_boilerplate(const std::string& reply) {
  std::string low;
  for (char c : reply) low.push_back(c >= 'A' && c <= 'Z' ? static_cast<char>(c + 32) : c);
  for (const char* p : {"as an ai language model", "as a language model", "as an ai,", "as an ai i", "i am an ai language model",
                        "i'm just an ai", "i cannot assist with that request", "كنموذج لغوي", "كذكاء اصطناعي"})
    if (low.find(p) != std::string::npos) return true;
  return false;
}

StyleFlags check_assistant_style(const std::string& reply, const std::string& user_msg) {
  StyleFlags f;
  static const char* phrases[] = {"i hope this helps", "feel free to ask", "in conclusion", "it is important to note",
                                  "as an ai", "i'm here to help", "let me know if you have", "certainly! here",
                                  "بالتأكيد", "يسعدني مساعدتك", "لا تتردد في", "في الختام", "من المهم أن"};
  std::string low;
  for (char c : reply) low.push_back(c >= 'A' && c <= 'Z' ? static_cast<char>(c + 32) : c);
  for (const char* p : phrases)
    if (low.find(p) != std::string::npos) f.matched_phrases.emplace_back(p);
  f.has_boilerplate = !f.matched_phrases.empty() || has_hard_ai_boilerplate(reply);
  std::istringstream ls(reply);
  for (std::string line; std::getline(ls, line);) {
    size_t i = 0;
    while (i < line.size() && (line[i] == ' ' || line[i] == '\t')) ++i;
    if (i < line.size() && (line[i] == '-' || line[i] == '*' || line.compare(i, 3, "•") == 0 ||
                            (std::isdigit(static_cast<unsigned char>(line[i])) && i + 1 < line.size() && (line[i + 1] == '.' || line[i + 1] == ')'))))
      ++f.bullet_count;
  }
  f.too_many_bullets = f.bullet_count > 6;
  f.msa_ratio = msa_ratio(reply);
  // a Darija question answered in Standard Arabic reads as a textbook, not a person
  const LangScore u = classify_language(user_msg);
  const bool user_darija = u.tag == LangTag::DarijaArab || u.tag == LangTag::DarijaLatn;
  f.excessive_msa = user_darija && f.msa_ratio > 0.12;
  f.too_long = uni::length(reply) > 1200;
  return f;
}

}  // namespace gbh
