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
  for (int i = 0; i < cfg_.num_hashes; ++i) seeds_.push_back((s = splitmix64(s)) | 1ull);
  bands_.resize(static_cast<size_t>(cfg_.bands));
}

std::vector<u64> Deduplicator::signature(const std::string& canonical) const {
  // Shingles of `shingle` consecutive WORDS (single-space joined), one FNV hash each, re-mixed per permutation.
  // Word shingles, not character ones: two template answers that differ in a few words share most character
  // 5-grams but few word 5-grams, and only the second is a near-duplicate by the reference's measure
  // (dataset/dedup.cpp:40-62).  A text shorter than one shingle hashes as a single short shingle.
  std::vector<std::pair<size_t, size_t>> words;   // [lo, hi) byte ranges
  for (size_t i = 0, lo = std::string::npos; i <= canonical.size();) {
    const size_t at = i;
    const bool end = i >= canonical.size();
    const u32 c = end ? ' ' : uni::decode(canonical, i);
    if (end) ++i;
    if (uni::is_whitespace(c)) {
      if (lo != std::string::npos) words.emplace_back(lo, at);
      lo = std::string::npos;
    } else if (lo == std::string::npos) {
      lo = at;
    }
  }
  std::vector<u64> sig(static_cast<size_t>(cfg_.num_hashes), ~0ull);
  if (words.empty()) return sig;
  const size_t k = static_cast<size_t>(cfg_.shingle);
  const size_t n_sh = words.size() >= k ? words.size() - k + 1 : 1;
  std::string sh;
  for (size_t i = 0; i < n_sh; ++i) {
    sh.clear();
    for (size_t j = i; j < std::min(words.size(), i + k); ++j) {
      if (j > i) sh.push_back(' ');
      sh.append(canonical, words[j].first, words[j].second - words[j].first);
    }
    const u64 h = fnv1a64(sh.data(), sh.size());
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
      "والو", "شي", "هضر", "دير", "كندير", "كنهضر", "معاك", "ليا", "ليك", "لينا",
      // pronouns, demonstratives, connectives
      "نتا", "نتي", "نتوما", "حنا", "هوما", "هادي", "هادو", "هاداك", "هاديك", "داك", "ديك", "داكشي", "ولا", "غير", "بلا", "بصح",
      "زعما", "واقيلا", "فاش", "ملي", "منين", "عاد", "بعدا", "باقي", "واخا", "يالاه", "يلاه", "دبا", "دروك", "لبارح", "غدا", "شوية",
      "بشوية", "دغيا", "بالزاف", "كولشي", "حتا", "معا", "معايا", "فيا", "فيك", "عندي", "عندك", "عندو", "عندنا",
      // verbs and negated forms as they are written apart
      "بغا", "بغينا", "بغيتي", "خاصني", "خاصك", "خاص", "مشيت", "مشا", "جيت", "جا", "شفت", "شوف", "عرفت", "كنعرف", "سير", "اجي",
      "گلس", "نوض", "خدام", "خدامة", "عرفتش", "بغيتش", "كاينش", "قدرتش", "فهمتش", "والله", "عفاك", "سمح", "سمحلي",
      // everyday nouns and adjectives
      "زوين", "زوينة", "مزيانة", "خايب", "دار", "الدار", "خدمة", "فلوس", "دراهم", "اتاي", "طاجين", "صاحبي", "ختي", "ولد", "بنت", "الواليد",
      "الواليدة", "بخير", "لاباس", "الحمدلله", "تبارك", "بسلامة"};
  static const std::unordered_set<std::string> darija_lat = {
      "wach", "bzaf", "bzzaf", "dyal", "daba", "kifach", "3lach", "chno", "fin", "ghadi", "kayn", "machi", "hadchi", "had",
      "dyali", "dyalk", "bghit", "kidayr", "mzyan", "khoya", "safi", "ch7al", "3afak", "b7al", "7it", "rah", "bach", "ga3",
      "walo", "chi", "hder", "dir", "m3a", "m3ak", "lik", "salam", "labas", "wakha", "3la", "ana", "nta", "nti",
      "ntoma", "7na", "homa", "hadi", "hado", "hadak", "dak", "dik", "dakchi", "wla", "ghir", "bla", "bsa7", "z3ma", "fach", "mli", "mnin",
      "3ad", "ba9i", "yallah", "db", "drok", "lbar7", "ghda", "chwiya", "bchwiya", "dghya", "kolchi", "7ta", "m3aya", "fia", "fik", "3ndi",
      "3ndk", "3ndo", "3ndna", "bgha", "bghina", "bghiti", "khasni", "khask", "khass", "mchit", "mcha", "jit", "ja", "cheft", "chouf",
      "3reft", "kan3ref", "sir", "aji", "gls", "nod", "khdam", "khdama", "ma3reftch", "mabghitch", "makaynch", "wallah", "sm7", "sm7li",
      "zwin", "zwina", "mzyana", "khayb", "dar", "khdma", "flous", "drahm", "atay", "tajine", "sa7bi", "khti", "wld", "bnt", "lwalid",
      "lwalida", "bikhir", "hamdollah", "hamdulillah", "tbarkllah", "bslama", "nhar", "lyoum", "souk", "bzef", "kifash", "3lash", "fin", "chkoun"};
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

// Script first, word evidence second, with the reference classifier's decision procedure and thresholds
// (dataset/langid.cpp:132-250 there), over this library's own word lists:
//   * the text is letter-folded; a script "dominates" above 60 % of the letters;
//   * words are runs of Arabic letters, Latin letters and the digits Arabizi uses as letters (2 3 5 6 7 8 9), ASCII
//     lower-cased; a word counts as Arabic when its first letter is;
//   * Arabic words: Darija list, Standard-Arabic list, and the verb shapes of Darija (a word of three or more letters that
//     opens with ki- / ka- counts, and one that opens with ki- / ka- / ta- / gha- / ma- and ends in -sh counts);
//     Latin words: Darija, French and English lists, and "Arabizi" = letters and such a digit in one word;
//   * densities are taken over the words of the script; Arabic-dominant text is Darija from a density of 0.06 or two hits,
//     otherwise Standard Arabic (confidently from a density of 0.10); Latin-dominant text goes through the
//     Darija / French / English cascade below and is "other" without evidence; neither dominant = mixed.
LangScore classify_language(const std::string& raw) {
  LangScore r;
  if (raw.empty()) return r;
  NormalizerConfig nc;
  nc.fold_letters = true;
  const std::string text = normalize(nc, raw);
  const uni::ScriptStats st = uni::script_stats(text);
  const double letters = static_cast<double>(st.arabic + st.latin);
  if (letters < 1) return r;
  r.arabic_ratio = st.arabic / letters;
  r.latin_ratio = st.latin / letters;

  std::vector<std::string> ws;
  {
    std::string cur;
    for (size_t i = 0; i < text.size();) {
      u32 c = uni::decode(text, i);
      if (uni::is_arabic_letter(c) || uni::is_latin_letter(c) || uni::is_arabizi_digit(c)) {
        if (c >= 'A' && c <= 'Z') c += 32;
        uni::encode(c, cur);
      } else if (!cur.empty()) {
        ws.push_back(std::move(cur));
        cur.clear();
      }
    }
    if (!cur.empty()) ws.push_back(std::move(cur));
  }
  if (ws.empty()) return r;

  auto starts = [](const std::string& w, const char* pre) { return w.rfind(pre, 0) == 0; };
  double dar_ar = 0, dar_lt = 0, msa = 0, fr = 0, en = 0, arabizi = 0, ar_words = 0, lt_words = 0;
  for (const auto& w : ws) {
    size_t at = 0;
    const bool is_ar = uni::is_arabic_letter(uni::decode(w, at));
    if (is_ar) {
      ++ar_words;
      dar_ar += lexicon(0).count(w);
      msa += lexicon(2).count(w);
      if (w.size() >= 6) {                                  // three Arabic letters or more
        const bool kik = starts(w, "كي") || starts(w, "كا");
        if (kik || starts(w, "تا") || starts(w, "غا") || starts(w, "ما")) {
          if (w.size() >= 4 && w.compare(w.size() - 2, 2, "ش") == 0) ++dar_ar;
          else if (kik) ++dar_ar;
        }
      }
    } else {
      ++lt_words;
      dar_lt += lexicon(1).count(w);
      fr += lexicon(3).count(w);
      en += lexicon(4).count(w);
      bool letter = false, digit = false;
      for (size_t q = 0; q < w.size();) {
        const u32 c = uni::decode(w, q);
        letter |= uni::is_latin_letter(c);
        digit |= uni::is_arabizi_digit(c);
      }
      if (letter && digit) ++arabizi;
    }
  }
  const double n = static_cast<double>(ws.size());
  r.darija_score = (dar_ar + dar_lt) / n;
  r.msa_score = msa / n;
  r.french_score = fr / n;
  r.english_score = en / n;
  r.arabizi_score = arabizi / n;
  const double arw = std::max(1.0, ar_words), ltw = std::max(1.0, lt_words);
  const double d_ar = dar_ar / arw, d_lt = (dar_lt + arabizi) / ltw, d_msa = msa / arw, d_fr = fr / ltw, d_en = en / ltw;

  if (r.arabic_ratio > 0.6) {
    if (d_ar >= 0.06 || dar_ar >= 2) {
      r.tag = LangTag::DarijaArab;
      r.confidence = std::min(1.0, 0.4 + d_ar * 4.0);
    } else {
      r.tag = LangTag::MSA;
      r.confidence = d_msa >= 0.10 ? std::min(1.0, 0.4 + d_msa * 3.0) : 0.3;
    }
  } else if (r.latin_ratio > 0.6) {
    const bool dar_hit = d_lt >= 0.08 || dar_lt + arabizi >= 2;
    const bool en_hit = d_en >= 0.08 || en >= 2;
    const bool fr_hit = d_fr >= 0.15;
    if (dar_hit && d_en <= d_lt) {
      r.tag = LangTag::DarijaLatn;
      r.confidence = std::min(1.0, 0.4 + d_lt * 4.0);
    } else if (fr_hit && d_fr > d_en && d_fr >= d_lt) {
      r.tag = LangTag::French;
      r.confidence = std::min(1.0, 0.35 + d_fr * 2.0);
    } else if (en_hit && d_en >= d_lt) {
      r.tag = LangTag::English;
      r.confidence = std::min(1.0, 0.35 + d_en * 2.0);
    } else if (dar_hit) {
      r.tag = LangTag::DarijaLatn;
      r.confidence = std::min(1.0, 0.4 + d_lt * 4.0);
    } else {
      r.tag = LangTag::Other;
      r.confidence = 0.2;
    }
  } else {
    r.tag = LangTag::Mixed;
    r.confidence = dar_ar + dar_lt + arabizi >= 1 ? 0.6 : 0.35;
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
