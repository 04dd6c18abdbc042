// Cleaner, PII scanner, quality gate and toxicity lexicon (see dataset.hpp).
#include <algorithm>
#include <cctype>
#include <sstream>

#include "dataset.hpp"

namespace gbh {

namespace {

inline bool is_digit(char c) { return c >= '0' && c <= '9'; }
inline bool is_alpha(char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z'); }
inline bool is_alnum(char c) { return is_digit(c) || is_alpha(c); }
inline bool is_local_char(char c) { return is_alnum(c) || c == '.' || c == '_' || c == '-' || c == '+'; }

std::string lower_ascii(std::string s) {
  for (char& c : s)
    if (c >= 'A' && c <= 'Z') c = static_cast<char>(c + 32);
  return s;
}

bool luhn_ok(const std::string& digits) {
  int sum = 0;
  bool dbl = false;
  for (size_t i = digits.size(); i-- > 0;) {
    int d = digits[i] - '0';
    if (dbl) {
      d *= 2;
      if (d > 9) d -= 9;
    }
    sum += d;
    dbl = !dbl;
  }
  return sum % 10 == 0;
}

struct Span {
  size_t lo, hi;
  const char* tag;
  int PiiReport::*field;
};

// Every scanner appends non-overlapping spans; the caller sorts and merges.
void find_emails(const std::string& s, std::vector<Span>& out) {
  for (size_t at = s.find('@'); at != std::string::npos; at = s.find('@', at + 1)) {
    size_t lo = at, hi = at + 1;
    while (lo > 0 && is_local_char(s[lo - 1])) --lo;
    bool dot = false;
    while (hi < s.size() && (is_alnum(s[hi]) || s[hi] == '.' || s[hi] == '-')) {
      dot |= s[hi] == '.';
      ++hi;
    }
    while (hi > at + 1 && (s[hi - 1] == '.' || s[hi - 1] == '-')) --hi;
    if (lo < at && hi > at + 3 && dot) out.push_back({lo, hi, "<EMAIL>", &PiiReport::emails});
  }
}

void find_urls_with_credentials(const std::string& s, std::vector<Span>& out) {
  for (size_t p = s.find("://"); p != std::string::npos; p = s.find("://", p + 3)) {
    size_t end = p + 3;
    while (end < s.size() && !std::isspace(static_cast<unsigned char>(s[end]))) ++end;
    const size_t at = s.find('@', p + 3), slash = s.find('/', p + 3);
    if (at != std::string::npos && at < end && (slash == std::string::npos || at < slash) &&
        s.find(':', p + 3) < at) {
      size_t lo = p;
      while (lo > 0 && is_alpha(s[lo - 1])) --lo;
      out.push_back({lo, end, "<URL>", &PiiReport::urls_with_creds});
    }
  }
}

// digit runs with separators: phones (8..15 digits, optional +), cards (13..19 digits, Luhn), IPv4
void find_numbers(const std::string& s, std::vector<Span>& out) {
  size_t i = 0;
  while (i < s.size()) {
    if (!(is_digit(s[i]) || (s[i] == '+' && i + 1 < s.size() && is_digit(s[i + 1])))) {
      ++i;
      continue;
    }
    if (i > 0 && is_alnum(s[i - 1])) {   // inside a word or a longer token: skip the whole run
      while (i < s.size() && is_alnum(s[i])) ++i;
      continue;
    }
    size_t j = i;
    std::string digits;
    int dots = 0;
    bool other_sep = false;
    if (s[j] == '+') ++j;
    while (j < s.size()) {
      if (is_digit(s[j])) digits.push_back(s[j]);
      else if (s[j] == '.' && j + 1 < s.size() && is_digit(s[j + 1])) ++dots;
      else if ((s[j] == ' ' || s[j] == '-' || s[j] == '(' || s[j] == ')') && j + 1 < s.size() &&
               (is_digit(s[j + 1]) || s[j + 1] == '('))
        other_sep = true;
      else break;
      ++j;
    }
    const size_t n = digits.size();
    if (dots == 3 && !other_sep && n >= 4 && n <= 12) {
      // dotted quad with every part <= 255
      bool ok = true;
      int part = 0, parts = 0;
      for (size_t k = i; k <= j; ++k) {
        if (k < j && is_digit(s[k])) part = part * 10 + (s[k] - '0');
        else {
          ok &= part <= 255;
          part = 0;
          ++parts;
        }
      }
      if (ok && parts == 4) out.push_back({i, j, "<IP>", &PiiReport::ips});
    } else if (n >= 13 && n <= 19 && dots == 0 && luhn_ok(digits)) {
      out.push_back({i, j, "<CARD>", &PiiReport::cards});
    } else if (n >= 8 && n <= 15 && dots == 0 && (s[i] == '+' || other_sep || (n >= 9 && digits[0] == '0'))) {
      out.push_back({i, j, "<PHONE>", &PiiReport::phones});
    }
    i = std::max(j, i + 1);
  }
}

void find_ibans_and_keys(const std::string& s, std::vector<Span>& out) {
  size_t i = 0;
  while (i < s.size()) {
    if (!is_alnum(s[i]) || (i > 0 && (is_alnum(s[i - 1]) || s[i - 1] == '_' || s[i - 1] == '-'))) {
      ++i;
      continue;
    }
    size_t j = i;
    int digits = 0, uppers = 0, lowers = 0;
    while (j < s.size() && (is_alnum(s[j]) || s[j] == '_' || s[j] == '-')) {
      digits += is_digit(s[j]);
      uppers += s[j] >= 'A' && s[j] <= 'Z';
      lowers += s[j] >= 'a' && s[j] <= 'z';
      ++j;
    }
    const size_t n = j - i;
    const bool iban = n >= 15 && n <= 34 && s[i] >= 'A' && s[i] <= 'Z' && s[i + 1] >= 'A' && s[i + 1] <= 'Z' &&
                      is_digit(s[i + 2]) && is_digit(s[i + 3]) && lowers == 0 && digits >= 10;
    const std::string head = lower_ascii(s.substr(i, std::min<size_t>(8, n)));
    const bool prefixed = head.rfind("sk-", 0) == 0 || head.rfind("ghp_", 0) == 0 || head.rfind("akia", 0) == 0 ||
                          head.rfind("xoxb-", 0) == 0 || head.rfind("aiza", 0) == 0;
    const bool key = (prefixed && n >= 20) || (n >= 32 && digits >= 6 && uppers + lowers >= 10 && (uppers > 0) + (lowers > 0) + (digits > 0) >= 2 &&
                                               s.substr(i, n).find('-') == std::string::npos);
    if (iban) out.push_back({i, j, "<IBAN>", &PiiReport::ibans});
    else if (key) out.push_back({i, j, "<KEY>", &PiiReport::api_keys});
    i = j;
  }
}

std::vector<Span> all_spans(const std::string& s) {
  std::vector<Span> v;
  find_urls_with_credentials(s, v);
  find_emails(s, v);
  find_ibans_and_keys(s, v);
  find_numbers(s, v);
  std::sort(v.begin(), v.end(), [](const Span& a, const Span& b) { return a.lo != b.lo ? a.lo < b.lo : a.hi > b.hi; });
  std::vector<Span> out;
  for (const auto& sp : v)
    if (out.empty() || sp.lo >= out.back().hi) out.push_back(sp);
  return out;
}

}  // namespace

PiiReport scan_pii(const std::string& text) {
  PiiReport r;
  for (const auto& sp : all_spans(text)) ++(r.*(sp.field));
  return r;
}

std::string redact_pii(const std::string& text, PiiReport* report) {
  std::string out;
  size_t at = 0;
  PiiReport r;
  for (const auto& sp : all_spans(text)) {
    out.append(text, at, sp.lo - at);
    out += sp.tag;
    at = sp.hi;
    ++(r.*(sp.field));
  }
  out.append(text, at, std::string::npos);
  if (report) *report = r;
  return out;
}

std::string strip_html_tags(const std::string& s) {
  std::string out;
  out.reserve(s.size());
  static const std::pair<const char*, const char*> entities[] = {{"&amp;", "&"}, {"&lt;", "<"}, {"&gt;", ">"},
                                                                 {"&quot;", "\""}, {"&#39;", "'"}, {"&nbsp;", " "}};
  for (size_t i = 0; i < s.size();) {
    if (s[i] == '<') {
      const size_t close = s.find('>', i + 1);
      const bool taglike = close != std::string::npos && close - i <= 200 && i + 1 < s.size() &&
                           (is_alpha(s[i + 1]) || s[i + 1] == '/' || s[i + 1] == '!');
      if (taglike) {
        out.push_back(' ');
        i = close + 1;
        continue;
      }
    }
    if (s[i] == '&') {
      bool hit = false;
      for (const auto& e : entities) {
        const size_t n = std::char_traits<char>::length(e.first);
        if (s.compare(i, n, e.first) == 0) {
          out += e.second;
          i += n;
          hit = true;
          break;
        }
      }
      if (hit) continue;
    }
    out.push_back(s[i++]);
  }
  return out;
}

std::string fix_mojibake(const std::string& s) {
  // "Ã©", "Ø§" ...: every character is in U+0080..U+00FF and the bytes they stand for form valid UTF-8
  int suspicious = 0;
  for (size_t i = 0; i + 1 < s.size(); ++i) {
    const u8 a = static_cast<u8>(s[i]), b = static_cast<u8>(s[i + 1]);
    if ((a == 0xC3 || a == 0xC2) && b >= 0x80 && b <= 0xBF) ++suspicious;
  }
  if (suspicious < 2) return s;
  std::string bytes;
  for (size_t i = 0; i < s.size();) {
    const u32 cp = uni::decode(s, i);
    if (cp > 0xFF) return s;   // a character that cannot be a mis-decoded byte: leave the text alone
    bytes.push_back(static_cast<char>(cp));
  }
  if (!uni::valid(bytes) || uni::length(bytes) >= uni::length(s)) return s;
  return bytes;
}

bool Cleaner::clean_line(const std::string& in, std::string& out, CleanStats& st) const {
  ++st.lines_in;
  st.bytes_in += in.size();
  if (!uni::valid(in)) {
    ++st.dropped_encoding;
    return false;
  }
  std::string t = in;
  if (cfg_.strip_html) t = strip_html_tags(t);
  if (cfg_.fix_mojibake) t = fix_mojibake(t);
  if (cfg_.drop_pii_lines || cfg_.redact_instead_drop) {
    PiiReport rep;
    std::string red = redact_pii(t, &rep);
    if (rep.any()) {
      if (cfg_.redact_instead_drop) t = std::move(red);
      else {
        ++st.dropped_pii;
        return false;
      }
    }
  }
  t = normalize(cfg_.normalizer, t);
  if (t.empty()) {
    ++st.dropped_empty;
    return false;
  }
  const size_t chars = uni::length(t);
  if (static_cast<int>(chars) < cfg_.min_chars) {
    ++st.dropped_short;
    return false;
  }
  if (static_cast<int>(chars) > cfg_.max_chars) {
    ++st.dropped_long;
    return false;
  }
  out = std::move(t);
  ++st.lines_out;
  st.bytes_out += out.size();
  return true;
}

// Limits for English chat text: code, tables and one-word replies are ordinary there (the reference's
// english_quality_config, dataset/cleaner.cpp:459-474 there); AI disclaimers are left to quality_check_english.
QualityConfig english_quality_config() {
  QualityConfig c;
  c.max_symbol_ratio = 0.35;
  c.max_digit_ratio = 0.50;
  c.max_upper_ratio = 0.60;
  c.max_repeat_line = 0.30;
  c.max_word_repeat = 0.40;
  c.min_letter_ratio = 0.30;
  c.min_words = 1;
  c.max_word_length = 80;
  c.reject_ai_disclaimers = false;
  return c;
}

// The reference's checks in its order, with its reasons (dataset/cleaner.cpp:351-457 there): AI disclaimers and
// unresolved placeholders first; then the character mix over ALL characters of the text (white space included): no
// content, no letters, letter / symbol / digit ratios, shouting (capitals among more than 20 Latin letters); then the
// white-space separated words: their number, the longest one, and from 8 words on the share of the most frequent word;
// last, from 5 non-empty lines on, the share of repeated lines.
QualityVerdict quality_check(const std::string& text, const QualityConfig& cfg) {
  QualityVerdict v;
  auto reject = [&](const char* why) {
    v.accept = false;
    v.reason = why;
    return v;
  };
  if (text.empty()) return reject("empty");
  if (cfg.reject_ai_disclaimers) {
    const std::string low = lower_ascii(text);
    for (const char* d : {"as an ai language model", "as a language model", "as an artificial intelligence",
                          "i don't have personal opinions", "i cannot fulfill this request", "i am an ai", "i'm an ai",
                          "i cannot provide", "i'm sorry, but i cannot", "i am a large language model"})
      if (low.find(d) != std::string::npos) return reject("ai_disclaimer");
  }
  if (cfg.reject_placeholders) {
    for (const char* ph : {"[insert ", "[Insert ", "<your_", "<YOUR_", "TODO:", "[Your Name]", "[your name]"})
      if (text.find(ph) != std::string::npos) return reject("unresolved_placeholder");
  }
  const uni::ScriptStats st = uni::script_stats(text);
  if (st.total == 0) return reject("no content");
  const size_t letters = st.arabic + st.latin;
  const double total = static_cast<double>(st.total);
  if (cfg.require_arabic_or_latin && letters == 0) return reject("no letters");
  if (letters / total < cfg.min_letter_ratio) return reject("low letter ratio");
  if ((st.punct + st.other) / total > cfg.max_symbol_ratio) return reject("symbol spam");
  if (st.digits / total > cfg.max_digit_ratio) return reject("digit spam");
  size_t upper = 0;
  for (size_t i = 0; i < text.size();) {
    const u32 c = uni::decode(text, i);
    upper += c >= 'A' && c <= 'Z';
  }
  if (st.latin > 20 && static_cast<double>(upper) / st.latin > cfg.max_upper_ratio) return reject("shouting");

  std::unordered_map<std::string, int> freq;
  size_t n_words = 0, longest = 0;
  {
    std::string cur;
    auto flush = [&]() {
      if (cur.empty()) return;
      ++n_words;
      longest = std::max(longest, uni::length(cur));
      ++freq[cur];
      cur.clear();
    };
    for (size_t i = 0; i < text.size();) {
      const size_t at = i;
      const u32 c = uni::decode(text, i);
      if (uni::is_whitespace(c)) flush();
      else cur.append(text, at, i - at);
    }
    flush();
  }
  if (static_cast<int>(n_words) < cfg.min_words) return reject("too few words");
  if (static_cast<int>(longest) > cfg.max_word_length) return reject("absurd word length");
  if (n_words >= 8) {
    int top = 0;
    for (const auto& kv : freq) top = std::max(top, kv.second);
    if (static_cast<double>(top) / n_words > cfg.max_word_repeat) return reject("word repetition");
  }
  {
    std::unordered_map<std::string, int> lines;
    std::istringstream ls(text);
    int n_lines = 0;
    for (std::string line; std::getline(ls, line);) {
      if (line.empty()) continue;
      ++lines[line];
      ++n_lines;
    }
    if (n_lines >= 5) {
      int dup = 0;
      for (const auto& kv : lines) dup += kv.second > 1 ? kv.second - 1 : 0;
      if (static_cast<double>(dup) / n_lines > cfg.max_repeat_line) return reject("duplicated lines");
    }
  }
  return v;
}

QualityVerdict quality_check_english(const std::string& text, const QualityConfig& cfg) {
  QualityConfig c = cfg;
  if (c.min_words == 2 && c.min_letter_ratio == 0.45) c = english_quality_config();
  QualityVerdict v = quality_check(text, c);
  if (!v.accept) return v;
  const std::string low = lower_ascii(text);
  for (const char* ph : {"as an ai", "as a language model", "as an ai language model", "i am a large language model",
                         "i cannot fulfill this request"})
    if (low.find(ph) != std::string::npos) {
      v.accept = false;
      v.reason = "ai_disclosure_hard";
      return v;
    }
  return v;
}

ToxicityResult check_toxicity(const std::string& text) {
  // A deliberately small lexicon of unambiguous terms per category; matching is on whole canonical words.
  static const std::pair<const char*, std::vector<const char*>> lex[] = {
      {"insult", {"idiot", "stupid", "moron", "7mar", "حمار", "كلب", "connard", "imbecile"}},
      {"hate", {"subhuman", "vermin", "exterminate"}},
      {"violence", {"i will kill you", "kill yourself", "نقتلك", "ghadi n9etlek"}},
      {"sexual", {"porn", "xxx video"}},
  };
  const std::string canon = " " + canonical_text(text) + " ";
  ToxicityResult r;
  for (const auto& cat : lex) {
    bool hit = false;
    for (const char* w : cat.second) {
      const std::string needle = " " + canonical_text(w) + " ";
      const bool phrase = std::string(w).find(' ') != std::string::npos;
      if ((phrase && canon.find(canonical_text(w)) != std::string::npos) || canon.find(needle) != std::string::npos) {
        ++r.hits;
        hit = true;
      }
    }
    if (hit) r.categories.push_back(cat.first);
  }
  r.toxic = r.hits > 0;
  return r;
}

}  // namespace gbh
