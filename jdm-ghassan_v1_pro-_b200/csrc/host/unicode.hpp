// UTF-8 codec and the character classes the tokenizer and the text pipeline are built on: Arabic letters,
// diacritics, presentation forms, Arabic-Indic digits, Latin letters (incl. Latin-1 / Extended-A/B), emoji
// blocks, punctuation, the digits used as letters in Arabizi.  The class boundaries are part of the tokenizer
// contract (a different boundary changes token ids), so they equal the reference's (core/unicode.cpp:5-285);
// they are expressed here as sorted range tables.
#pragma once
#include <string>
#include <vector>

#include "core.hpp"

namespace gbh {
namespace uni {

struct Range { u32 lo, hi; };

template <size_t N>
constexpr bool in_ranges(const Range (&t)[N], u32 cp) {
  for (size_t i = 0; i < N; ++i)
    if (cp >= t[i].lo && cp <= t[i].hi) return true;
  return false;
}

// ------------------------------------------------------------------ UTF-8
inline int seq_len(u8 b) { return b < 0x80 ? 1 : (b & 0xE0) == 0xC0 ? 2 : (b & 0xF0) == 0xE0 ? 3 : (b & 0xF8) == 0xF0 ? 4 : 0; }

// Decode one scalar value at s[i]; malformed input yields U+FFFD and advances by one byte.
inline u32 decode(const std::string& s, size_t& i) {
  if (i >= s.size()) return 0;
  const u8 b0 = static_cast<u8>(s[i]);
  const int len = seq_len(b0);
  if (!len || i + static_cast<size_t>(len) > s.size()) { ++i; return 0xFFFD; }
  static const u8 lead_mask[5] = {0, 0x7F, 0x1F, 0x0F, 0x07};
  u32 cp = b0 & lead_mask[len];
  for (int k = 1; k < len; ++k) {
    const u8 c = static_cast<u8>(s[i + k]);
    if ((c & 0xC0) != 0x80) { ++i; return 0xFFFD; }
    cp = (cp << 6) | (c & 0x3F);
  }
  static const u32 min_for_len[5] = {0, 0, 0x80, 0x800, 0x10000};
  if (cp < min_for_len[len] || (cp >= 0xD800 && cp <= 0xDFFF) || cp > 0x10FFFF) { ++i; return 0xFFFD; }
  i += static_cast<size_t>(len);
  return cp;
}
inline void encode(u32 cp, std::string& out) {
  if (cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) cp = 0xFFFD;
  if (cp < 0x80) out.push_back(static_cast<char>(cp));
  else if (cp < 0x800) { out.push_back(char(0xC0 | (cp >> 6))); out.push_back(char(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) {
    out.push_back(char(0xE0 | (cp >> 12))); out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F)));
  } else {
    out.push_back(char(0xF0 | (cp >> 18))); out.push_back(char(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F)));
  }
}
inline std::vector<u32> to_cps(const std::string& s) {
  std::vector<u32> v;
  v.reserve(s.size());
  for (size_t i = 0; i < s.size();) v.push_back(decode(s, i));
  return v;
}
inline std::string from_cps(const std::vector<u32>& v) {
  std::string s;
  s.reserve(v.size() * 2);
  for (u32 c : v) encode(c, s);
  return s;
}
inline size_t length(const std::string& s) {
  size_t n = 0;
  for (size_t i = 0; i < s.size(); ++n) decode(s, i);
  return n;
}
// valid = decodes without replacement characters other than a literal U+FFFD in the input
inline bool valid(const std::string& s) {
  for (size_t i = 0; i < s.size();) {
    const size_t at = i;
    if (decode(s, i) == 0xFFFD &&
        !(s.size() - at >= 3 && u8(s[at]) == 0xEF && u8(s[at + 1]) == 0xBF && u8(s[at + 2]) == 0xBD))
      return false;
  }
  return true;
}
// complete = no sequence is cut off at the end and every continuation byte is well formed
inline bool complete(const std::string& s) {
  for (size_t i = 0; i < s.size();) {
    const int len = seq_len(static_cast<u8>(s[i]));
    if (!len || i + static_cast<size_t>(len) > s.size()) return false;
    for (int k = 1; k < len; ++k)
      if ((static_cast<u8>(s[i + k]) & 0xC0) != 0x80) return false;
    i += static_cast<size_t>(len);
  }
  return true;
}

// ------------------------------------------------------------------ classes
inline bool is_arabic_letter(u32 c) {
  constexpr Range t[] = {{0x0620, 0x063F}, {0x0641, 0x064A}, {0x066E, 0x06D3}, {0x06FA, 0x06FF}, {0x0750, 0x077F}, {0x08A0, 0x08BF}};
  return in_ranges(t, c);
}
inline bool is_arabic_diacritic(u32 c) {
  constexpr Range t[] = {{0x064B, 0x065F}, {0x0670, 0x0670}, {0x06D6, 0x06ED}, {0x08D3, 0x08FF}};
  return in_ranges(t, c);
}
inline bool is_arabic_punct(u32 c) {
  constexpr Range t[] = {{0x0600, 0x0600}, {0x060C, 0x060C}, {0x061B, 0x061B}, {0x061E, 0x061F}, {0x066A, 0x066D}, {0x06D4, 0x06D4}};
  return in_ranges(t, c);
}
inline bool is_arabic_digit(u32 c) { return (c >= 0x0660 && c <= 0x0669) || (c >= 0x06F0 && c <= 0x06F9); }
inline bool is_tatweel(u32 c) { return c == 0x0640; }
inline bool is_latin_letter(u32 c) {
  if ((c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z')) return true;
  return c >= 0x00C0 && c <= 0x024F && c != 0x00D7 && c != 0x00F7;
}
inline bool is_ascii_digit(u32 c) { return c >= '0' && c <= '9'; }
inline bool is_whitespace(u32 c) {
  constexpr Range t[] = {{0x09, 0x0D}, {0x20, 0x20}, {0xA0, 0xA0}, {0x1680, 0x1680}, {0x2000, 0x200A}, {0x2028, 0x2029},
                         {0x202F, 0x202F}, {0x205F, 0x205F}, {0x3000, 0x3000}};
  return in_ranges(t, c);
}
inline bool is_control(u32 c) { return (c < 0x20 && c != '\n' && c != '\t' && c != '\r') || (c >= 0x7F && c <= 0x9F); }
inline bool is_zero_width(u32 c) {
  constexpr Range t[] = {{0x200B, 0x200F}, {0x202A, 0x202E}, {0x2066, 0x2069}, {0xFEFF, 0xFEFF}};
  return in_ranges(t, c);
}
inline bool is_punct(u32 c) {
  if (c < 0x80) return (c >= '!' && c <= '/') || (c >= ':' && c <= '@') || (c >= '[' && c <= '`') || (c >= '{' && c <= '~');
  return is_arabic_punct(c) || (c >= 0x2010 && c <= 0x205E) || (c >= 0x00A1 && c <= 0x00BF);
}
inline bool is_emoji(u32 c) {
  constexpr Range t[] = {{0x203C, 0x203C}, {0x2049, 0x2049}, {0x2190, 0x21FF}, {0x2600, 0x27BF}, {0xFE00, 0xFE0F},
                         {0x1F000, 0x1F2FF}, {0x1F300, 0x1FAFF}};
  return in_ranges(t, c);
}
// digits that stand for Arabic letters in Latin-script Darija ("3", "7", "9", ...)
inline bool is_arabizi_digit(u32 c) { return c == '2' || c == '3' || (c >= '5' && c <= '9'); }

// ------------------------------------------------------------------ foldings
// isolated / final / initial / medial presentation forms (U+FE80..U+FEF4) -> base letter; 0 = not a form
inline u32 presentation_to_base(u32 c) {
  // number of presentation forms of each base letter starting at U+FE80, in code-point order
  static const struct { u32 base; u8 forms; } seq[] = {
      {0x0621, 1}, {0x0622, 2}, {0x0623, 2}, {0x0624, 2}, {0x0625, 2}, {0x0626, 4}, {0x0627, 2}, {0x0628, 4}, {0x0629, 2},
      {0x062A, 4}, {0x062B, 4}, {0x062C, 4}, {0x062D, 4}, {0x062E, 4}, {0x062F, 2}, {0x0630, 2}, {0x0631, 2}, {0x0632, 2},
      {0x0633, 4}, {0x0634, 4}, {0x0635, 4}, {0x0636, 4}, {0x0637, 4}, {0x0638, 4}, {0x0639, 4}, {0x063A, 4}, {0x0641, 4},
      {0x0642, 4}, {0x0643, 4}, {0x0644, 4}, {0x0645, 4}, {0x0646, 4}, {0x0647, 4}, {0x0648, 2}, {0x0649, 2}, {0x064A, 4}};
  if (c >= 0xFE80 && c <= 0xFEF4) {
    u32 at = 0xFE80;
    for (const auto& e : seq) {
      if (c < at + e.forms) return e.base;
      at += e.forms;
    }
  }
  if (c >= 0xFEF5 && c <= 0xFEFC) return 0x0644;  // lam-alef ligatures (expanded by the normaliser)
  return 0;
}
inline u32 arabic_digit_to_ascii(u32 c) {
  if (c >= 0x0660 && c <= 0x0669) return '0' + (c - 0x0660);
  if (c >= 0x06F0 && c <= 0x06F9) return '0' + (c - 0x06F0);
  return c;
}
// alef variants -> alef, alef maqsura -> ya, ta marbuta -> ha, hamza carriers -> hamza
inline u32 fold_arabic_letter(u32 c) {
  switch (c) {
    case 0x0622: case 0x0623: case 0x0625: case 0x0671: return 0x0627;
    case 0x0649: return 0x064A;
    case 0x0629: return 0x0647;
    case 0x0624: case 0x0626: return 0x0621;
  }
  return c;
}
inline u32 lower_latin(u32 c) {
  if (c >= 'A' && c <= 'Z') return c + 32;
  if (c >= 0x00C0 && c <= 0x00DE && c != 0x00D7) return c + 32;
  return c;
}
inline u32 fold_fullwidth(u32 c) { return (c >= 0xFF01 && c <= 0xFF5E) ? c - 0xFEE0 : (c == 0x3000 ? u32(' ') : c); }
inline std::string to_lower(const std::string& s) {
  std::string out;
  out.reserve(s.size());
  for (size_t i = 0; i < s.size();) encode(lower_latin(decode(s, i)), out);
  return out;
}

struct ScriptStats { size_t total = 0, arabic = 0, latin = 0, digits = 0, punct = 0, emoji = 0, whitespace = 0, other = 0; };
inline ScriptStats script_stats(const std::string& s) {
  ScriptStats st;
  for (size_t i = 0; i < s.size();) {
    const u32 c = decode(s, i);
    ++st.total;
    if (is_whitespace(c)) ++st.whitespace;
    else if (is_arabic_letter(c) || is_arabic_diacritic(c)) ++st.arabic;
    else if (is_latin_letter(c)) ++st.latin;
    else if (is_ascii_digit(c) || is_arabic_digit(c)) ++st.digits;
    else if (is_emoji(c)) ++st.emoji;
    else if (is_punct(c)) ++st.punct;
    else ++st.other;
  }
  return st;
}

}  // namespace uni
}  // namespace gbh
