// Normaliser and pre-tokeniser (see text.hpp for the contract).
#include "text.hpp"

namespace gbh {

namespace {
struct FlagBit {
  bool NormalizerConfig::*field;
  int bit;
};
const FlagBit kFlagBits[] = {
    {&NormalizerConfig::strip_diacritics, 0},   {&NormalizerConfig::strip_tatweel, 1},
    {&NormalizerConfig::unify_presentation, 2}, {&NormalizerConfig::arabic_digits_ascii, 3},
    {&NormalizerConfig::fold_letters, 4},       {&NormalizerConfig::lowercase_latin, 5},
    {&NormalizerConfig::collapse_whitespace, 6}, {&NormalizerConfig::strip_control, 7},
    {&NormalizerConfig::strip_zero_width, 8},   {&NormalizerConfig::collapse_repeats, 9},
    {&NormalizerConfig::fold_fullwidth, 10},
};
}  // namespace

u32 NormalizerConfig::pack() const {
  u32 bits = 0;
  for (const auto& f : kFlagBits)
    if (this->*(f.field)) bits |= 1u << f.bit;
  return bits | ((static_cast<u32>(max_repeat) & 0xFu) << 16);
}

NormalizerConfig NormalizerConfig::unpack(u32 bits) {
  NormalizerConfig c;
  for (const auto& f : kFlagBits) c.*(f.field) = (bits >> f.bit) & 1u;
  const int rep = static_cast<int>((bits >> 16) & 0xFu);
  c.max_repeat = rep > 0 ? rep : 3;
  return c;
}

std::string normalize(const NormalizerConfig& cfg, const std::string& text) {
  const std::vector<u32> in = uni::to_cps(text);
  std::vector<u32> out;
  out.reserve(in.size());
  const size_t n = in.size();
  const size_t rep = static_cast<size_t>(cfg.max_repeat);

  auto is_blank = [](u32 c) { return c == ' ' || c == '\n'; };

  for (size_t i = 0; i < n; ++i) {
    u32 c = in[i];
    if (cfg.strip_control && uni::is_control(c)) continue;
    if (cfg.strip_zero_width && uni::is_zero_width(c)) {
      // a zero-width non-joiner between two Arabic letters carries meaning (it blocks the ligature) and stays
      const bool zwnj_inside_word = c == 0x200C && i > 0 && i + 1 < n && uni::is_arabic_letter(in[i - 1]) &&
                                    uni::is_arabic_letter(in[i + 1]);
      if (!zwnj_inside_word) continue;
    }
    if (cfg.unify_presentation && c >= 0xFE70 && c <= 0xFEFF) {
      if (c >= 0xFEF5 && c <= 0xFEFC) {   // lam-alef ligatures expand to the two letters
        out.push_back(0x0644);
        out.push_back(0x0627);
        continue;
      }
      if (const u32 base = uni::presentation_to_base(c)) c = base;
    }
    if (cfg.strip_tatweel && uni::is_tatweel(c)) continue;
    if (cfg.strip_diacritics && uni::is_arabic_diacritic(c)) continue;
    if (cfg.arabic_digits_ascii) c = uni::arabic_digit_to_ascii(c);
    if (cfg.fold_fullwidth) c = uni::fold_fullwidth(c);
    if (cfg.fold_letters) c = uni::fold_arabic_letter(c);
    if (cfg.lowercase_latin) c = uni::lower_latin(c);

    if (uni::is_whitespace(c)) {
      const u32 ws = c == '\n' ? u32('\n') : u32(' ');
      if (cfg.collapse_whitespace && !out.empty() && is_blank(out.back())) {
        if (ws == '\n' && out.back() == ' ') out.back() = '\n';   // a run containing a newline collapses to a newline
        continue;
      }
      out.push_back(ws);
      continue;
    }
    if (cfg.collapse_repeats && out.size() >= rep) {
      bool all_same = true;
      for (size_t r = 1; r <= rep && all_same; ++r) all_same = out[out.size() - r] == c;
      if (all_same) continue;
    }
    out.push_back(c);
  }
  size_t a = 0, b = out.size();
  while (a < b && is_blank(out[a])) ++a;
  while (b > a && is_blank(out[b - 1])) --b;
  std::string res;
  res.reserve((b - a) * 2);
  for (size_t i = a; i < b; ++i) uni::encode(out[i], res);
  return res;
}

std::string canonical_text(const std::string& text) {
  NormalizerConfig c;
  c.fold_letters = true;
  c.lowercase_latin = true;
  c.collapse_repeats = true;
  c.max_repeat = 3;
  return normalize(c, text);
}

// ------------------------------------------------------------------ pre-tokeniser
namespace {

ChunkKind kind_of(u32 c) {
  if (uni::is_whitespace(c)) return ChunkKind::Space;
  if (uni::is_arabic_letter(c) || uni::is_arabic_diacritic(c)) return ChunkKind::Arabic;
  if (uni::is_latin_letter(c)) return ChunkKind::Latin;
  if (uni::is_ascii_digit(c) || uni::is_arabic_digit(c)) return ChunkKind::Number;
  if (uni::is_emoji(c)) return ChunkKind::Emoji;
  if (uni::is_punct(c)) return ChunkKind::Punct;
  return ChunkKind::Other;
}

// Cursor over the code points of one text; each take_* consumes one chunk body and appends it to `dst`.
struct Scanner {
  const std::vector<u32>& cp;
  size_t i = 0;
  explicit Scanner(const std::vector<u32>& v) : cp(v) {}
  size_t n() const { return cp.size(); }
  bool more() const { return i < cp.size(); }
  u32 cur() const { return cp[i]; }
  bool next_is(bool (*pred)(u32)) const { return i + 1 < cp.size() && pred(cp[i + 1]); }
  void emit(std::string& dst) { uni::encode(cp[i++], dst); }

  void take_arabic(std::string& dst) {
    while (more() && (uni::is_arabic_letter(cur()) || uni::is_arabic_diacritic(cur()) || cur() == 0x200C)) emit(dst);
  }
  // Latin words keep inner apostrophes ("don't") and the digits Darija writers use as letters ("3lach", "m3a")
  void take_latin(std::string& dst) {
    bool started = false;
    while (more()) {
      const u32 c = cur();
      bool ok = uni::is_latin_letter(c);
      if (!ok && (c == '\'' || c == 0x2019)) ok = started && next_is(uni::is_latin_letter);
      if (!ok && uni::is_arabizi_digit(c))
        ok = started || next_is(uni::is_latin_letter) || next_is(uni::is_arabizi_digit);
      if (!ok) break;
      emit(dst);
      started = true;
    }
    if (!started) emit(dst);
  }
  void take_number(std::string& dst) {
    while (more()) {
      const u32 c = cur();
      const bool digit = uni::is_ascii_digit(c) || uni::is_arabic_digit(c);
      const bool separator = (c == '.' || c == ',') && next_is(uni::is_ascii_digit);
      if (!digit && !separator) break;
      emit(dst);
    }
  }
  void take_punct_run(std::string& dst) {
    const u32 first = cur();
    while (more() && cur() == first) emit(dst);
  }
  void take_emoji(std::string& dst) {
    while (more() && (uni::is_emoji(cur()) || cur() == 0x200D)) emit(dst);
  }
};

}  // namespace

std::vector<Chunk> pre_tokenize(const std::string& normalized) {
  const std::vector<u32> cps = uni::to_cps(normalized);
  Scanner s(cps);
  std::vector<Chunk> out;
  while (s.more()) {
    Chunk c;
    if (uni::is_whitespace(s.cur())) {
      const size_t start = s.i;
      bool newline = false;
      while (s.more() && uni::is_whitespace(s.cur())) {
        newline |= s.cur() == '\n';
        ++s.i;
      }
      // a single plain space glues onto the word that follows; anything else is a chunk of its own
      if (newline || s.i - start > 1 || !s.more()) {
        c.kind = ChunkKind::Space;
        for (size_t k = start; k < s.i; ++k) uni::encode(cps[k], c.text);
        out.push_back(std::move(c));
        continue;
      }
      c.text = " ";
    }
    ChunkKind kind = kind_of(s.cur());
    if (kind == ChunkKind::Number && uni::is_arabizi_digit(s.cur()) && s.next_is(uni::is_latin_letter))
      kind = ChunkKind::Latin;
    c.kind = kind;
    switch (kind) {
      case ChunkKind::Arabic: s.take_arabic(c.text); break;
      case ChunkKind::Latin: s.take_latin(c.text); break;
      case ChunkKind::Number: s.take_number(c.text); break;
      case ChunkKind::Punct: s.take_punct_run(c.text); break;
      case ChunkKind::Emoji: s.take_emoji(c.text); break;
      default: s.emit(c.text); break;
    }
    out.push_back(std::move(c));
  }
  return out;
}

}  // namespace gbh
