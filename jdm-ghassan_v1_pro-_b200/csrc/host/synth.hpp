// Synthetic dialogue generators: Moroccan Darija (Arabic script, Arabizi, some MSA, French code-switching) and
// English (dialog acts with a style policy).  They fill the role of the reference's synthesis engines
// (dataset/darija_synthesis_engine.cpp:133-576, dataset/english_synthesis_engine.cpp:67-214,
// dataset/english_style_policy.cpp): same knobs and the same kinds of rejection (duplicate, template cap, style,
// entropy), with this project's own templates, transliteration rules and thresholds.  Deterministic for a seed.
#pragma once
#include <map>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "core.hpp"

namespace gbh {

// Arabic-script Darija -> Latin "Arabizi".  heavy_digits: 7 / 3 / 9 / 2 / 5 stand for the letters Latin lacks;
// otherwise each of them is sometimes spelled with letters (h, a, q, ', kh), as lighter typists do.
std::string arabic_to_arabizi(const std::string& arabic, Rng& rng, bool heavy_digits = true);
// Typing habits of chat Latin script: dropped short vowels, doubled letters, ou/o, ch/sh, q/9/k swaps, lost spaces.
std::string orthographic_noise(const std::string& latin, Rng& rng, double rate = 0.04);
// Shannon entropy (bits per code point) and share of distinct words: the two "is there any information here" measures.
double char_entropy_bits(const std::string& text);
double distinct_word_ratio(const std::string& text);

struct SynthMessage {
  std::string role, content;
};
struct SynthConversation {
  std::vector<SynthMessage> messages;
  std::string domain, script;      // script: "arab", "latn", "msa" or "en"
  u64 template_id = 0;
};

struct SynthConfig {
  u64 seed = 1234;
  int num_conversations = 20000;
  int min_turns = 2, max_turns = 10;            // messages per conversation (without the system prompt)
  double p_arabic_script = 0.60, p_latin_script = 0.30, p_msa = 0.10;
  double p_french_switch = 0.10, p_followup = 0.40, p_correction = 0.08, p_misunderstand = 0.06;
  double p_governor = 0.0, p_reasoning = 0.0;
  bool include_system = true;
  double p_system = 0.30;
  int max_template_uses = 400;
  int max_attempts_multiplier = 60;
  double min_entropy_bits = 3.2;                 // of the whole conversation text
  double min_distinct_words = 0.35;
  double noise_rate = 0.04;                      // Arabizi typing noise
  double p_heavy_digits = 0.7;
};

struct SynthStats {
  u64 attempts = 0, accepted = 0, rejected_duplicate = 0, rejected_style = 0, rejected_entropy = 0,
      rejected_template_cap = 0;
  std::map<std::string, u64> by_domain, by_script;
  std::string summary() const;
};

class DarijaSynth {
 public:
  explicit DarijaSynth(const SynthConfig& cfg);
  // One attempt: true and `out` filled when a conversation was accepted; false when it was rejected (see stats).
  bool generate(SynthConversation& out);
  // Up to n accepted conversations, giving up after n * max_attempts_multiplier attempts.
  std::vector<SynthConversation> generate_many(int n);
  const SynthStats& stats() const { return stats_; }
  static std::vector<std::string> domains();

 private:
  bool build(SynthConversation& c);
  SynthConfig cfg_;
  Rng rng_;
  SynthStats stats_;
  std::unordered_map<u64, int> uses_;
  std::unordered_set<u64> seen_;
};

// ------------------------------------------------------------------ English
// Dialog act of a user message (keyword rules) and whether a reply has the shape that act asks for.
std::string classify_dialog_act(const std::string& user_text);
struct StyleVerdict {
  bool ok = true;
  std::string reason;
};
StyleVerdict english_reply_fits(const std::string& act, const std::string& user_text, const std::string& reply);

struct EnglishSynthConfig {
  u64 seed = 4321;
  int min_turns = 2, max_turns = 6;
  double p_followup = 0.35, p_system = 0.25;
  int max_template_uses = 400;
  int max_attempts_multiplier = 60;
  double min_entropy_bits = 3.0, min_distinct_words = 0.35;
};

class EnglishSynth {
 public:
  explicit EnglishSynth(const EnglishSynthConfig& cfg);
  bool generate(SynthConversation& out);
  std::vector<SynthConversation> generate_many(int n);
  const SynthStats& stats() const { return stats_; }
  static std::vector<std::string> acts();

 private:
  EnglishSynthConfig cfg_;
  Rng rng_;
  SynthStats stats_;
  std::unordered_map<u64, int> uses_;
  std::unordered_set<u64> seen_;
};

}  // namespace gbh
