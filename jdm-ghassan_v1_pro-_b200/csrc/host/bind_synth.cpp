// Python bindings of the synthetic dialogue generators (synth.hpp).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "synth.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {
py::dict conv_dict(const SynthConversation& c) {
  py::list msgs;
  for (const auto& m : c.messages) {
    py::dict d;
    d["role"] = m.role;
    d["content"] = m.content;
    msgs.append(d);
  }
  py::dict out;
  out["messages"] = msgs;
  out["domain"] = c.domain;
  out["script"] = c.script;
  out["template_id"] = c.template_id;
  return out;
}
py::dict stats_dict(const SynthStats& s) {
  py::dict d;
  d["attempts"] = s.attempts;
  d["accepted"] = s.accepted;
  d["rejected_duplicate"] = s.rejected_duplicate;
  d["rejected_style"] = s.rejected_style;
  d["rejected_entropy"] = s.rejected_entropy;
  d["rejected_template_cap"] = s.rejected_template_cap;
  d["by_domain"] = s.by_domain;
  d["by_script"] = s.by_script;
  d["summary"] = s.summary();
  return d;
}
}  // namespace

void bind_synth(py::module_& m) {
  m.def("arabic_to_arabizi", [](const std::string& s, u64 seed, bool heavy) {
    Rng r(seed);
    return arabic_to_arabizi(s, r, heavy);
  }, py::arg("text"), py::arg("seed") = 1, py::arg("heavy_digits") = true);
  m.def("orthographic_noise", [](const std::string& s, u64 seed, double rate) {
    Rng r(seed);
    return orthographic_noise(s, r, rate);
  }, py::arg("text"), py::arg("seed") = 1, py::arg("rate") = 0.04);
  m.def("char_entropy_bits", &char_entropy_bits);
  m.def("distinct_word_ratio", &distinct_word_ratio);
  m.def("classify_dialog_act", &classify_dialog_act);
  m.def("english_reply_fits", [](const std::string& act, const std::string& user, const std::string& reply) {
    const StyleVerdict v = english_reply_fits(act, user, reply);
    return py::make_tuple(v.ok, v.reason);
  });

  py::class_<SynthConfig>(m, "SynthConfig")
      .def(py::init<>())
      .def_readwrite("seed", &SynthConfig::seed)
      .def_readwrite("num_conversations", &SynthConfig::num_conversations)
      .def_readwrite("min_turns", &SynthConfig::min_turns)
      .def_readwrite("max_turns", &SynthConfig::max_turns)
      .def_readwrite("p_arabic_script", &SynthConfig::p_arabic_script)
      .def_readwrite("p_latin_script", &SynthConfig::p_latin_script)
      .def_readwrite("p_msa", &SynthConfig::p_msa)
      .def_readwrite("p_french_switch", &SynthConfig::p_french_switch)
      .def_readwrite("p_followup", &SynthConfig::p_followup)
      .def_readwrite("p_correction", &SynthConfig::p_correction)
      .def_readwrite("p_misunderstand", &SynthConfig::p_misunderstand)
      .def_readwrite("p_governor", &SynthConfig::p_governor)
      .def_readwrite("p_reasoning", &SynthConfig::p_reasoning)
      .def_readwrite("include_system", &SynthConfig::include_system)
      .def_readwrite("p_system", &SynthConfig::p_system)
      .def_readwrite("max_template_uses", &SynthConfig::max_template_uses)
      .def_readwrite("max_attempts_multiplier", &SynthConfig::max_attempts_multiplier)
      .def_readwrite("min_entropy_bits", &SynthConfig::min_entropy_bits)
      .def_readwrite("min_distinct_words", &SynthConfig::min_distinct_words)
      .def_readwrite("noise_rate", &SynthConfig::noise_rate)
      .def_readwrite("p_heavy_digits", &SynthConfig::p_heavy_digits);
  py::class_<DarijaSynth>(m, "DarijaSynth")
      .def(py::init<const SynthConfig&>())
      .def("generate", [](DarijaSynth& g) -> py::object {
        SynthConversation c;
        if (!g.generate(c)) return py::none();
        return conv_dict(c);
      })
      .def("generate_many", [](DarijaSynth& g, int n) {
        py::list out;
        for (const auto& c : g.generate_many(n)) out.append(conv_dict(c));
        return out;
      })
      .def("stats", [](const DarijaSynth& g) { return stats_dict(g.stats()); })
      .def_static("domains", &DarijaSynth::domains);

  py::class_<EnglishSynthConfig>(m, "EnglishSynthConfig")
      .def(py::init<>())
      .def_readwrite("seed", &EnglishSynthConfig::seed)
      .def_readwrite("min_turns", &EnglishSynthConfig::min_turns)
      .def_readwrite("max_turns", &EnglishSynthConfig::max_turns)
      .def_readwrite("p_followup", &EnglishSynthConfig::p_followup)
      .def_readwrite("p_system", &EnglishSynthConfig::p_system)
      .def_readwrite("max_template_uses", &EnglishSynthConfig::max_template_uses)
      .def_readwrite("max_attempts_multiplier", &EnglishSynthConfig::max_attempts_multiplier)
      .def_readwrite("min_entropy_bits", &EnglishSynthConfig::min_entropy_bits)
      .def_readwrite("min_distinct_words", &EnglishSynthConfig::min_distinct_words);
  py::class_<EnglishSynth>(m, "EnglishSynth")
      .def(py::init<const EnglishSynthConfig&>())
      .def("generate", [](EnglishSynth& g) -> py::object {
        SynthConversation c;
        if (!g.generate(c)) return py::none();
        return conv_dict(c);
      })
      .def("generate_many", [](EnglishSynth& g, int n) {
        py::list out;
        for (const auto& c : g.generate_many(n)) out.append(conv_dict(c));
        return out;
      })
      .def("stats", [](const EnglishSynth& g) { return stats_dict(g.stats()); })
      .def_static("acts", &EnglishSynth::acts);
}
