// Python bindings of the text-pipeline primitives (dataset.hpp).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "dataset.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {
py::dict pii_dict(const PiiReport& r) {
  py::dict d;
  d["emails"] = r.emails;
  d["phones"] = r.phones;
  d["urls_with_creds"] = r.urls_with_creds;
  d["ibans"] = r.ibans;
  d["cards"] = r.cards;
  d["api_keys"] = r.api_keys;
  d["ids"] = r.ids;
  d["ips"] = r.ips;
  d["total"] = r.total();
  return d;
}
}  // namespace

void bind_dataset(py::module_& m) {
  m.def("scan_pii", [](const std::string& s) { return pii_dict(scan_pii(s)); });
  m.def("redact_pii", [](const std::string& s) {
    PiiReport r;
    std::string out = redact_pii(s, &r);
    return py::make_tuple(out, pii_dict(r));
  });
  m.def("strip_html_tags", &strip_html_tags);
  m.def("fix_mojibake", &fix_mojibake);

  py::class_<CleanConfig>(m, "CleanConfig")
      .def(py::init<>())
      .def_readwrite("strip_html", &CleanConfig::strip_html)
      .def_readwrite("fix_mojibake", &CleanConfig::fix_mojibake)
      .def_readwrite("drop_pii_lines", &CleanConfig::drop_pii_lines)
      .def_readwrite("redact_instead_drop", &CleanConfig::redact_instead_drop)
      .def_readwrite("min_chars", &CleanConfig::min_chars)
      .def_readwrite("max_chars", &CleanConfig::max_chars)
      .def_readwrite("normalizer", &CleanConfig::normalizer);
  py::class_<CleanStats>(m, "CleanStats")
      .def(py::init<>())
      .def_readonly("lines_in", &CleanStats::lines_in)
      .def_readonly("lines_out", &CleanStats::lines_out)
      .def_readonly("dropped_empty", &CleanStats::dropped_empty)
      .def_readonly("dropped_short", &CleanStats::dropped_short)
      .def_readonly("dropped_long", &CleanStats::dropped_long)
      .def_readonly("dropped_pii", &CleanStats::dropped_pii)
      .def_readonly("dropped_encoding", &CleanStats::dropped_encoding)
      .def_readonly("dropped_quality", &CleanStats::dropped_quality)
      .def_readonly("bytes_in", &CleanStats::bytes_in)
      .def_readonly("bytes_out", &CleanStats::bytes_out);
  py::class_<Cleaner>(m, "Cleaner")
      .def(py::init<CleanConfig>(), py::arg("config") = CleanConfig{})
      .def("clean_line", [](const Cleaner& c, const py::bytes& in, CleanStats& st) -> py::object {
        std::string out;
        if (!c.clean_line(std::string(in), out, st)) return py::none();
        return py::str(out);
      });

  py::class_<QualityConfig>(m, "QualityConfig")
      .def(py::init<>())
      .def_readwrite("max_symbol_ratio", &QualityConfig::max_symbol_ratio)
      .def_readwrite("max_digit_ratio", &QualityConfig::max_digit_ratio)
      .def_readwrite("max_upper_ratio", &QualityConfig::max_upper_ratio)
      .def_readwrite("max_word_repeat", &QualityConfig::max_word_repeat)
      .def_readwrite("max_repeat_line", &QualityConfig::max_repeat_line)
      .def_readwrite("min_letter_ratio", &QualityConfig::min_letter_ratio)
      .def_readwrite("min_words", &QualityConfig::min_words)
      .def_readwrite("max_word_length", &QualityConfig::max_word_length)
      .def_readwrite("require_arabic_or_latin", &QualityConfig::require_arabic_or_latin)
      .def_readwrite("reject_ai_disclaimers", &QualityConfig::reject_ai_disclaimers)
      .def_readwrite("reject_placeholders", &QualityConfig::reject_placeholders);
  m.def("english_quality_config", &english_quality_config);
  m.def("quality_check", [](const std::string& s, const QualityConfig& c) {
    const QualityVerdict v = quality_check(s, c);
    return py::make_tuple(v.accept, v.reason);
  }, py::arg("text"), py::arg("config") = QualityConfig{});
  m.def("quality_check_english", [](const std::string& s, const QualityConfig& c) {
    const QualityVerdict v = quality_check_english(s, c);
    return py::make_tuple(v.accept, v.reason);
  }, py::arg("text"), py::arg("config") = QualityConfig{});
  m.def("check_toxicity", [](const std::string& s) {
    const ToxicityResult r = check_toxicity(s);
    py::dict d;
    d["toxic"] = r.toxic;
    d["hits"] = r.hits;
    d["categories"] = r.categories;
    return d;
  });

  py::class_<Deduplicator::Config>(m, "DedupConfig")
      .def(py::init<>())
      .def_readwrite("exact", &Deduplicator::Config::exact)
      .def_readwrite("near", &Deduplicator::Config::near)
      .def_readwrite("num_hashes", &Deduplicator::Config::num_hashes)
      .def_readwrite("bands", &Deduplicator::Config::bands)
      .def_readwrite("shingle", &Deduplicator::Config::shingle)
      .def_readwrite("jaccard_threshold", &Deduplicator::Config::jaccard_threshold)
      .def_readwrite("seed", &Deduplicator::Config::seed);
  py::class_<Deduplicator>(m, "Deduplicator")
      .def(py::init<>())
      .def(py::init<const Deduplicator::Config&>())
      .def("add", &Deduplicator::add)
      .def("is_duplicate", &Deduplicator::is_duplicate)
      .def("add_blocklist_text", &Deduplicator::add_blocklist_text)
      .def_property_readonly("seen", &Deduplicator::seen)
      .def_property_readonly("exact_dups", &Deduplicator::exact_dups)
      .def_property_readonly("near_dups", &Deduplicator::near_dups)
      .def_property_readonly("blocked", &Deduplicator::blocked);

  m.def("classify_language", [](const std::string& s) {
    const LangScore r = classify_language(s);
    py::dict d;
    d["tag"] = std::string(lang_name(r.tag));
    d["confidence"] = r.confidence;
    d["darija_score"] = r.darija_score;
    d["msa_score"] = r.msa_score;
    d["french_score"] = r.french_score;
    d["english_score"] = r.english_score;
    d["arabizi_score"] = r.arabizi_score;
    d["arabic_ratio"] = r.arabic_ratio;
    d["latin_ratio"] = r.latin_ratio;
    return d;
  });
  m.def("msa_ratio", &msa_ratio);
  m.def("has_hard_ai_boilerplate", &has_hard_ai_boilerplate);
  m.def("check_assistant_style", [](const std::string& reply, const std::string& user) {
    const StyleFlags f = check_assistant_style(reply, user);
    py::dict d;
    d["robotic"] = f.robotic();
    d["has_boilerplate"] = f.has_boilerplate;
    d["excessive_msa"] = f.excessive_msa;
    d["too_many_bullets"] = f.too_many_bullets;
    d["too_long"] = f.too_long;
    d["bullet_count"] = f.bullet_count;
    d["msa_ratio"] = f.msa_ratio;
    d["matched_phrases"] = f.matched_phrases;
    return d;
  }, py::arg("reply"), py::arg("user_msg") = "");
}
