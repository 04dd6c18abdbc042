// Python bindings of the text stack (normaliser, pre-tokeniser, tokenizer, streaming detokeniser, BPE trainer).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "text.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {

NormalizerConfig ncfg_from(const py::object& o) {
  if (o.is_none()) return NormalizerConfig{};
  if (py::isinstance<py::int_>(o)) return NormalizerConfig::unpack(o.cast<u32>());
  return o.cast<NormalizerConfig>();
}

py::array_t<i32> ids_array(const std::vector<i32>& v) {
  py::array_t<i32> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(i32));
  return a;
}

// token bytes are not always valid UTF-8 on their own (a character may span tokens): hand them over as bytes
py::bytes as_bytes(const std::string& s) { return py::bytes(s); }

}  // namespace

void bind_text(py::module_& m) {
  py::class_<NormalizerConfig>(m, "NormalizerConfig")
      .def(py::init<>())
      .def_readwrite("strip_diacritics", &NormalizerConfig::strip_diacritics)
      .def_readwrite("strip_tatweel", &NormalizerConfig::strip_tatweel)
      .def_readwrite("unify_presentation", &NormalizerConfig::unify_presentation)
      .def_readwrite("arabic_digits_ascii", &NormalizerConfig::arabic_digits_ascii)
      .def_readwrite("fold_letters", &NormalizerConfig::fold_letters)
      .def_readwrite("lowercase_latin", &NormalizerConfig::lowercase_latin)
      .def_readwrite("collapse_whitespace", &NormalizerConfig::collapse_whitespace)
      .def_readwrite("strip_control", &NormalizerConfig::strip_control)
      .def_readwrite("strip_zero_width", &NormalizerConfig::strip_zero_width)
      .def_readwrite("collapse_repeats", &NormalizerConfig::collapse_repeats)
      .def_readwrite("fold_fullwidth", &NormalizerConfig::fold_fullwidth)
      .def_readwrite("max_repeat", &NormalizerConfig::max_repeat)
      .def("pack", &NormalizerConfig::pack)
      .def_static("unpack", &NormalizerConfig::unpack);

  m.def("normalize", [](const std::string& text, const py::object& cfg) { return normalize(ncfg_from(cfg), text); },
        py::arg("text"), py::arg("config") = py::none());
  m.def("canonical_text", &canonical_text);
  m.def("pre_tokenize", [](const std::string& text) {
    py::list out;
    for (const Chunk& c : pre_tokenize(text)) out.append(py::make_tuple(c.text, static_cast<int>(c.kind)));
    return out;
  });
  m.def("special_tokens", [] { return special_token_strings(); });
  m.def("script_stats", [](const std::string& s) {
    const auto st = uni::script_stats(s);
    py::dict d;
    d["total"] = st.total;
    d["arabic"] = st.arabic;
    d["latin"] = st.latin;
    d["digits"] = st.digits;
    d["punct"] = st.punct;
    d["emoji"] = st.emoji;
    d["whitespace"] = st.whitespace;
    d["other"] = st.other;
    return d;
  });
  m.def("utf8_valid", [](const py::bytes& b) { return uni::valid(std::string(b)); });
  m.def("utf8_length", [](const std::string& s) { return uni::length(s); });

  py::class_<Tokenizer> tok(m, "Tokenizer");
  tok.def(py::init<>())
      .def("init_empty", [](Tokenizer& t, const py::object& cfg) { t.init_empty(ncfg_from(cfg)); },
           py::arg("config") = py::none())
      .def("build",
           [](Tokenizer& t, const std::vector<py::bytes>& vocab, const std::vector<std::pair<py::bytes, py::bytes>>& merges,
              const py::object& cfg) {
             std::vector<std::string> v(vocab.begin(), vocab.end());
             std::vector<std::pair<std::string, std::string>> mm;
             mm.reserve(merges.size());
             for (const auto& p : merges) mm.emplace_back(std::string(p.first), std::string(p.second));
             t.build(std::move(v), mm, ncfg_from(cfg));
           },
           py::arg("vocab"), py::arg("merges"), py::arg("config") = py::none())
      .def("load", &Tokenizer::load)
      .def("load_bytes", [](Tokenizer& t, const py::bytes& b) { return t.load_bytes(std::string(b)); })
      .def("save", &Tokenizer::save)
      .def("to_bytes", [](const Tokenizer& t) { return as_bytes(t.to_bytes()); })
      .def("encode",
           [](const Tokenizer& t, const std::string& text, bool bos, bool eos) { return ids_array(t.encode(text, bos, eos)); },
           py::arg("text"), py::arg("add_bos") = false, py::arg("add_eos") = false)
      .def("encode_with_specials",
           [](const Tokenizer& t, const std::string& text) { return ids_array(t.encode_with_specials(text)); })
      .def("encode_batch",
           [](const Tokenizer& t, const std::vector<std::string>& texts, bool bos, bool eos, int threads) {
             std::vector<std::vector<i32>> res;
             {
               py::gil_scoped_release nogil;
               res = t.encode_batch(texts, bos, eos, threads);
             }
             py::list out;
             for (const auto& v : res) out.append(ids_array(v));
             return out;
           },
           py::arg("texts"), py::arg("add_bos") = false, py::arg("add_eos") = false, py::arg("threads") = 0)
      .def("decode_bytes",
           [](const Tokenizer& t, const std::vector<i32>& ids, bool skip) { return as_bytes(t.decode(ids, skip)); },
           py::arg("ids"), py::arg("skip_special") = false)
      .def("decode",
           [](const Tokenizer& t, const std::vector<i32>& ids, bool skip) {
             const std::string s = t.decode(ids, skip);
             return py::reinterpret_steal<py::str>(PyUnicode_DecodeUTF8(s.data(), static_cast<py::ssize_t>(s.size()), "replace"));
           },
           py::arg("ids"), py::arg("skip_special") = false)
      .def_property_readonly("vocab_size", &Tokenizer::vocab_size)
      .def_property_readonly("merge_count", &Tokenizer::merge_count)
      .def_property_readonly("normalizer_bits", [](const Tokenizer& t) { return t.normalizer_config().pack(); })
      .def_property_readonly("normalizer_config", [](const Tokenizer& t) { return t.normalizer_config(); })
      .def("token_bytes", [](const Tokenizer& t, i32 id) { return as_bytes(t.token_text(id)); })
      .def("token_to_id", [](const Tokenizer& t, const py::bytes& b) { return t.token_to_id(std::string(b)); })
      .def("is_special", &Tokenizer::is_special)
      .def("vocab_bytes",
           [](const Tokenizer& t) {
             py::list out;
             for (const auto& s : t.vocab()) out.append(as_bytes(s));
             return out;
           })
      .def("merges",
           [](const Tokenizer& t) {
             py::list out;
             for (const auto& p : t.merges_in_rank_order()) out.append(py::make_tuple(as_bytes(p.first), as_bytes(p.second)));
             return out;
           })
      .def("measure", [](const Tokenizer& t, const std::vector<std::string>& lines) {
        const auto f = t.measure(lines);
        py::dict d;
        d["tokens_per_word"] = f.tokens_per_word;
        d["bytes_per_token"] = f.bytes_per_token;
        d["tokens"] = f.tokens;
        d["words"] = f.words;
        d["bytes"] = f.bytes;
        return d;
      });

  py::class_<Tokenizer::Stream>(m, "TokenStream")
      .def(py::init<const Tokenizer&>(), py::keep_alive<1, 2>())
      .def("push", [](Tokenizer::Stream& s, i32 id) { return as_bytes(s.push(id)); })
      .def("flush", [](Tokenizer::Stream& s) { return as_bytes(s.flush()); });

  py::class_<BpeTrainerConfig>(m, "BpeTrainerConfig")
      .def(py::init<>())
      .def_readwrite("vocab_size", &BpeTrainerConfig::vocab_size)
      .def_readwrite("min_frequency", &BpeTrainerConfig::min_frequency)
      .def_readwrite("max_token_bytes", &BpeTrainerConfig::max_token_bytes)
      .def_readwrite("normalizer", &BpeTrainerConfig::normalizer);

  py::class_<BpeTrainer>(m, "BpeTrainer")
      .def(py::init<BpeTrainerConfig>())
      .def("add_text", &BpeTrainer::add_text)
      .def("add_file", &BpeTrainer::add_file, py::call_guard<py::gil_scoped_release>())
      .def("add_chunk_counts", &BpeTrainer::add_chunk_counts)
      .def("train", &BpeTrainer::train, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("unique_chunks", &BpeTrainer::unique_chunks)
      .def_property_readonly("total_chunks", &BpeTrainer::total_chunks)
      .def_property_readonly("merges_done", &BpeTrainer::merges_done);
}
