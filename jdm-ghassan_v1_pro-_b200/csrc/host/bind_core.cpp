// pybind11 bindings: random stream, hashes, 16-bit codecs, shards and the batch sampler.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "core.hpp"
#include "hostres.hpp"
#include "shards.hpp"

namespace py = pybind11;
using namespace gbh;

void bind_text(py::module_& m);      // tokenizer, normaliser, chat template, BPE trainer
void bind_formats(py::module_& m);   // checkpoint, GGUF, GAI, quantisers
void bind_sampler(py::module_& m);   // host sampler reference
void bind_dataset(py::module_& m);   // cleaner, dedup, langid, retrieval
void bind_synth(py::module_& m);     // synthetic dialogue generators

template <typename T>
using arr = py::array_t<T, py::array::c_style | py::array::forcecast>;

static py::tuple rng_get_state(const Rng& r) {
  const RngState& s = r.state();
  return py::make_tuple(py::make_tuple(s.s[0], s.s[1], s.s[2], s.s[3]), s.spare, s.has_spare);
}
static void rng_set_state(Rng& r, py::tuple t) {
  RngState s;
  py::tuple w = t[0].cast<py::tuple>();
  for (int i = 0; i < 4; ++i) s.s[i] = w[i].cast<u64>();
  s.spare = t[1].cast<float>();
  s.has_spare = t[2].cast<bool>();
  r.set_state(s);
}

PYBIND11_MODULE(_gb200_host, m) {
  m.doc() = "host-native runtime of the framework (C++20)";
  py::register_exception<Error>(m, "HostError", PyExc_RuntimeError);

  py::class_<Rng>(m, "Rng")
      .def(py::init<u64>(), py::arg("seed") = 1234567891011ULL)
      .def("reseed", &Rng::reseed)
      .def("next_u64", &Rng::next_u64)
      .def("next_u32", &Rng::next_u32)
      .def("uniform", &Rng::uniform)
      .def("below", &Rng::below)
      .def("normal", &Rng::normal, py::arg("mean") = 0.f, py::arg("stddev") = 1.f)
      .def("truncated_normal", &Rng::truncated_normal)
      .def("get_state", &rng_get_state)
      .def("set_state", &rng_set_state)
      .def("fill_truncated_normal",
           [](Rng& r, py::array_t<float, py::array::c_style> out, float stddev) {
             auto buf = out.mutable_unchecked<1>();
             const py::ssize_t n = buf.shape(0);
             float* p = buf.mutable_data(0);
             py::gil_scoped_release rel;
             for (py::ssize_t i = 0; i < n; ++i) p[i] = r.truncated_normal(stddev);
           },
           "fill a flat float32 array sequentially from the stream")
      .def("fill_uniform_ids",
           [](Rng& r, py::array_t<i32, py::array::c_style> out, u64 n_vocab) {
             auto buf = out.mutable_unchecked<1>();
             i32* p = buf.mutable_data(0);
             for (py::ssize_t i = 0; i < buf.shape(0); ++i) p[i] = static_cast<i32>(r.below(n_vocab));
           });

  m.def("fnv1a64", [](py::bytes b) {
    std::string s = b;
    return fnv1a64(s.data(), s.size());
  });
  m.def("splitmix64", &splitmix64);
  m.def("physical_ram_bytes", &physical_ram_bytes);
  m.def("free_disk_bytes", &free_disk_bytes);
  m.def("tree_size_bytes", [](const std::string& root, const std::vector<std::string>& skip) {
    const TreeSize t = tree_size_bytes(root, skip);
    return py::make_tuple(t.bytes, t.unique_files);
  }, py::arg("root"), py::arg("skip_dirs") = std::vector<std::string>());
  m.def("fingerprint_file", &fingerprint_file);
  m.def("fingerprint_hex", &fingerprint_hex);

  m.def("f32_to_f16_bits", [](arr<float> a) {
    py::array_t<u16> out(a.size());
    const float* s = a.data();
    u16* d = out.mutable_data();
    for (py::ssize_t i = 0; i < a.size(); ++i) d[i] = f32_to_f16(s[i]);
    return out;
  });
  m.def("f16_bits_to_f32", [](arr<u16> a) {
    py::array_t<float> out(a.size());
    const u16* s = a.data();
    float* d = out.mutable_data();
    for (py::ssize_t i = 0; i < a.size(); ++i) d[i] = f16_to_f32(s[i]);
    return out;
  });
  m.def("f32_to_bf16_bits", [](arr<float> a) {
    py::array_t<u16> out(a.size());
    const float* s = a.data();
    u16* d = out.mutable_data();
    for (py::ssize_t i = 0; i < a.size(); ++i) d[i] = f32_to_bf16(s[i]);
    return out;
  });
  m.def("bf16_bits_to_f32", [](arr<u16> a) {
    py::array_t<float> out(a.size());
    const u16* s = a.data();
    float* d = out.mutable_data();
    for (py::ssize_t i = 0; i < a.size(); ++i) d[i] = bf16_to_f32(s[i]);
    return out;
  });

  // ------------------------------------------------------------------ shards
  py::class_<ShardWriter>(m, "ShardWriter")
      .def(py::init<std::string, int, bool>(), py::arg("path"), py::arg("vocab_size"), py::arg("with_mask"))
      .def("add_document",
           [](ShardWriter& w, arr<i32> toks, py::object mask) {
             if (mask.is_none()) {
               w.add_document(toks.data(), static_cast<size_t>(toks.size()), nullptr);
             } else {
               arr<u8> mk = mask.cast<arr<u8>>();
               GBH_CHECK(mk.size() == toks.size(),
                         sfmt("loss mask length %zu != token length %zu", size_t(mk.size()), size_t(toks.size())));
               w.add_document(toks.data(), static_cast<size_t>(toks.size()), mk.data());
             }
           },
           py::arg("tokens"), py::arg("mask") = py::none())
      .def("close", &ShardWriter::close)
      .def_property_readonly("token_count", &ShardWriter::token_count)
      .def_property_readonly("doc_count", &ShardWriter::doc_count);

  py::class_<ShardFile>(m, "ShardFile")
      .def(py::init<>())
      .def("open",
           [](ShardFile& s, const std::string& p) {
             std::string why;
             bool ok = s.open(p, &why);
             return py::make_tuple(ok, why);
           })
      .def_property_readonly("n_tokens", &ShardFile::n_tokens)
      .def_property_readonly("n_docs", &ShardFile::n_docs)
      .def_property_readonly("has_mask", &ShardFile::has_mask)
      .def("token", [](const ShardFile& s, u64 i) { GBH_CHECK(i < s.n_tokens(), "token index out of range"); return s.token(i); })
      .def("mask", [](const ShardFile& s, u64 i) { GBH_CHECK(i < s.n_tokens(), "mask index out of range"); return int(s.mask(i)); })
      .def("doc_start", &ShardFile::doc_start)
      .def("doc_end_after", &ShardFile::doc_end_after)
      .def("tokens",
           [](const ShardFile& s, u64 start, u64 n) {
             GBH_CHECK(start <= s.n_tokens() && n <= s.n_tokens() - start, "window out of range");
             py::array_t<i32> out(static_cast<py::ssize_t>(n));
             i32* d = out.mutable_data();
             for (u64 i = 0; i < n; ++i) d[i] = s.token(start + i);
             return out;
           })
      .def("masks", [](const ShardFile& s, u64 start, u64 n) {
        GBH_CHECK(start <= s.n_tokens() && n <= s.n_tokens() - start, "window out of range");
        py::array_t<u8> out(static_cast<py::ssize_t>(n));
        u8* d = out.mutable_data();
        for (u64 i = 0; i < n; ++i) d[i] = s.mask(start + i);
        return out;
      });

  m.def("list_shards", &list_shards);

  py::class_<BatchSampler>(m, "BatchSampler")
      .def(py::init<>())
      .def("open", &BatchSampler::open, py::arg("paths"), py::arg("batch"), py::arg("seq"), py::arg("pack"),
           py::arg("seed"))
      .def("open_glob", &BatchSampler::open_glob)
      .def("open_mix", &BatchSampler::open_mix)
      .def("set_vocab", &BatchSampler::set_vocab)
      .def("next",
           [](BatchSampler& s, py::array_t<i32, py::array::c_style> ids, py::array_t<i32, py::array::c_style> tgt,
              py::array_t<i32, py::array::c_style> seg) {
             const py::ssize_t n = py::ssize_t(s.batch()) * s.seq();
             GBH_CHECK(ids.size() == n && tgt.size() == n && seg.size() == n, "batch buffers have the wrong size");
             BatchOut o{ids.mutable_data(), tgt.mutable_data(), seg.mutable_data(), 0};
             {
               py::gil_scoped_release rel;
               s.next(o);
             }
             return o.supervised;
           },
           "fill [B*T] int32 buffers in place; returns the number of supervised positions")
      .def("fast_forward", &BatchSampler::fast_forward)
      .def("reseed", &BatchSampler::reseed)
      .def("get_state",
           [](const BatchSampler& s) {
             SamplerState st = s.state();
             return py::make_tuple(py::make_tuple(st.rng[0], st.rng[1], st.rng[2], st.rng[3]), st.batches,
                                   st.rng_spare, st.rng_has_spare);
           })
      .def("set_state",
           [](BatchSampler& s, py::tuple t) {
             SamplerState st;
             py::tuple w = t[0].cast<py::tuple>();
             for (int i = 0; i < 4; ++i) st.rng[i] = w[i].cast<u64>();
             st.batches = t[1].cast<i64>();
             st.rng_spare = t[2].cast<float>();
             st.rng_has_spare = t[3].cast<i32>();
             s.set_state(st);
           })
      .def_property_readonly("total_tokens", &BatchSampler::total_tokens)
      .def_property_readonly("num_shards", &BatchSampler::num_shards)
      .def_property_readonly("batches_seen", &BatchSampler::batches_seen)
      .def_property_readonly("using_mix", &BatchSampler::using_mix)
      .def_property_readonly("all_have_mask", &BatchSampler::all_have_mask)
      .def("mix_report", &BatchSampler::mix_report);

  bind_text(m);
  bind_formats(m);
  bind_sampler(m);
  bind_dataset(m);
  bind_synth(m);
}
