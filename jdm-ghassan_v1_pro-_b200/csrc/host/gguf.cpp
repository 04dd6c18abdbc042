// GGUF v3 container: writer and reader.  Layout (little-endian): magic "GGUF", u32 version, u64 tensor count,
// u64 metadata count, metadata entries {string key, u32 type, value} sorted by key, tensor infos {string name,
// u32 n_dims, u64 dims (fastest first), u32 ggml type, u64 offset}, zero padding to 32 bytes, tensor payloads each
// padded to 32 bytes.  Tensor types written: F32 (0), F16 (1), Q4_0 (2), Q8_0 (8).  Files written here are
// byte-identical to the reference writer's for the same inputs (format/gguf_codec.cpp:60-520): same key order (a
// sorted map), same value types, same rounding in the f16 / Q8_0 / Q4_0 encoders, same padding.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdio>
#include <filesystem>
#include <fstream>
#include <map>

#include "core.hpp"
#include "quant.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {

constexpr u32 kMagic = 0x46554747u, kVersion = 3;
enum GgufType : u32 { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };
enum GgmlType : u32 { G_F32 = 0, G_F16 = 1, G_Q4_0 = 2, G_Q8_0 = 8 };
constexpr u64 kAlign = 32;

u64 align_up(u64 x) { return (x + kAlign - 1) / kAlign * kAlign; }

u64 ggml_nbytes(u32 type, u64 n) {
  switch (type) {
    case G_F32: return n * 4;
    case G_F16: return n * 2;
    case G_Q8_0: return (n + 31) / 32 * 34;
    case G_Q4_0: return (n + 31) / 32 * 18;
  }
  fail("gguf: unsupported tensor type " + std::to_string(type));
}

std::vector<u8> encode_tensor(const float* src, u64 n, u32 type) {
  std::vector<u8> out(ggml_nbytes(type, n));
  switch (type) {
    case G_F32: std::memcpy(out.data(), src, n * 4); break;
    case G_F16: {
      u16* d = reinterpret_cast<u16*>(out.data());
      for (u64 i = 0; i < n; ++i) d[i] = f32_to_f16(src[i]);
      break;
    }
    case G_Q8_0: quant::ggml_quantize_q8_0(src, out.data(), static_cast<i64>(n)); break;
    case G_Q4_0: quant::ggml_quantize_q4_0(src, out.data(), static_cast<i64>(n)); break;
  }
  return out;
}

void decode_tensor(const u8* src, u64 n, u32 type, float* dst) {
  switch (type) {
    case G_F32: std::memcpy(dst, src, n * 4); return;
    case G_F16: {
      const u16* s = reinterpret_cast<const u16*>(src);
      for (u64 i = 0; i < n; ++i) dst[i] = f16_to_f32(s[i]);
      return;
    }
    case G_Q8_0: quant::ggml_dequantize_q8_0(src, dst, static_cast<i64>(n)); return;
    case G_Q4_0: quant::ggml_dequantize_q4_0(src, dst, static_cast<i64>(n)); return;
  }
  fail("gguf: cannot decode tensor type " + std::to_string(type));
}

struct MetaValue {
  u32 type = T_STR;
  std::vector<u8> data;   // encoded value (for strings: u64 length + bytes; arrays: u32 elem type, u64 count, items)
};

template <typename T>
void push(std::vector<u8>& v, const T& x) {
  const u8* p = reinterpret_cast<const u8*>(&x);
  v.insert(v.end(), p, p + sizeof(T));
}
void push_str(std::vector<u8>& v, const std::string& s) {
  push<u64>(v, s.size());
  v.insert(v.end(), s.begin(), s.end());
}

class GgufWriter {
 public:
  void set_str(const std::string& k, const std::string& s) { MetaValue m; m.type = T_STR; push_str(m.data, s); meta_[k] = std::move(m); }
  void set_u32(const std::string& k, u32 x) { MetaValue m; m.type = T_U32; push(m.data, x); meta_[k] = std::move(m); }
  void set_u64(const std::string& k, u64 x) { MetaValue m; m.type = T_U64; push(m.data, x); meta_[k] = std::move(m); }
  void set_f32(const std::string& k, float x) { MetaValue m; m.type = T_F32; push(m.data, x); meta_[k] = std::move(m); }
  void set_bool(const std::string& k, bool x) { MetaValue m; m.type = T_BOOL; m.data.push_back(x ? 1 : 0); meta_[k] = std::move(m); }
  void set_str_array(const std::string& k, const std::vector<std::string>& items) {
    MetaValue m; m.type = T_ARR;
    push<u32>(m.data, T_STR);
    push<u64>(m.data, items.size());
    for (const auto& s : items) push_str(m.data, s);
    meta_[k] = std::move(m);
  }
  template <typename T>
  void set_pod_array(const std::string& k, u32 elem_type, const T* p, size_t n) {
    MetaValue m; m.type = T_ARR;
    push<u32>(m.data, elem_type);
    push<u64>(m.data, n);
    const u8* b = reinterpret_cast<const u8*>(p);
    m.data.insert(m.data.end(), b, b + n * sizeof(T));
    meta_[k] = std::move(m);
  }
  void add_tensor(const std::string& name, std::vector<u64> shape, std::vector<float> data, u32 type) {
    u64 n = 1;
    for (u64 d : shape) n *= d;
    GBH_CHECK(n == data.size(), "gguf: tensor '" + name + "' shape does not match its data");
    ggml_nbytes(type, n);
    tensors_.push_back(Tensor{name, std::move(shape), std::move(data), type});
  }
  size_t tensor_count() const { return tensors_.size(); }
  size_t metadata_count() const { return meta_.size(); }

  void write(const std::string& path) const {
    namespace fs = std::filesystem;
    const fs::path p(path);
    if (p.has_parent_path()) fs::create_directories(p.parent_path());
    const std::string tmp = path + ".tmp";
    {
      std::ofstream f(tmp, std::ios::binary);
      GBH_CHECK(f.good(), "gguf: cannot open for write: " + tmp);
      std::vector<u8> head;
      push<u32>(head, kMagic);
      push<u32>(head, kVersion);
      push<u64>(head, tensors_.size());
      push<u64>(head, meta_.size());
      for (const auto& kv : meta_) {   // std::map: ascending byte order of the keys
        push_str(head, kv.first);
        push<u32>(head, kv.second.type);
        head.insert(head.end(), kv.second.data.begin(), kv.second.data.end());
      }
      u64 offset = 0;
      for (const auto& t : tensors_) {
        push_str(head, t.name);
        push<u32>(head, static_cast<u32>(t.shape.size()));
        for (auto it = t.shape.rbegin(); it != t.shape.rend(); ++it) push<u64>(head, *it);   // fastest dimension first
        push<u32>(head, t.type);
        push<u64>(head, offset);
        offset = align_up(offset + ggml_nbytes(t.type, t.data.size()));
      }
      head.resize(align_up(head.size()), 0);
      f.write(reinterpret_cast<const char*>(head.data()), static_cast<std::streamsize>(head.size()));
      for (const auto& t : tensors_) {
        std::vector<u8> payload = encode_tensor(t.data.data(), t.data.size(), t.type);
        payload.resize(align_up(payload.size()), 0);
        f.write(reinterpret_cast<const char*>(payload.data()), static_cast<std::streamsize>(payload.size()));
      }
      f.flush();
      GBH_CHECK(f.good(), "gguf: write failed: " + tmp);
    }
    std::error_code ec;
    fs::rename(tmp, path, ec);
    GBH_CHECK(!ec, "gguf: cannot finalise file: " + ec.message());
  }

 private:
  struct Tensor {
    std::string name;
    std::vector<u64> shape;   // row-major, slowest first
    std::vector<float> data;
    u32 type;
  };
  std::map<std::string, MetaValue> meta_;
  std::vector<Tensor> tensors_;
};

// ------------------------------------------------------------------ reader
struct Cursor {
  const u8* p;
  size_t n, at = 0;
  template <typename T>
  T get() {
    GBH_CHECK(at + sizeof(T) <= n, "gguf: unexpected end of file");
    T v;
    std::memcpy(&v, p + at, sizeof(T));
    at += sizeof(T);
    return v;
  }
  std::string str() {
    const u64 len = get<u64>();
    GBH_CHECK(len <= n - at, "gguf: string runs past the end of the file");
    std::string s(reinterpret_cast<const char*>(p + at), len);
    at += len;
    return s;
  }
};

py::object read_scalar(Cursor& c, u32 type) {
  switch (type) {
    case T_U8: return py::int_(c.get<u8>());
    case T_I8: return py::int_(c.get<i8>());
    case T_U16: return py::int_(c.get<u16>());
    case T_I16: return py::int_(c.get<int16_t>());
    case T_U32: return py::int_(c.get<u32>());
    case T_I32: return py::int_(c.get<i32>());
    case T_F32: return py::float_(c.get<float>());
    case T_BOOL: return py::bool_(c.get<u8>() != 0);
    case T_STR: return py::bytes(c.str());
    case T_U64: return py::int_(c.get<u64>());
    case T_I64: return py::int_(c.get<i64>());
    case T_F64: return py::float_(c.get<double>());
  }
  fail("gguf: unknown metadata type " + std::to_string(type));
}

size_t pod_size(u32 type) {
  switch (type) {
    case T_U8: case T_I8: case T_BOOL: return 1;
    case T_U16: case T_I16: return 2;
    case T_U32: case T_I32: case T_F32: return 4;
    case T_U64: case T_I64: case T_F64: return 8;
  }
  return 0;
}

py::object read_value(Cursor& c, u32 type) {
  if (type != T_ARR) return read_scalar(c, type);
  const u32 et = c.get<u32>();
  const u64 count = c.get<u64>();
  GBH_CHECK(count <= (1ull << 31), "gguf: absurd array length");
  if (et == T_U8) {   // byte blobs come back as bytes
    GBH_CHECK(count <= c.n - c.at, "gguf: array runs past the end of the file");
    py::bytes b(reinterpret_cast<const char*>(c.p + c.at), count);
    c.at += count;
    return std::move(b);
  }
  if (const size_t sz = pod_size(et); sz && et != T_BOOL) {
    GBH_CHECK(count * sz <= c.n - c.at, "gguf: array runs past the end of the file");
    py::object arr;
    auto fill = [&](auto tag) {
      using T = decltype(tag);
      py::array_t<T> a(static_cast<py::ssize_t>(count));
      std::memcpy(a.mutable_data(), c.p + c.at, count * sizeof(T));
      arr = std::move(a);
    };
    switch (et) {
      case T_I8: fill(i8{}); break;
      case T_U16: fill(u16{}); break;
      case T_I16: fill(int16_t{}); break;
      case T_U32: fill(u32{}); break;
      case T_I32: fill(i32{}); break;
      case T_F32: fill(float{}); break;
      case T_U64: fill(u64{}); break;
      case T_I64: fill(i64{}); break;
      case T_F64: fill(double{}); break;
    }
    c.at += count * sz;
    return arr;
  }
  py::list out;
  for (u64 i = 0; i < count; ++i) out.append(read_value(c, et));
  return std::move(out);
}

std::vector<u8> slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  GBH_CHECK(f.good(), "gguf: cannot open " + path);
  f.seekg(0, std::ios::end);
  const std::streamsize sz = f.tellg();
  f.seekg(0, std::ios::beg);
  std::vector<u8> buf(static_cast<size_t>(sz));
  GBH_CHECK(sz == 0 || static_cast<bool>(f.read(reinterpret_cast<char*>(buf.data()), sz)), "gguf: cannot read " + path);
  return buf;
}

// Parsed file held in memory: metadata as Python objects, tensors decodable on demand.
class GgufFile {
 public:
  explicit GgufFile(const std::string& path) : buf_(slurp(path)) {
    Cursor c{buf_.data(), buf_.size()};
    GBH_CHECK(c.get<u32>() == kMagic, "gguf: bad magic in " + path);
    version_ = c.get<u32>();
    GBH_CHECK(version_ == 2 || version_ == 3, "gguf: unsupported version " + std::to_string(version_));
    const u64 nt = c.get<u64>(), nk = c.get<u64>();
    GBH_CHECK(nt <= 100000 && nk <= 100000, "gguf: absurd header counts");
    for (u64 i = 0; i < nk; ++i) {
      std::string key = c.str();
      const u32 type = c.get<u32>();
      meta_[py::str(key)] = read_value(c, type);
    }
    for (u64 i = 0; i < nt; ++i) {
      Info t;
      t.name = c.str();
      const u32 nd = c.get<u32>();
      GBH_CHECK(nd <= 8, "gguf: too many tensor dimensions");
      std::vector<u64> dims(nd);
      for (auto& d : dims) d = c.get<u64>();
      t.shape.assign(dims.rbegin(), dims.rend());
      t.type = c.get<u32>();
      t.offset = c.get<u64>();
      t.numel = 1;
      for (u64 d : t.shape) t.numel *= d;
      t.nbytes = ggml_nbytes(t.type, t.numel);
      infos_.push_back(std::move(t));
    }
    data_start_ = align_up(c.at);
    for (const auto& t : infos_)
      GBH_CHECK(data_start_ + t.offset + t.nbytes <= buf_.size(), "gguf: tensor '" + t.name + "' runs past the end of the file");
  }
  py::dict metadata() const { return meta_; }
  u32 version() const { return version_; }
  py::list tensors() const {
    py::list out;
    for (const auto& t : infos_) {
      py::dict d;
      d["name"] = t.name;
      d["shape"] = t.shape;
      d["type"] = t.type;
      d["offset"] = t.offset;
      d["nbytes"] = t.nbytes;
      out.append(d);
    }
    return out;
  }
  py::array_t<float> tensor_f32(const std::string& name) const {
    const auto& t = info(name);
    std::vector<py::ssize_t> shape(t.shape.begin(), t.shape.end());
    py::array_t<float> a(shape);
    decode_tensor(buf_.data() + data_start_ + t.offset, t.numel, t.type, a.mutable_data());
    return a;
  }
  py::bytes tensor_raw(const std::string& name) const {
    const auto& t = info(name);
    return py::bytes(reinterpret_cast<const char*>(buf_.data() + data_start_ + t.offset), t.nbytes);
  }
  u64 data_start() const { return data_start_; }

 private:
  struct Info {
    std::string name;
    std::vector<u64> shape;
    u32 type = 0;
    u64 offset = 0, numel = 0, nbytes = 0;
  };
  const Info& info(const std::string& name) const {
    for (const auto& t : infos_)
      if (t.name == name) return t;
    fail("gguf: no tensor named '" + name + "'");
  }
  std::vector<u8> buf_;
  u32 version_ = 0;
  py::dict meta_;
  std::vector<Info> infos_;
  u64 data_start_ = 0;
};

}  // namespace

void bind_gguf(py::module_& m) {
  using farr = py::array_t<float, py::array::c_style | py::array::forcecast>;
  py::class_<GgufWriter>(m, "GgufWriter")
      .def(py::init<>())
      .def("set_str", [](GgufWriter& w, const std::string& k, const py::bytes& v) { w.set_str(k, std::string(v)); })
      .def("set_u32", &GgufWriter::set_u32)
      .def("set_u64", &GgufWriter::set_u64)
      .def("set_f32", &GgufWriter::set_f32)
      .def("set_bool", &GgufWriter::set_bool)
      .def("set_str_array", [](GgufWriter& w, const std::string& k, const std::vector<py::bytes>& items) {
        std::vector<std::string> v(items.begin(), items.end());
        w.set_str_array(k, v);
      })
      .def("set_f32_array", [](GgufWriter& w, const std::string& k, farr a) { w.set_pod_array<float>(k, T_F32, a.data(), a.size()); })
      .def("set_i32_array", [](GgufWriter& w, const std::string& k, py::array_t<i32, py::array::c_style | py::array::forcecast> a) {
        w.set_pod_array<i32>(k, T_I32, a.data(), a.size());
      })
      .def("set_u8_array", [](GgufWriter& w, const std::string& k, const py::bytes& b) {
        const std::string s(b);
        w.set_pod_array<u8>(k, T_U8, reinterpret_cast<const u8*>(s.data()), s.size());
      })
      .def("add_tensor", [](GgufWriter& w, const std::string& name, farr a, u32 type) {
        std::vector<u64> shape;
        for (py::ssize_t i = 0; i < a.ndim(); ++i) shape.push_back(static_cast<u64>(a.shape(i)));
        w.add_tensor(name, std::move(shape), std::vector<float>(a.data(), a.data() + a.size()), type);
      })
      .def_property_readonly("tensor_count", &GgufWriter::tensor_count)
      .def_property_readonly("metadata_count", &GgufWriter::metadata_count)
      .def("write", &GgufWriter::write, py::call_guard<py::gil_scoped_release>());
  py::class_<GgufFile>(m, "GgufFile")
      .def(py::init<const std::string&>())
      .def_property_readonly("version", &GgufFile::version)
      .def_property_readonly("metadata", &GgufFile::metadata)
      .def_property_readonly("tensors", &GgufFile::tensors)
      .def_property_readonly("data_start", &GgufFile::data_start)
      .def("tensor_f32", &GgufFile::tensor_f32)
      .def("tensor_raw", &GgufFile::tensor_raw);
  m.def("ggml_tensor_nbytes", &ggml_nbytes);
}
