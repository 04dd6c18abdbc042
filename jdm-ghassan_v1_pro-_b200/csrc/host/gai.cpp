// Legacy ".gai" model container and the raw weight dump ("GRAW").
//
// .gai (format/legacy_gai_format.cpp:28-162 in the reference), little-endian:
//   u32 magic 0x31494147 ("GAI1"), u32 version 1, u32 header bytes, header = "key=value\n" lines sorted by key,
//   u64 tensor count, directory entries {u32 name length, name, u32 dtype id, u32 rank, i64 dims[rank], u64 offset,
//   u64 nbytes}, u64 tokenizer blob bytes + blob (.gtok image), then every payload at the next multiple of 64 bytes.
//   dtype ids: F32 0, F16 1, BF16 2, I32 3, I8 4, Q8_0 5 (68-byte blocks of 64), Q4_0 6, Q4_1 7, U16 8, I64 9.
// The reader maps the file (read-only) so that payloads can be handed out without copying.
//
// GRAW (model/model.cpp:1696-1798): u32 magic 0x57415247, u32 count, per tensor {u32 name length, name, u64 numel,
// u32 rank, i64 dims[rank], f32 payload}.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <filesystem>
#include <fstream>
#include <map>
#include <sstream>

#include "core.hpp"
#include "quant.hpp"

namespace py = pybind11;
using namespace gbh;

namespace {

constexpr u32 kGaiMagic = 0x31494147u, kGaiVersion = 1u, kRawMagic = 0x57415247u;
inline u64 align64(u64 x) { return (x + 63ull) & ~63ull; }

struct Entry {
  std::string name;
  u32 dtype = 0;
  std::vector<i64> dims;
  u64 offset = 0, nbytes = 0;
  i64 numel() const {
    i64 n = 1;
    for (i64 d : dims) n *= d;
    return n;
  }
};

class GaiWriter {
 public:
  void set_meta(const std::string& k, const std::string& v) { meta_[k] = v; }
  void set_tokenizer_blob(const std::string& blob) { tok_ = blob; }
  // data: fp32 values, stored as `dtype` (quantised with the internal codecs)
  void add_tensor(const std::string& name, const std::vector<i64>& dims, const float* data, i64 n, u32 dtype) {
    Entry e;
    e.name = name;
    e.dims = dims;
    GBH_CHECK(e.numel() == n, "gai: tensor '" + name + "' shape does not match its data");
    if (quant::is_quantized(dtype) && n % quant::block_size(dtype) != 0) dtype = quant::F16;   // ragged: keep 16-bit
    e.dtype = dtype;
    e.nbytes = quant::nbytes(dtype, static_cast<size_t>(n));
    std::string payload(e.nbytes, '\0');
    quant::quantize(dtype, data, payload.data(), n);
    entries_.push_back(std::move(e));
    payloads_.push_back(std::move(payload));
  }
  void write(const std::string& path) {
    namespace fs = std::filesystem;
    if (fs::path(path).has_parent_path()) fs::create_directories(fs::path(path).parent_path());
    std::string header;
    for (const auto& kv : meta_) header += kv.first + "=" + kv.second + "\n";
    // directory size is known up front, so offsets can be computed before anything is written
    u64 at = 4 + 4 + 4 + header.size() + 8;
    for (const auto& e : entries_) at += 4 + e.name.size() + 4 + 4 + 8 * e.dims.size() + 8 + 8;
    at += 8 + tok_.size();
    for (size_t i = 0; i < entries_.size(); ++i) {
      at = align64(at);
      entries_[i].offset = at;
      at += entries_[i].nbytes;
    }
    ByteWriter w;
    w.put<u32>(kGaiMagic);
    w.put<u32>(kGaiVersion);
    w.put<u32>(static_cast<u32>(header.size()));
    w.put_bytes(header.data(), header.size());
    w.put<u64>(entries_.size());
    for (const auto& e : entries_) {
      w.put_str32(e.name);
      w.put<u32>(e.dtype);
      w.put<u32>(static_cast<u32>(e.dims.size()));
      for (i64 d : e.dims) w.put<i64>(d);
      w.put<u64>(e.offset);
      w.put<u64>(e.nbytes);
    }
    w.put<u64>(tok_.size());
    w.put_bytes(tok_.data(), tok_.size());
    const std::string tmp = path + ".tmp";
    {
      std::ofstream f(tmp, std::ios::binary);
      GBH_CHECK(f.good(), "gai: cannot write " + tmp);
      f.write(reinterpret_cast<const char*>(w.buf.data()), static_cast<std::streamsize>(w.buf.size()));
      u64 pos = w.buf.size();
      for (size_t i = 0; i < entries_.size(); ++i) {
        for (; pos < entries_[i].offset; ++pos) f.put('\0');
        f.write(payloads_[i].data(), static_cast<std::streamsize>(payloads_[i].size()));
        pos += payloads_[i].size();
      }
      f.flush();
      GBH_CHECK(f.good(), "gai: write failed");
    }
    std::error_code ec;
    fs::rename(tmp, path, ec);
    GBH_CHECK(!ec, "gai: cannot finalise model file: " + ec.message());
  }
  size_t tensor_count() const { return entries_.size(); }

 private:
  std::map<std::string, std::string> meta_;
  std::string tok_;
  std::vector<Entry> entries_;
  std::vector<std::string> payloads_;
};

// Read-only mapping of a whole file.
class Mapping {
 public:
  explicit Mapping(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    GBH_CHECK(fd_ >= 0, "cannot open " + path);
    struct stat st;
    GBH_CHECK(::fstat(fd_, &st) == 0, "cannot stat " + path);
    size_ = static_cast<size_t>(st.st_size);
    if (size_ > 0) {
      void* p = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
      GBH_CHECK(p != MAP_FAILED, "cannot map " + path);
      base_ = static_cast<const u8*>(p);
    }
  }
  ~Mapping() {
    if (base_) ::munmap(const_cast<u8*>(base_), size_);
    if (fd_ >= 0) ::close(fd_);
  }
  Mapping(const Mapping&) = delete;
  Mapping& operator=(const Mapping&) = delete;
  const u8* data() const { return base_; }
  size_t size() const { return size_; }

 private:
  int fd_ = -1;
  const u8* base_ = nullptr;
  size_t size_ = 0;
};

class GaiFile {
 public:
  explicit GaiFile(const std::string& path) : map_(std::make_shared<Mapping>(path)) {
    ByteReader r(map_->data(), map_->size());
    GBH_CHECK(r.get<u32>() == kGaiMagic, "not a .gai model file: " + path);
    GBH_CHECK(r.get<u32>() == kGaiVersion, "unsupported .gai version in " + path);
    const u32 hb = r.get<u32>();
    GBH_CHECK(hb <= (1u << 22), "gai: header too large");
    std::istringstream hs(std::string(reinterpret_cast<const char*>(r.take(hb)), hb));
    for (std::string line; std::getline(hs, line);) {
      const size_t eq = line.find('=');
      if (eq != std::string::npos) meta_[line.substr(0, eq)] = line.substr(eq + 1);
    }
    const u64 count = r.get<u64>();
    GBH_CHECK(count <= 1000000ull, "gai: absurd tensor count");
    for (u64 i = 0; i < count; ++i) {
      Entry e;
      const u32 nl = r.get<u32>();
      GBH_CHECK(nl <= 4096, "gai: tensor name too long");
      e.name.assign(reinterpret_cast<const char*>(r.take(nl)), nl);
      e.dtype = r.get<u32>();
      const u32 nd = r.get<u32>();
      GBH_CHECK(nd <= 8, "gai: too many dimensions");
      e.dims.resize(nd);
      for (auto& d : e.dims) d = r.get<i64>();
      e.offset = r.get<u64>();
      e.nbytes = r.get<u64>();
      GBH_CHECK(e.nbytes <= map_->size() && e.offset <= map_->size() - e.nbytes,
                "gai: tensor range out of file bounds for " + e.name);
      GBH_CHECK(e.numel() >= 0 && quant::nbytes(e.dtype, static_cast<size_t>(e.numel())) == e.nbytes,
                "gai: tensor size mismatch for " + e.name);
      entries_.push_back(std::move(e));
    }
    const u64 tb = r.get<u64>();
    GBH_CHECK(tb < (1ull << 32), "gai: tokenizer blob too large");
    tok_.assign(reinterpret_cast<const char*>(r.take(tb)), tb);
  }
  const std::map<std::string, std::string>& meta() const { return meta_; }
  py::bytes tokenizer_blob() const { return py::bytes(tok_); }
  py::list tensors() const {
    py::list out;
    for (const auto& e : entries_) {
      py::dict d;
      d["name"] = e.name;
      d["dtype"] = e.dtype;
      d["dtype_name"] = std::string(quant::dtype_name(e.dtype));
      d["shape"] = e.dims;
      d["offset"] = e.offset;
      d["nbytes"] = e.nbytes;
      out.append(d);
    }
    return out;
  }
  const Entry& find(const std::string& name) const {
    for (const auto& e : entries_)
      if (e.name == name) return e;
    fail("tensor not found in model file: " + name);
  }
  py::array_t<float> tensor_f32(const std::string& name) const {
    const Entry& e = find(name);
    std::vector<py::ssize_t> shape(e.dims.begin(), e.dims.end());
    py::array_t<float> a(shape);
    quant::dequantize(e.dtype, map_->data() + e.offset, a.mutable_data(), e.numel());
    return a;
  }
  // zero-copy view of the stored bytes; the mapping stays alive as long as the array does
  py::array_t<u8> tensor_view(const std::string& name) const {
    const Entry& e = find(name);
    auto keep = new std::shared_ptr<Mapping>(map_);
    py::capsule owner(keep, [](void* p) { delete static_cast<std::shared_ptr<Mapping>*>(p); });
    return py::array_t<u8>({static_cast<py::ssize_t>(e.nbytes)}, {1}, map_->data() + e.offset, owner);
  }

 private:
  std::shared_ptr<Mapping> map_;
  std::map<std::string, std::string> meta_;
  std::vector<Entry> entries_;
  std::string tok_;
};

using farr = py::array_t<float, py::array::c_style | py::array::forcecast>;

void write_graw(const std::string& path, const std::vector<std::pair<std::string, farr>>& tensors) {
  std::ofstream f(path, std::ios::binary);
  GBH_CHECK(f.good(), "cannot write model: " + path);
  ByteWriter w;
  w.put<u32>(kRawMagic);
  w.put<u32>(static_cast<u32>(tensors.size()));
  f.write(reinterpret_cast<const char*>(w.buf.data()), static_cast<std::streamsize>(w.buf.size()));
  for (const auto& t : tensors) {
    ByteWriter h;
    h.put_str32(t.first);
    h.put<u64>(static_cast<u64>(t.second.size()));
    h.put<u32>(static_cast<u32>(t.second.ndim()));
    for (py::ssize_t i = 0; i < t.second.ndim(); ++i) h.put<i64>(t.second.shape(i));
    f.write(reinterpret_cast<const char*>(h.buf.data()), static_cast<std::streamsize>(h.buf.size()));
    f.write(reinterpret_cast<const char*>(t.second.data()), static_cast<std::streamsize>(t.second.size() * 4));
  }
  GBH_CHECK(f.good(), "model write failed: " + path);
}

py::list read_graw(const std::string& path) {
  Mapping m(path);
  ByteReader r(m.data(), m.size());
  GBH_CHECK(r.get<u32>() == kRawMagic, "[raw] bad magic in " + path);
  const u32 n = r.get<u32>();
  py::list out;
  for (u32 i = 0; i < n; ++i) {
    const std::string name = r.get_str32();
    const u64 numel = r.get<u64>();
    const u32 nd = r.get<u32>();
    GBH_CHECK(nd <= 8, "[raw] too many dimensions for " + name);
    std::vector<py::ssize_t> shape(nd);
    u64 prod = 1;
    for (auto& d : shape) {
      d = static_cast<py::ssize_t>(r.get<i64>());
      prod *= static_cast<u64>(d);
    }
    GBH_CHECK(prod == numel, "[raw] shape does not match element count for " + name);
    py::array_t<float> a(shape);
    std::memcpy(a.mutable_data(), r.take(numel * 4), numel * 4);
    out.append(py::make_tuple(name, a));
  }
  return out;
}

}  // namespace

void bind_gai(py::module_& m) {
  py::class_<GaiWriter>(m, "GaiWriter")
      .def(py::init<>())
      .def("set_meta", &GaiWriter::set_meta)
      .def("set_tokenizer_blob", [](GaiWriter& w, const py::bytes& b) { w.set_tokenizer_blob(std::string(b)); })
      .def("add_tensor", [](GaiWriter& w, const std::string& name, farr a, const std::string& dtype) {
        std::vector<i64> dims;
        for (py::ssize_t i = 0; i < a.ndim(); ++i) dims.push_back(a.shape(i));
        w.add_tensor(name, dims, a.data(), a.size(), quant::dtype_from_name(dtype));
      })
      .def_property_readonly("tensor_count", &GaiWriter::tensor_count)
      .def("write", &GaiWriter::write, py::call_guard<py::gil_scoped_release>());
  py::class_<GaiFile>(m, "GaiFile")
      .def(py::init<const std::string&>())
      .def_property_readonly("meta", &GaiFile::meta)
      .def_property_readonly("tensors", &GaiFile::tensors)
      .def_property_readonly("tokenizer_blob", &GaiFile::tokenizer_blob)
      .def("tensor_f32", &GaiFile::tensor_f32)
      .def("tensor_view", &GaiFile::tensor_view);
  m.def("write_graw", &write_graw);
  m.def("read_graw", &read_graw);
}
