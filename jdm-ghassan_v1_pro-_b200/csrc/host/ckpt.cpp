// Training checkpoint container (.ckpt), versions 3..12, byte-compatible with the reference engine
// (training/checkpoint.cpp:13-22, 76-158, 394-468, 503-625; optimizer blobs training/optimizer.cpp).
//
// Layout of version 12 (little endian, packed):
//   u32 magic 0x54504B47 | u32 version
//   config : 7 x i32 | 6 x f32 | 4 x u8 | 3 x i32 | 2 x f32 | u8 | 2 x f32 | 2 x i32
//   state  : i64 step, tokens | f64 best_val, last_loss | u64 seed | LOADER | f64 loss_scale
//            | i32 clean_steps, tok_vocab | i64 sched_total, sched_warmup | f32 peak, min_ratio,
//            decay_frac | i32 sched_kind, ddp_world | u64 tok_fingerprint | LOADER(val)
//   LOADER : u64 rng[4] | i64 batches | f32 spare | i32 has_spare
//   bias   : u64 layers | layers x (u32 ne | f32[ne])                       (version >= 10)
//   params : u64 n | n x (u32 len | name | u64 numel | f32[numel])
//   opt    : u8 has | [u8 kind | blob]     kind 0 adamw, 1 lion, 2 muon
// This file only encodes and decodes; which differences are fatal on resume is decided by the trainer.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cmath>
#include <cstdio>
#include <filesystem>

#include "core.hpp"

namespace py = pybind11;
namespace fs = std::filesystem;
using namespace gbh;

namespace {

constexpr u32 kCkptMagic = 0x54504B47u;
constexpr u32 kCkptVersion = 12u;

struct FileSink {
  std::FILE* f = nullptr;
  std::string path;
  explicit FileSink(const std::string& p) : path(p) {
    f = std::fopen(p.c_str(), "wb");
    GBH_CHECK(f != nullptr, "cannot write checkpoint: " + p);
  }
  ~FileSink() {
    if (f) std::fclose(f);
  }
  void bytes(const void* p, size_t n) {
    if (n && std::fwrite(p, 1, n, f) != n) fail("checkpoint write failed: " + path);
  }
  template <typename T>
  void put(T v) { bytes(&v, sizeof(T)); }
  void finish() {
    GBH_CHECK(std::fflush(f) == 0, "checkpoint write failed: " + path);
    std::fclose(f);
    f = nullptr;
  }
};

template <typename T>
T item(const py::dict& d, const char* k) {
  GBH_CHECK(d.contains(k), std::string("checkpoint: missing field '") + k + "'");
  return d[k].cast<T>();
}

void put_loader(FileSink& o, const py::dict& s) {
  py::tuple rng = item<py::tuple>(s, "rng");
  for (int i = 0; i < 4; ++i) o.put<u64>(rng[i].cast<u64>());
  o.put<i64>(item<i64>(s, "batches"));
  o.put<float>(item<float>(s, "rng_spare"));
  o.put<i32>(item<i32>(s, "rng_has_spare"));
}

py::dict get_loader(ByteReader& r, bool with_spare) {
  py::dict s;
  py::tuple rng(4);
  for (int i = 0; i < 4; ++i) rng[i] = r.get<u64>();
  s["rng"] = rng;
  s["batches"] = r.get<i64>();
  s["rng_spare"] = with_spare ? r.get<float>() : 0.f;
  s["rng_has_spare"] = with_spare ? r.get<i32>() : 0;
  return s;
}

void put_config(FileSink& o, const py::dict& c) {
  for (const char* k : {"vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                        "max_seq_len"})
    o.put<i32>(item<i32>(c, k));
  for (const char* k : {"rope_theta", "rms_eps", "init_std", "moe_aux_scale", "z_loss_scale", "rope_scale"})
    o.put<float>(item<float>(c, k));
  for (const char* k : {"tie_embeddings", "use_moe", "moe_shared", "use_qk_norm"}) o.put<u8>(item<bool>(c, k) ? 1 : 0);
  for (const char* k : {"num_experts", "moe_top_k", "moe_expert_dim"}) o.put<i32>(item<i32>(c, k));
  o.put<float>(item<float>(c, "moe_jitter"));
  o.put<float>(item<float>(c, "rope_yarn_mscale"));
  o.put<u8>(item<bool>(c, "moe_aux_free") ? 1 : 0);
  o.put<float>(item<float>(c, "rope_yarn_low"));
  o.put<float>(item<float>(c, "rope_yarn_high"));
  o.put<i32>(item<i32>(c, "sliding_window"));
  o.put<i32>(item<i32>(c, "rope_type"));
}

py::dict get_config(ByteReader& r, u32 version) {
  py::dict c;
  if (version < 5) {
    // versions 3 and 4 stored the in-memory image of the configuration record (108 bytes, natural alignment)
    const u8* b = r.take(108);
    auto i32at = [&](size_t o) { i32 v; std::memcpy(&v, b + o, 4); return v; };
    auto f32at = [&](size_t o) { float v; std::memcpy(&v, b + o, 4); return v; };
    const char* ints[] = {"vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                          "max_seq_len"};
    for (int i = 0; i < 7; ++i) c[ints[i]] = i32at(4 * i);
    c["rope_theta"] = f32at(28); c["rms_eps"] = f32at(32); c["tie_embeddings"] = b[36] != 0;
    c["init_std"] = f32at(40); c["use_moe"] = b[44] != 0;
    c["num_experts"] = i32at(48); c["moe_top_k"] = i32at(52); c["moe_expert_dim"] = i32at(56);
    c["moe_shared"] = b[60] != 0; c["moe_aux_scale"] = f32at(64); c["moe_jitter"] = f32at(68);
    c["moe_allow_dense"] = b[72] != 0; c["use_qk_norm"] = b[73] != 0;
    c["z_loss_scale"] = f32at(76); c["rope_scale"] = f32at(80); c["rope_yarn_mscale"] = f32at(84);
    c["moe_aux_free"] = b[88] != 0; c["rope_yarn_low"] = f32at(92); c["rope_yarn_high"] = f32at(96);
    c["sliding_window"] = i32at(100); c["rope_type"] = i32at(104);
    return c;
  }
  for (const char* k : {"vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                        "max_seq_len"})
    c[k] = r.get<i32>();
  for (const char* k : {"rope_theta", "rms_eps", "init_std", "moe_aux_scale", "z_loss_scale", "rope_scale"})
    c[k] = r.get<float>();
  for (const char* k : {"tie_embeddings", "use_moe", "moe_shared", "use_qk_norm"}) c[k] = r.get<u8>() != 0;
  for (const char* k : {"num_experts", "moe_top_k", "moe_expert_dim"}) c[k] = r.get<i32>();
  c["moe_jitter"] = version >= 6 ? r.get<float>() : 0.f;
  c["rope_yarn_mscale"] = version >= 6 ? r.get<float>() : 0.f;
  if (version >= 9) {
    c["moe_aux_free"] = r.get<u8>() != 0;
    c["rope_yarn_low"] = r.get<float>();
    c["rope_yarn_high"] = r.get<float>();
    c["sliding_window"] = r.get<i32>();
    c["rope_type"] = r.get<i32>();
  }
  return c;
}

const float* f32_data(const py::handle& h, size_t* n) {
  py::array a = py::reinterpret_borrow<py::array>(h);
  GBH_CHECK(a.dtype().is(py::dtype::of<float>()), "checkpoint tensors must be float32");
  GBH_CHECK((a.flags() & py::array::c_style) != 0, "checkpoint tensors must be C-contiguous");
  *n = static_cast<size_t>(a.size());
  return static_cast<const float*>(a.data());
}

void put_tensor(FileSink& o, const py::handle& h) {
  size_t n;
  const float* p = f32_data(h, &n);
  o.put<u64>(n);
  o.bytes(p, n * 4);
}

// opt: {"kind": "adamw"|"lion"|"muon", "t": int, "hyper": {...}, "m": [array|None], "v": [array|None], "fmt": 1|2}
void put_optimizer(FileSink& o, const py::dict& opt) {
  const std::string kind = item<std::string>(opt, "kind");
  py::list m = item<py::list>(opt, "m");
  py::list v = opt.contains("v") ? opt["v"].cast<py::list>() : py::list();
  py::dict h = item<py::dict>(opt, "hyper");
  const u64 count = m.size();
  const u8 fmt = opt.contains("fmt") ? item<int>(opt, "fmt") : 1;
  o.put<u8>(kind == "adamw" ? 0 : kind == "lion" ? 1 : 2);
  o.put<u64>(count);
  o.put<i64>(item<i64>(opt, "t"));
  o.put<u8>(fmt);
  if (kind == "adamw") {
    for (const char* k : {"lr", "beta1", "beta2", "eps", "weight_decay", "grad_clip"}) o.put<float>(item<float>(h, k));
    for (u64 i = 0; i < count; ++i) {
      const bool has = !m[i].is_none();
      o.put<u8>(has ? 1 : 0);
      if (!has) continue;
      size_t n, n2;
      const float* pm = f32_data(m[i], &n);
      const float* pv = f32_data(v[i], &n2);
      GBH_CHECK(n == n2, "adamw moments differ in size");
      o.put<u64>(n);
      o.bytes(pm, n * 4);
      o.bytes(pv, n * 4);
    }
  } else if (kind == "lion") {
    for (const char* k : {"lr", "beta1", "beta2", "weight_decay", "grad_clip"}) o.put<float>(item<float>(h, k));
    for (u64 i = 0; i < count; ++i) {
      const bool has = !m[i].is_none();
      o.put<u8>(has ? 1 : 0);
      if (has) put_tensor(o, m[i]);
    }
  } else if (kind == "muon") {
    for (const char* k : {"lr", "vec_ratio", "beta1", "beta2", "eps", "weight_decay", "grad_clip"})
      o.put<float>(item<float>(h, k));
    o.put<i32>(item<i32>(h, "ns_steps"));
    if (fmt == 2) o.put<i32>(item<i32>(h, "min_ns_dim"));
    for (u64 i = 0; i < count; ++i) {
      u8 mask = 0;
      if (!m[i].is_none()) mask |= 1;
      if (i < v.size() && !v[i].is_none()) mask |= 2;
      o.put<u8>(mask);
      if (mask & 1) put_tensor(o, m[i]);
      if (mask & 2) put_tensor(o, v[i]);
    }
  } else {
    fail("unknown optimizer kind: " + kind);
  }
}

py::array_t<float> take_f32(ByteReader& r, u64 n) {
  GBH_CHECK(n <= r.remaining() / 4, "checkpoint tensor runs past the end of the file");
  py::array_t<float> a(static_cast<py::ssize_t>(n));
  std::memcpy(a.mutable_data(), r.take(n * 4), n * 4);
  return a;
}

py::object get_optimizer(ByteReader& r, u32 version, const std::vector<u64>& numels) {
  // returns None when the blob is in a layout that cannot be decoded (pre-7 formats)
  py::dict opt;
  u8 kind = 0;
  if (version != 3) kind = r.get<u8>();
  if (version < 7) return py::none();
  const u64 count = r.get<u64>();
  GBH_CHECK(count <= 100000, "optimizer state: implausible tensor count");
  opt["t"] = r.get<i64>();
  const u8 fmt = r.get<u8>();
  GBH_CHECK(fmt == 1 || (kind == 2 && fmt == 2), "optimizer state: unknown format byte");
  opt["fmt"] = int(fmt);
  py::dict h;
  py::list m, v;
  auto tensor_for = [&](u64 i) {
    const u64 n = r.get<u64>();
    if (i < numels.size()) GBH_CHECK(n == numels[i], "optimizer state: moment size differs from its parameter");
    return take_f32(r, n);
  };
  if (kind == 0) {
    opt["kind"] = "adamw";
    for (const char* k : {"lr", "beta1", "beta2", "eps", "weight_decay", "grad_clip"}) h[k] = r.get<float>();
    for (u64 i = 0; i < count; ++i) {
      if (r.get<u8>()) {
        const u64 n = r.get<u64>();
        if (i < numels.size()) GBH_CHECK(n == numels[i], "optimizer state: moment size differs from its parameter");
        m.append(take_f32(r, n));
        v.append(take_f32(r, n));
      } else {
        m.append(py::none());
        v.append(py::none());
      }
    }
  } else if (kind == 1) {
    opt["kind"] = "lion";
    for (const char* k : {"lr", "beta1", "beta2", "weight_decay", "grad_clip"}) h[k] = r.get<float>();
    for (u64 i = 0; i < count; ++i) {
      if (r.get<u8>()) m.append(tensor_for(i));
      else m.append(py::none());
      v.append(py::none());
    }
  } else if (kind == 2) {
    opt["kind"] = "muon";
    for (const char* k : {"lr", "vec_ratio", "beta1", "beta2", "eps", "weight_decay", "grad_clip"}) h[k] = r.get<float>();
    h["ns_steps"] = r.get<i32>();
    if (fmt == 2) h["min_ns_dim"] = r.get<i32>();
    for (u64 i = 0; i < count; ++i) {
      const u8 mask = r.get<u8>();
      if (mask & 1) m.append(tensor_for(i)); else m.append(py::none());
      if (mask & 2) v.append(tensor_for(i)); else v.append(py::none());
    }
  } else {
    fail("optimizer state: unknown kind byte");
  }
  opt["hyper"] = h;
  opt["m"] = m;
  opt["v"] = v;
  return opt;
}

// Replace `path` by `tmp`: previous file is parked as .bak until the rename succeeded, and put back if it fails.
void publish(const std::string& path, const std::string& tmp) {
  const fs::path target(path), staged(tmp), backup(path + ".bak");
  std::error_code ec;
  if (fs::exists(target, ec) && !ec) {
    GBH_CHECK(!fs::is_directory(target, ec), "checkpoint path is a directory: " + path);
    if (fs::exists(backup, ec) && !ec) {
      fs::remove(backup, ec);
      GBH_CHECK(!ec, "cannot clear stale checkpoint backup: " + ec.message());
    }
    fs::rename(target, backup, ec);
    GBH_CHECK(!ec, "cannot stage previous checkpoint: " + ec.message());
  }
  fs::rename(staged, target, ec);
  if (ec) {
    const std::string why = ec.message();
    std::error_code rec;
    if (fs::exists(backup, rec) && !rec) fs::rename(backup, target, rec);
    fail("cannot finalise checkpoint: " + why);
  }
  std::error_code cec;
  if (fs::exists(backup, cec) && !cec) fs::remove(backup, cec);
}

void write_checkpoint(const std::string& path, const py::dict& config, const py::dict& state, const py::list& bias,
                      const py::list& params, const py::object& optimizer) {
  fs::path p(path);
  if (p.has_parent_path()) fs::create_directories(p.parent_path());
  std::error_code ec;
  if (fs::exists(p, ec) && !ec) GBH_CHECK(!fs::is_directory(p, ec), "checkpoint path is a directory: " + path);
  const std::string tmp = path + ".tmp";
  try {
    FileSink o(tmp);
    o.put<u32>(kCkptMagic);
    o.put<u32>(kCkptVersion);
    put_config(o, config);
    o.put<i64>(item<i64>(state, "step"));
    o.put<i64>(item<i64>(state, "tokens_seen"));
    o.put<double>(item<double>(state, "best_val"));
    o.put<double>(item<double>(state, "last_loss"));
    o.put<u64>(item<u64>(state, "seed"));
    put_loader(o, item<py::dict>(state, "loader"));
    o.put<double>(item<double>(state, "loss_scale"));
    o.put<i32>(item<i32>(state, "clean_steps"));
    o.put<i32>(item<i32>(state, "tok_vocab"));
    o.put<i64>(item<i64>(state, "sched_total"));
    o.put<i64>(item<i64>(state, "sched_warmup"));
    o.put<float>(item<float>(state, "sched_peak"));
    o.put<float>(item<float>(state, "sched_min_ratio"));
    o.put<float>(item<float>(state, "sched_decay_frac"));
    o.put<i32>(item<i32>(state, "sched_kind"));
    o.put<i32>(item<i32>(state, "ddp_world"));
    o.put<u64>(item<u64>(state, "tok_fingerprint"));
    put_loader(o, item<py::dict>(state, "val_loader"));
    o.put<u64>(bias.size());
    for (const auto& row : bias) {
      size_t n;
      const float* d = f32_data(row, &n);
      o.put<u32>(static_cast<u32>(n));
      o.bytes(d, n * 4);
    }
    o.put<u64>(params.size());
    for (const auto& it : params) {
      py::tuple t = it.cast<py::tuple>();
      const std::string name = t[0].cast<std::string>();
      o.put<u32>(static_cast<u32>(name.size()));
      o.bytes(name.data(), name.size());
      put_tensor(o, t[1]);
    }
    if (optimizer.is_none()) {
      o.put<u8>(0);
    } else {
      o.put<u8>(1);
      put_optimizer(o, optimizer.cast<py::dict>());
    }
    o.finish();
  } catch (...) {
    std::error_code rm;
    fs::remove(tmp, rm);
    throw;
  }
  try {
    publish(path, tmp);
  } catch (...) {
    std::error_code rm;
    fs::remove(tmp, rm);
    throw;
  }
}

// weights_only: stop after the parameter table (used by export / SFT initialisation / peek with tensors)
py::dict read_checkpoint(const std::string& path, bool header_only, bool with_optimizer) {
  std::vector<u8> raw = read_file(path);
  ByteReader r(raw.data(), raw.size());
  py::dict out;
  GBH_CHECK(r.remaining() >= 8 && r.get<u32>() == kCkptMagic, "not a checkpoint file: " + path);
  const u32 version = r.get<u32>();
  GBH_CHECK(version >= 3 && version <= kCkptVersion, sfmt("unsupported checkpoint version %u", version));
  out["version"] = version;
  out["config"] = get_config(r, version);
  py::dict st;
  st["step"] = r.get<i64>();
  st["tokens_seen"] = r.get<i64>();
  st["best_val"] = r.get<double>();
  st["last_loss"] = r.get<double>();
  st["seed"] = r.get<u64>();
  st["loader"] = get_loader(r, version >= 5);
  st["loss_scale"] = r.get<double>();
  st["clean_steps"] = r.get<i32>();
  st["tok_vocab"] = r.get<i32>();
  if (version >= 8) {
    st["sched_total"] = r.get<i64>();
    st["sched_warmup"] = r.get<i64>();
    st["sched_peak"] = r.get<float>();
    st["sched_min_ratio"] = r.get<float>();
    st["sched_decay_frac"] = r.get<float>();
    st["sched_kind"] = r.get<i32>();
    st["ddp_world"] = r.get<i32>();
  } else {
    st["sched_total"] = 0; st["sched_warmup"] = 0; st["sched_peak"] = 0.f; st["sched_min_ratio"] = 0.1f;
    st["sched_decay_frac"] = 0.2f; st["sched_kind"] = 0; st["ddp_world"] = 1;
  }
  st["tok_fingerprint"] = version >= 11 ? r.get<u64>() : u64(0);
  if (version >= 12) {
    st["val_loader"] = get_loader(r, true);
  } else {
    py::dict v;
    v["rng"] = py::make_tuple(u64(0), u64(0), u64(0), u64(0));
    v["batches"] = i64(-1);  // "absent"
    v["rng_spare"] = 0.f;
    v["rng_has_spare"] = 0;
    st["val_loader"] = v;
  }
  out["state"] = st;
  py::list bias;
  if (version >= 10) {
    const u64 layers = r.get<u64>();
    GBH_CHECK(layers <= 4096, "checkpoint corrupt: router-bias layer count implausible");
    for (u64 l = 0; l < layers; ++l) {
      const u32 n = r.get<u32>();
      GBH_CHECK(n <= 64, "checkpoint corrupt: router-bias row too wide");
      bias.append(take_f32(r, n));
    }
  }
  out["moe_bias"] = bias;
  if (header_only) return out;
  const u64 n = r.get<u64>();
  GBH_CHECK(n <= 10000, "checkpoint corrupt: param count implausible");
  py::list params;
  std::vector<u64> numels;
  bool finite = true;
  std::string first_bad;
  for (u64 i = 0; i < n; ++i) {
    const u32 len = r.get<u32>();
    GBH_CHECK(len <= 512, "checkpoint corrupt: parameter name too long");
    std::string name(reinterpret_cast<const char*>(r.take(len)), len);
    const u64 ne = r.get<u64>();
    py::array_t<float> a = take_f32(r, ne);
    if (finite) {
      const float* d = a.data();
      for (u64 j = 0; j < ne; ++j)
        if (!std::isfinite(d[j])) {
          finite = false;
          first_bad = name;
          break;
        }
    }
    numels.push_back(ne);
    params.append(py::make_tuple(name, a));
  }
  out["params"] = params;
  out["payload_finite"] = finite;
  out["first_nonfinite"] = first_bad;
  const u8 has_opt = r.get<u8>();
  out["has_optimizer"] = has_opt != 0;
  out["optimizer"] = py::none();
  out["trailing_bytes"] = size_t(0);
  if (has_opt && with_optimizer) {
    out["optimizer"] = get_optimizer(r, version, numels);
    if (!out["optimizer"].is_none()) out["trailing_bytes"] = r.remaining();
  } else if (!has_opt) {
    out["trailing_bytes"] = r.remaining();
  }
  return out;
}

}  // namespace

void bind_ckpt(py::module_& m) {
  m.def("write_checkpoint", &write_checkpoint, py::arg("path"), py::arg("config"), py::arg("state"), py::arg("moe_bias"),
        py::arg("params"), py::arg("optimizer"),
        "serialise a version-12 checkpoint to <path>.tmp and publish it atomically (previous file kept as .bak "
        "until the rename succeeded)");
  m.def("read_checkpoint", &read_checkpoint, py::arg("path"), py::arg("header_only") = false,
        py::arg("with_optimizer") = true);
  m.def("publish_file", &publish);
  m.attr("CKPT_VERSION") = kCkptVersion;
}
