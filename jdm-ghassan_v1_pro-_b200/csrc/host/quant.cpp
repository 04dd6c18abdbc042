#include "quant.hpp"

#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

namespace py = pybind11;

namespace gbh {
namespace quant {

const char* dtype_name(u32 t) {
  static const char* names[] = {"f32", "f16", "bf16", "i32", "i8", "q8_0", "q4_0", "q4_1", "u16", "i64"};
  return t < 10 ? names[t] : "?";
}

u32 dtype_from_name(const std::string& s) {
  static const std::pair<const char*, u32> table[] = {
      {"f32", F32}, {"fp32", F32}, {"f16", F16}, {"fp16", F16}, {"bf16", BF16}, {"i32", I32}, {"i8", I8},
      {"int8", I8}, {"q8_0", Q8_0}, {"q8", Q8_0}, {"q4_0", Q4_0}, {"q4", Q4_0}, {"q4_1", Q4_1}, {"u16", U16},
      {"i64", I64}};
  for (const auto& [k, v] : table)
    if (s == k) return v;
  fail("unknown dtype: " + s);
}

int block_size(u32 t) { return t == Q8_0 ? 64 : (t == Q4_0 || t == Q4_1) ? 32 : 1; }

size_t block_bytes(u32 t) {
  switch (t) {
    case F32: case I32: return 4;
    case F16: case BF16: case U16: return 2;
    case I8: return 1;
    case I64: return 8;
    case Q8_0: return 68;
    case Q4_0: return 18;
    case Q4_1: return 20;
  }
  fail("unknown dtype id");
}

size_t nbytes(u32 t, size_t numel) {
  const size_t bs = static_cast<size_t>(block_size(t));
  return (numel + bs - 1) / bs * block_bytes(t);
}

namespace {

inline int round_clamp(float v, int lo, int hi) { return std::clamp(static_cast<int>(std::lround(v)), lo, hi); }

// Scan `len` live values of a block: false when one is not finite.
inline bool scan_absmax(const float* x, i64 len, float& amax) {
  amax = 0.f;
  for (i64 i = 0; i < len; ++i) {
    if (!std::isfinite(x[i])) return false;
    amax = std::max(amax, std::fabs(x[i]));
  }
  return true;
}

inline void put_u16(u8* p, u16 v) { std::memcpy(p, &v, 2); }
inline u16 get_u16(const u8* p) { u16 v; std::memcpy(&v, p, 2); return v; }

// --- one block each; `len` <= block size is the number of live values, the rest is padding -------------
void enc_q8_64(const float* x, i64 len, u8* out) {
  float amax;
  if (!scan_absmax(x, len, amax)) {
    std::memset(out, 0, 68);
    return;
  }
  const float scale = amax / 127.0f, inv = scale > 0.f ? 1.0f / scale : 0.f;
  std::memcpy(out, &scale, 4);
  i8* q = reinterpret_cast<i8*>(out + 4);
  for (i64 i = 0; i < 64; ++i) q[i] = i < len ? static_cast<i8>(round_clamp(x[i] * inv, -127, 127)) : 0;
}
void dec_q8_64(const u8* in, i64 len, float* y) {
  float s;
  std::memcpy(&s, in, 4);
  const i8* q = reinterpret_cast<const i8*>(in + 4);
  for (i64 i = 0; i < len; ++i) y[i] = static_cast<float>(q[i]) * s;
}

// nibble pairs are adjacent values: byte i = (code[2i+1] << 4) | code[2i]
void enc_q4_sym(const float* x, i64 len, u8* out) {
  float amax;
  if (!scan_absmax(x, len, amax)) {
    put_u16(out, f32_to_f16(0.f));
    std::memset(out + 2, 0x88, 16);
    return;
  }
  const float scale = amax / 8.0f, inv = scale > 0.f ? 1.0f / scale : 0.f;
  put_u16(out, f32_to_f16(scale));
  for (i64 i = 0; i < 16; ++i) {
    const int lo = 2 * i < len ? round_clamp(x[2 * i] * inv, -8, 7) + 8 : 8;
    const int hi = 2 * i + 1 < len ? round_clamp(x[2 * i + 1] * inv, -8, 7) + 8 : 8;
    out[2 + i] = static_cast<u8>((hi << 4) | lo);
  }
}
void dec_q4_sym(const u8* in, i64 len, float* y) {
  const float s = f16_to_f32(get_u16(in));
  for (i64 i = 0; i < len; ++i) {
    const u8 b = in[2 + i / 2];
    y[i] = (static_cast<float>((i & 1) ? (b >> 4) : (b & 0x0F)) - 8.0f) * s;
  }
}

void enc_q4_affine(const float* x, i64 len, u8* out) {
  float amax;
  if (!scan_absmax(x, len, amax)) {
    put_u16(out, f32_to_f16(0.f));
    put_u16(out + 2, f32_to_f16(0.f));
    std::memset(out + 4, 0, 16);
    return;
  }
  float mn = x[0], mx = x[0];
  for (i64 i = 1; i < len; ++i) {
    mn = std::min(mn, x[i]);
    mx = std::max(mx, x[i]);
  }
  const float scale = (mx - mn) / 15.0f, inv = scale > 0.f ? 1.0f / scale : 0.f;
  put_u16(out, f32_to_f16(scale));
  put_u16(out + 2, f32_to_f16(mn));
  const int zero_code = round_clamp((0.0f - mn) * inv, 0, 15);
  for (i64 i = 0; i < 16; ++i) {
    const int lo = 2 * i < len ? round_clamp((x[2 * i] - mn) * inv, 0, 15) : zero_code;
    const int hi = 2 * i + 1 < len ? round_clamp((x[2 * i + 1] - mn) * inv, 0, 15) : zero_code;
    out[4 + i] = static_cast<u8>((hi << 4) | lo);
  }
}
void dec_q4_affine(const u8* in, i64 len, float* y) {
  const float s = f16_to_f32(get_u16(in)), m = f16_to_f32(get_u16(in + 2));
  for (i64 i = 0; i < len; ++i) {
    const u8 b = in[4 + i / 2];
    y[i] = static_cast<float>((i & 1) ? (b >> 4) : (b & 0x0F)) * s + m;
  }
}

void enc_ggml_q8(const float* x, i64 len, u8* out) {
  float amax;
  if (!scan_absmax(x, len, amax)) {
    put_u16(out, f32_to_f16(0.f));
    std::memset(out + 2, 0, 32);
    return;
  }
  const float scale = amax / 127.f, inv = scale != 0.f ? 1.f / scale : 0.f;
  put_u16(out, f32_to_f16(scale));
  for (i64 i = 0; i < 32; ++i)
    out[2 + i] = static_cast<u8>(static_cast<i8>(i < len ? round_clamp(x[i] * inv, -127, 127) : 0));
}
void dec_ggml_q8(const u8* in, i64 len, float* y) {
  const float s = f16_to_f32(get_u16(in));
  for (i64 i = 0; i < len; ++i) y[i] = static_cast<float>(static_cast<i8>(in[2 + i])) * s;
}

template <int BLOCK, int BYTES, typename Enc>
void encode_all(const float* src, u8* dst, i64 n, Enc enc) {
  GBH_CHECK(n >= 0, "element count must be non-negative");
  const i64 blocks = (n + BLOCK - 1) / BLOCK;
  for (i64 b = 0; b < blocks; ++b) enc(src + b * BLOCK, std::min<i64>(BLOCK, n - b * BLOCK), dst + b * BYTES);
}
template <int BLOCK, int BYTES, typename Dec>
void decode_all(const u8* src, float* dst, i64 n, Dec dec) {
  GBH_CHECK(n >= 0, "element count must be non-negative");
  const i64 blocks = (n + BLOCK - 1) / BLOCK;
  for (i64 b = 0; b < blocks; ++b) dec(src + b * BYTES, std::min<i64>(BLOCK, n - b * BLOCK), dst + b * BLOCK);
}

}  // namespace

void quantize(u32 type, const float* src, void* dst, i64 n) {
  u8* d = static_cast<u8*>(dst);
  switch (type) {
    case F32: std::memcpy(dst, src, static_cast<size_t>(n) * 4); return;
    case F16: for (i64 i = 0; i < n; ++i) { u16 h = f32_to_f16(src[i]); std::memcpy(d + 2 * i, &h, 2); } return;
    case BF16: for (i64 i = 0; i < n; ++i) { u16 h = f32_to_bf16(src[i]); std::memcpy(d + 2 * i, &h, 2); } return;
    case Q8_0: encode_all<64, 68>(src, d, n, enc_q8_64); return;
    case Q4_0: encode_all<32, 18>(src, d, n, enc_q4_sym); return;
    case Q4_1: encode_all<32, 20>(src, d, n, enc_q4_affine); return;
  }
  fail(std::string("unsupported quantization target: ") + dtype_name(type));
}

void dequantize(u32 type, const void* src, float* dst, i64 n) {
  const u8* s = static_cast<const u8*>(src);
  switch (type) {
    case F32: std::memcpy(dst, src, static_cast<size_t>(n) * 4); return;
    case F16: for (i64 i = 0; i < n; ++i) dst[i] = f16_to_f32(get_u16(s + 2 * i)); return;
    case BF16: for (i64 i = 0; i < n; ++i) dst[i] = bf16_to_f32(get_u16(s + 2 * i)); return;
    case Q8_0: decode_all<64, 68>(s, dst, n, dec_q8_64); return;
    case Q4_0: decode_all<32, 18>(s, dst, n, dec_q4_sym); return;
    case Q4_1: decode_all<32, 20>(s, dst, n, dec_q4_affine); return;
  }
  fail(std::string("unsupported dequantization source: ") + dtype_name(type));
}

void ggml_quantize_q8_0(const float* src, u8* dst, i64 n) { encode_all<32, 34>(src, dst, n, enc_ggml_q8); }
void ggml_dequantize_q8_0(const u8* src, float* dst, i64 n) { decode_all<32, 34>(src, dst, n, dec_ggml_q8); }
void ggml_quantize_q4_0(const float* src, u8* dst, i64 n) { encode_all<32, 18>(src, dst, n, enc_q4_sym); }
void ggml_dequantize_q4_0(const u8* src, float* dst, i64 n) { decode_all<32, 18>(src, dst, n, dec_q4_sym); }

ErrorStats measure_error(const float* a, const float* b, i64 n) {
  ErrorStats e;
  e.numel = n;
  if (n == 0) return e;
  double se = 0, sa = 0, dot = 0, nb = 0;
  i64 finite = 0;
  for (i64 i = 0; i < n; ++i) {
    if (!std::isfinite(a[i]) || !std::isfinite(b[i])) {
      e.max_abs = INFINITY;
      continue;
    }
    ++finite;
    const double x = a[i], y = b[i], d = x - y;
    se += d * d;
    sa += x * x;
    dot += x * y;
    nb += y * y;
    e.max_abs = std::max(e.max_abs, std::fabs(d));
  }
  const double denom = static_cast<double>(finite > 0 ? finite : 1);
  e.rmse = std::sqrt(se / denom);
  const double rms_a = std::sqrt(sa / denom);
  e.rel_rmse = rms_a > 0 ? e.rmse / rms_a : 0.0;
  e.cosine = (sa > 0 && nb > 0) ? dot / (std::sqrt(sa) * std::sqrt(nb)) : 0.0;
  return e;
}

}  // namespace quant
}  // namespace gbh

using namespace gbh;

void bind_quant(py::module_& m) {
  using farr = py::array_t<float, py::array::c_style | py::array::forcecast>;
  using barr = py::array_t<u8, py::array::c_style | py::array::forcecast>;
  m.def("dtype_id", &quant::dtype_from_name);
  m.def("dtype_name", [](u32 t) { return std::string(quant::dtype_name(t)); });
  m.def("dtype_nbytes", &quant::nbytes);
  m.def("dtype_block_size", &quant::block_size);
  m.def("quantize", [](farr src, const std::string& type) {
    const u32 t = quant::dtype_from_name(type);
    py::array_t<u8> out(static_cast<py::ssize_t>(quant::nbytes(t, static_cast<size_t>(src.size()))));
    quant::quantize(t, src.data(), out.mutable_data(), src.size());
    return out;
  }, "float32 array -> packed bytes in one of f32/f16/bf16/q8_0/q4_0/q4_1 (internal block formats)");
  m.def("dequantize", [](barr src, const std::string& type, i64 n) {
    const u32 t = quant::dtype_from_name(type);
    GBH_CHECK(static_cast<size_t>(src.size()) >= quant::nbytes(t, static_cast<size_t>(n)), "packed buffer too small");
    py::array_t<float> out(static_cast<py::ssize_t>(n));
    quant::dequantize(t, src.data(), out.mutable_data(), n);
    return out;
  });
  m.def("ggml_quantize", [](farr src, int ggml_type) {
    const i64 n = src.size();
    const size_t bytes = ggml_type == 8 ? 34 : 18;
    GBH_CHECK(ggml_type == 8 || ggml_type == 2, "ggml_quantize supports Q8_0 (8) and Q4_0 (2)");
    py::array_t<u8> out(static_cast<py::ssize_t>((n + 31) / 32 * bytes));
    if (ggml_type == 8) quant::ggml_quantize_q8_0(src.data(), out.mutable_data(), n);
    else quant::ggml_quantize_q4_0(src.data(), out.mutable_data(), n);
    return out;
  });
  m.def("ggml_dequantize", [](barr src, int ggml_type, i64 n) {
    GBH_CHECK(ggml_type == 8 || ggml_type == 2, "ggml_dequantize supports Q8_0 (8) and Q4_0 (2)");
    const size_t bytes = ggml_type == 8 ? 34 : 18;
    GBH_CHECK(static_cast<size_t>(src.size()) >= static_cast<size_t>((n + 31) / 32) * bytes, "packed buffer too small");
    py::array_t<float> out(static_cast<py::ssize_t>(n));
    if (ggml_type == 8) quant::ggml_dequantize_q8_0(src.data(), out.mutable_data(), n);
    else quant::ggml_dequantize_q4_0(src.data(), out.mutable_data(), n);
    return out;
  });
  m.def("quant_error", [](farr a, farr b) {
    GBH_CHECK(a.size() == b.size(), "arrays differ in size");
    quant::ErrorStats e = quant::measure_error(a.data(), b.data(), a.size());
    py::dict d;
    d["rmse"] = e.rmse; d["rel_rmse"] = e.rel_rmse; d["cosine"] = e.cosine; d["max_abs"] = e.max_abs; d["numel"] = e.numel;
    return d;
  });
}

// GGUF and GAI codecs live in their own files.
