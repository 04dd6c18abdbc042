// Host runtime basics: error type, bit-exact random stream, hashes, fp16/bf16 codecs.
//
// The random stream, the FNV-1a file fingerprint and the half-precision rounding rules are part of
// the on-disk contract (checkpoints store the generator state, weight initialisation and the data
// stream are derived from it), so they reproduce the reference's definitions bit for bit
// (core/rng.h:8-107, core/common.cpp:95-111, core/dtype.cpp:5-70 in the reference tree).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace gbh {

using u8 = uint8_t;
using i8 = int8_t;
using u16 = uint16_t;
using u32 = uint32_t;
using u64 = uint64_t;
using i32 = int32_t;
using i64 = int64_t;

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
[[noreturn]] inline void fail(const std::string& m) { throw Error(m); }
#define GBH_CHECK(cond, msg) \
  do {                       \
    if (!(cond)) ::gbh::fail(msg); \
  } while (0)

std::string sfmt(const char* fmt, ...);

// ------------------------------------------------------------------ hashes
constexpr u64 kFnvOffset = 1469598103934665603ULL;
constexpr u64 kFnvPrime = 1099511628211ULL;
inline u64 fnv1a64(const void* data, size_t n, u64 h = kFnvOffset) {
  const u8* p = static_cast<const u8*>(data);
  for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * kFnvPrime;
  return h;
}
inline u64 splitmix64(u64 x) {
  x += 0x9E3779B97F4A7C15ULL;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
  return x ^ (x >> 31);
}
// FNV-1a over the file bytes; 0 means "unreadable", a readable file never hashes to 0.
u64 fingerprint_file(const std::string& path);
std::string fingerprint_hex(u64 fp);

// ------------------------------------------------------------------ random stream (xoshiro256**)
struct RngState {
  u64 s[4] = {0, 0, 0, 0};
  float spare = 0.f;
  bool has_spare = false;
};

class Rng {
 public:
  explicit Rng(u64 seed = 1234567891011ULL) { reseed(seed); }
  void reseed(u64 seed) {
    // four rounds of splitmix64 over a running counter
    for (auto& w : st_.s) {
      w = splitmix64(seed);
      seed += 0x9E3779B97F4A7C15ULL;
    }
    st_.has_spare = false;
  }
  u64 next_u64() {
    u64* s = st_.s;
    const u64 out = rotl(s[1] * 5, 7) * 9;
    const u64 t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl(s[3], 45);
    return out;
  }
  u32 next_u32() { return static_cast<u32>(next_u64() >> 32); }
  // top 24 bits -> [0, 1)
  float uniform() { return static_cast<float>((next_u64() >> 40) * (1.0 / 16777216.0)); }
  u64 below(u64 n) {
    GBH_CHECK(n > 0, "Rng::below(0)");
    return next_u64() % n;
  }
  // Marsaglia polar method; the second variate is kept for the next call.
  float normal(float mean = 0.f, float stddev = 1.f) {
    if (st_.has_spare) {
      st_.has_spare = false;
      return mean + stddev * st_.spare;
    }
    float u, v, r2;
    do {
      u = uniform() * 2.0f - 1.0f;
      v = uniform() * 2.0f - 1.0f;
      r2 = u * u + v * v;
    } while (r2 >= 1.0f || r2 == 0.0f);
    const float m = std::sqrt(-2.0f * std::log(r2) / r2);
    st_.spare = v * m;
    st_.has_spare = true;
    return mean + stddev * (u * m);
  }
  // up to eight draws, first one within two sigma wins, otherwise 0
  float truncated_normal(float stddev) {
    for (int tries = 0; tries < 8; ++tries) {
      const float x = normal(0.f, stddev);
      if (std::fabs(x) <= 2.0f * stddev) return x;
    }
    return 0.f;
  }
  const RngState& state() const { return st_; }
  void set_state(const RngState& s) { st_ = s; }
  // state without the cached variate (older checkpoints)
  void set_words(const u64 w[4]) {
    for (int i = 0; i < 4; ++i) st_.s[i] = w[i];
    st_.has_spare = false;
    st_.spare = 0.f;
  }

 private:
  static u64 rotl(u64 x, int k) { return (x << k) | (x >> (64 - k)); }
  RngState st_;
};

// ------------------------------------------------------------------ 16-bit float codecs
inline u32 f32_bits(float f) {
  u32 u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float bits_f32(u32 u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
// Normal range: round-to-nearest-even (a carry may roll into the exponent, up to infinity).
// Subnormal range: round half up on the first dropped bit; magnitudes below 2^-25 flush to zero.
// NaN maps to the single quiet pattern 0x7E00.  These are the rules the stored quantisation scales
// were written with, so they are kept as they are.
inline u16 f32_to_f16(float f) {
  const u32 x = f32_bits(f);
  const u32 sign = (x >> 16) & 0x8000u;
  u32 mant = x & 0x7FFFFFu;
  const u32 e8 = (x >> 23) & 0xFFu;
  if (e8 == 0xFFu) return static_cast<u16>(sign | 0x7C00u | (mant ? 0x200u : 0u));
  const i32 exp = static_cast<i32>(e8) - 127 + 15;
  if (exp >= 31) return static_cast<u16>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<u16>(sign);
    mant |= 0x800000u;
    const u32 shift = static_cast<u32>(14 - exp);
    u32 h = mant >> shift;
    if ((mant >> (shift - 1)) & 1u) ++h;
    return static_cast<u16>(sign | h);
  }
  u32 h = sign | (static_cast<u32>(exp) << 10) | (mant >> 13);
  const u32 rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
  return static_cast<u16>(h);
}
inline float f16_to_f32(u16 h) {
  const u32 sign = (static_cast<u32>(h) & 0x8000u) << 16;
  u32 exp = (h >> 10) & 0x1Fu;
  u32 mant = h & 0x3FFu;
  if (exp == 0) {
    if (mant == 0) return bits_f32(sign);
    int e = -1;
    do {
      ++e;
      mant <<= 1;
    } while (!(mant & 0x400u));
    mant &= 0x3FFu;
    return bits_f32(sign | (static_cast<u32>(127 - 15 - e) << 23) | (mant << 13));
  }
  if (exp == 31) return bits_f32(sign | 0x7F800000u | (mant << 13));
  return bits_f32(sign | ((exp + 112) << 23) | (mant << 13));
}
// round-to-nearest-even; inf and NaN are truncated (exponent-all-ones inputs keep their top 16 bits)
inline u16 f32_to_bf16(float f) {
  u32 x = f32_bits(f);
  if (((x >> 23) & 0xFFu) == 0xFFu) return static_cast<u16>(x >> 16);
  x += 0x7FFFu + ((x >> 16) & 1u);
  return static_cast<u16>(x >> 16);
}
inline float bf16_to_f32(u16 h) { return bits_f32(static_cast<u32>(h) << 16); }

// ------------------------------------------------------------------ little-endian byte buffers
class ByteWriter {
 public:
  std::vector<u8> buf;
  template <typename T>
  void put(const T& v) {
    const u8* p = reinterpret_cast<const u8*>(&v);
    buf.insert(buf.end(), p, p + sizeof(T));
  }
  void put_bytes(const void* p, size_t n) {
    const u8* b = static_cast<const u8*>(p);
    buf.insert(buf.end(), b, b + n);
  }
  void put_str32(const std::string& s) {
    put<u32>(static_cast<u32>(s.size()));
    put_bytes(s.data(), s.size());
  }
};

class ByteReader {
 public:
  ByteReader(const u8* p, size_t n) : p_(p), n_(n) {}
  template <typename T>
  T get() {
    GBH_CHECK(pos_ + sizeof(T) <= n_, "unexpected end of data");
    T v;
    std::memcpy(&v, p_ + pos_, sizeof(T));
    pos_ += sizeof(T);
    return v;
  }
  const u8* take(size_t n) {
    GBH_CHECK(n <= n_ - pos_, "unexpected end of data");
    const u8* r = p_ + pos_;
    pos_ += n;
    return r;
  }
  std::string get_str32() {
    const u32 n = get<u32>();
    const u8* b = take(n);
    return std::string(reinterpret_cast<const char*>(b), n);
  }
  size_t pos() const { return pos_; }
  size_t remaining() const { return n_ - pos_; }
  void seek(size_t p) {
    GBH_CHECK(p <= n_, "seek past end");
    pos_ = p;
  }

 private:
  const u8* p_;
  size_t n_;
  size_t pos_ = 0;
};

std::vector<u8> read_file(const std::string& path);
void write_file_atomic(const std::string& path, const void* data, size_t n);

}  // namespace gbh
