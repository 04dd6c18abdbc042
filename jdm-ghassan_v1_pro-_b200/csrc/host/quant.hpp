// Block quantisers shared by the GAI / GGUF codecs and the `quantize` command.
//
// Internal (".gai") formats, byte-exact with the reference (core/dtype.h:24-47,
// quantization/quantize.cpp:16-333):
//   Q8_0 : 64 values  -> f32 scale (amax/127)            + 64 x i8            (68 B)
//   Q4_0 : 32 values  -> f16 scale (amax/8)              + 16 B, v = (nib-8)*s (18 B)
//   Q4_1 : 32 values  -> f16 scale ((max-min)/15), f16 min + 16 B, v = nib*s+min (20 B)
// ggml formats written into GGUF files (format/gguf_codec.cpp in the reference):
//   GGML_Q8_0 : 32 values -> f16 scale (amax/127) + 32 x i8 (34 B)
//   GGML_Q4_0 : 32 values -> f16 scale            + 16 B with the ggml nibble order (low nibbles = first half)
// A block that contains a non-finite value is stored as zeros; a ragged tail is padded with the code for 0.
#pragma once
#include <algorithm>
#include <cmath>

#include "core.hpp"

namespace gbh {
namespace quant {

enum DTypeId : u32 { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, I8 = 4, Q8_0 = 5, Q4_0 = 6, Q4_1 = 7, U16 = 8, I64 = 9 };

const char* dtype_name(u32 t);
u32 dtype_from_name(const std::string& s);
int block_size(u32 t);      // values per block (1 for plain types)
size_t block_bytes(u32 t);  // bytes per block / element
size_t nbytes(u32 t, size_t numel);
inline bool is_quantized(u32 t) { return t == Q8_0 || t == Q4_0 || t == Q4_1; }

void quantize(u32 type, const float* src, void* dst, i64 n);
void dequantize(u32 type, const void* src, float* dst, i64 n);

// ggml block formats (GGUF tensor types 8 and 2)
constexpr size_t kGgmlQ80Bytes = 34, kGgmlQ40Bytes = 18;
void ggml_quantize_q8_0(const float* src, u8* dst, i64 n);   // n % 32 == 0
void ggml_dequantize_q8_0(const u8* src, float* dst, i64 n);
void ggml_quantize_q4_0(const float* src, u8* dst, i64 n);   // n % 32 == 0
void ggml_dequantize_q4_0(const u8* src, float* dst, i64 n);

struct ErrorStats {
  double rmse = 0, rel_rmse = 0, cosine = 0, max_abs = 0;
  i64 numel = 0;
};
ErrorStats measure_error(const float* a, const float* b, i64 n);

}  // namespace quant
}  // namespace gbh
