// Stored weight rows of the decode kernels: how eight consecutive values of a row are expanded into floats, per
// storage format (formats and block layouts in gb_decode.h).  Shared by the per-kernel token step (decode.cu) and
// the single-kernel token step (decode_mega.cu).
#pragma once
#include "sm100_common.cuh"
#include "gb_decode.h"

namespace gb {

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// Expand unit u (values 8u .. 8u+7) of one stored row into floats.
template <int FMT>
__device__ __forceinline__ void load8(const uint8_t* __restrict__ row, int u, float (&w)[8]) {
  if constexpr (FMT == GB_W_F16) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + 16 * (size_t)u);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else if constexpr (FMT == GB_W_BF16) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + 16 * (size_t)u);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else if constexpr (FMT == GB_W_GGML_Q8_0) {
    const uint8_t* p = row + (size_t)(u >> 2) * 34;
    const float d = h2f(ld_u16(p));
    const uint8_t* q = p + 2 + (u & 3) * 8;           // 2-byte aligned: blocks are 34 bytes
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint16_t v = ld_u16(q + 2 * i);
      w[2 * i] = d * (float)(int8_t)(v & 0xFF);
      w[2 * i + 1] = d * (float)(int8_t)(v >> 8);
    }
  } else if constexpr (FMT == GB_W_Q4_0) {
    const uint8_t* p = row + (size_t)(u >> 2) * 18;
    const float d = h2f(ld_u16(p));
    const uint8_t* q = p + 2 + (u & 3) * 4;
    const uint32_t v = (uint32_t)ld_u16(q) | ((uint32_t)ld_u16(q + 2) << 16);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)((int)((v >> (4 * i)) & 0xF) - 8);   // byte i: low nibble = value 2i
  } else if constexpr (FMT == GB_W_Q8_64) {
    const uint8_t* p = row + (size_t)(u >> 3) * 68;
    const float d = *reinterpret_cast<const float*>(p);
    // blocks are 68 bytes: the quants are 4-byte aligned but not 8-byte aligned, so two 32-bit loads
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(p + 4 + (u & 7) * 8);
    const uint32_t vx = qp[0], vy = qp[1];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = d * (float)(int8_t)((vx >> (8 * i)) & 0xFF);
      w[4 + i] = d * (float)(int8_t)((vy >> (8 * i)) & 0xFF);
    }
  } else {   // GB_W_Q4_1
    const uint8_t* p = row + (size_t)(u >> 2) * 20;
    const float d = h2f(ld_u16(p)), m = h2f(ld_u16(p + 2));
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p + 4 + (u & 3) * 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)((v >> (4 * i)) & 0xF) + m;
  }
}

}  // namespace gb
