// MXFP8 block format used by every stage: 32 consecutive elements along the
// contraction dimension share one UE8M0 scale byte; elements are E4M3.
//
// Scale rule (the arithmetic of the reference's mxfp8::quantize_* lives in an
// un-vendored submodule, call sites campaigns/mok/port/act_gptoss/swiglu.cuh:187,395-409;
// this library fixes the rule below and its CPU oracle implements the same one):
//   q      = amax / 448                     (IEEE fp32 division)
//   e      = clamp(ceil(log2 q), -127, 127) computed exactly from q's bit pattern;
//            amax == 0 gives e = -127
//   byte   = e + 127
//   elem_i = cvt.rn.satfinite.e4m3(x_i * 2^-e)
//
// Scale bytes for a [rows, cols] tensor live in a [rows/128, cols/128, 32, 16] u8
// tensor (campaigns/mok/host/resources.py:62-68): inside one 128x128 block the byte
// for row r, 32-column group g sits at (r % 32) * 16 + (r / 32) * 4 + g
// (campaigns/mok/port/act_gptoss/swiglu.cuh:367). That 512-byte block is exactly
// what one tcgen05.cp.32x128b.warpx4 moves into tensor memory.
#pragma once
#include "common.cuh"

namespace plb {

__device__ __forceinline__ uint32_t e8m0_from_amax(float amax) {
  const float q = __fdiv_rn(amax, 448.0f);
  const uint32_t bits = __float_as_uint(q);
  const uint32_t exp = (bits >> 23) & 0xFFu;
  const uint32_t mant = bits & 0x7FFFFFu;
  uint32_t e;
  if (exp == 0u) {
    e = mant > 0x400000u ? 1u : 0u;  // subnormal q: 2^-127 < q -> ceil = -126
  } else {
    e = exp + (mant != 0u ? 1u : 0u);
  }
  return e > 254u ? 254u : e;
}

// 2^(127 - byte): the factor elements are multiplied by before the E4M3 cast.
__device__ __forceinline__ float e8m0_inverse(uint32_t byte) {
  const uint32_t field = 254u - byte;
  return __uint_as_float(field == 0u ? 0x00400000u : field << 23);
}

// 2^(byte - 127): the factor a stored element is multiplied by to recover its value.
__device__ __forceinline__ float e8m0_value(uint32_t byte) {
  return __uint_as_float(byte == 0u ? 0x00400000u : byte << 23);
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(__half(h));
}

// Byte offset of the scale for (row, 32-column group) in the [R/128, C/128, 32, 16] tensor.
__host__ __device__ __forceinline__ size_t scale_offset(int64_t row, int64_t group,
                                                        int64_t col_blocks /* C/128 */) {
  return (static_cast<size_t>(row >> 7) * col_blocks + (group >> 2)) * 512 +
         (row & 31) * 16 + ((row & 127) >> 5) * 4 + (group & 3);
}

}  // namespace plb
