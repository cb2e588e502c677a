// Epilogue arithmetic of the gate/up projection, shared by the library kernel
// (grouped_gemm2.cu) and the separately packed epilogue stage (stages/moe): bf16 rounding of the
// accumulator, the (optionally clamped) SwiGLU, and the MXFP8 requantisation of 32 hidden values.
// One definition, so the linked image and the library produce the same bits.
#pragma once
#include "mxfp8.cuh"

namespace plb {

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf16(uint32_t a_bits, uint32_t b_bits) {
  __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(a_bits), __uint_as_float(b_bits));
  return *reinterpret_cast<uint32_t*>(&t);
}

// 32 gate + 32 up accumulator values -> 32 E4M3 bytes (two uint4) and the block's scale byte.
// Clamped SwiGLU of one bf16-valued pair (campaigns/mok/port/act_gptoss/swiglu.cuh:143-147 applies
// the same bounds: gate from above only, up from both sides); limit = +inf leaves both unchanged.
__device__ __forceinline__ float swiglu_clamped(float gf, float uf, float limit) {
  gf = fminf(gf, limit);
  uf = fminf(fmaxf(uf, -limit), limit);
  return __fdividef(gf, 1.0f + __expf(-gf)) * uf;
}

__device__ __forceinline__ uint32_t swiglu_quant32(const uint32_t* g, const uint32_t* u, float limit,
                                                   uint4& q0, uint4& q1) {
  float h[32];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float gf = bf16r(__uint_as_float(g[i]));
    const float uf = bf16r(__uint_as_float(u[i]));
    h[i] = bf16r(swiglu_clamped(gf, uf, limit));
    amax = fmaxf(amax, fabsf(h[i]));
  }
  const uint32_t e = e8m0_from_amax(amax);
  const float inv = e8m0_inverse(e);
  q0.x = cvt_e4m3x4(h[0] * inv, h[1] * inv, h[2] * inv, h[3] * inv);
  q0.y = cvt_e4m3x4(h[4] * inv, h[5] * inv, h[6] * inv, h[7] * inv);
  q0.z = cvt_e4m3x4(h[8] * inv, h[9] * inv, h[10] * inv, h[11] * inv);
  q0.w = cvt_e4m3x4(h[12] * inv, h[13] * inv, h[14] * inv, h[15] * inv);
  q1.x = cvt_e4m3x4(h[16] * inv, h[17] * inv, h[18] * inv, h[19] * inv);
  q1.y = cvt_e4m3x4(h[20] * inv, h[21] * inv, h[22] * inv, h[23] * inv);
  q1.z = cvt_e4m3x4(h[24] * inv, h[25] * inv, h[26] * inv, h[27] * inv);
  q1.w = cvt_e4m3x4(h[28] * inv, h[29] * inv, h[30] * inv, h[31] * inv);
  return e;
}

}  // namespace plb
