// Stage gemm.epilogue.bias-silu: four warps drain the accumulator, add bias, apply SiLU, store bf16.
#include "gemm3.cuh"

extern "C" __device__ void gemm_epilogue_bias_silu_role(const void* params, unsigned variant);
PL_STAGE("gemm.epilogue.bias-silu", "1.0.0");
PL_PARAMS(Gemm3EpilogueParams, bias, out, N);
PL_ROLE(epilogue, gemm_epilogue_bias_silu_role, 4);
GEMM3_TOPOLOGY();
PL_ENDPOINT(accumulator, gemm3::accumulator(pl::consume, "epilogue"));
PL_CLAIM_WARPS(pipelink_gemm_warp_epilogue, epilogue, 4, 4);
GEMM3_CLAIM_ACCUMULATOR();

#ifndef PIPELINK_EMIT
#include <cuda_bf16.h>
extern "C" __device__ void gemm_epilogue_bias_silu_role(const void* raw_params, unsigned) {
  using namespace gemm3;
  const Gemm3EpilogueParams& p = *static_cast<const Gemm3EpilogueParams*>(raw_params);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int quad = warp & 3;  // the TMEM lane quadrant a warp may read is warp index mod 4
  if (!wait(barrier_addr(smem, pipelink_gemm_acc_ready()), 0)) return;
  plb::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot());
  const uint32_t taddr = tmem + pipelink_gemm_acc() + (static_cast<uint32_t>(quad * 32) << 16);
  const int row = blockIdx.x * TileM + quad * 32 + lane;
  const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(p.bias) + blockIdx.y * TileN;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.N + blockIdx.y * TileN;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    plb::tc_ld_32x32b_x32(taddr + c * 32, v);
    plb::tc_wait_ld();
    uint4* dst = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = q * 8 + e * 2;
        float x0 = __uint_as_float(v[col]) + __bfloat162float(bias[c * 32 + col]);
        float x1 = __uint_as_float(v[col + 1]) + __bfloat162float(bias[c * 32 + col + 1]);
        x0 = x0 / (1.0f + __expf(-x0));
        x1 = x1 / (1.0f + __expf(-x1));
        __nv_bfloat162 t = __floats2bfloat162_rn(x0, x1);
        w[e] = *reinterpret_cast<uint32_t*>(&t);
      }
      dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  plb::tc_fence_before();
  // accumulator released: one arrival per epilogue warp on the channel's empty side
  __syncwarp();
  if (lane == 0) plb::mbar_arrive(barrier_addr(smem, pipelink_gemm_acc_empty()));
}
#endif  // !PIPELINK_EMIT
