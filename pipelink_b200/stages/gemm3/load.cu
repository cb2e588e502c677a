// Stage gemm.load: one elected lane feeds the operands ring with TMA.
#include "gemm3.cuh"

extern "C" __device__ void gemm_load_role(const void* params, unsigned variant);
PL_STAGE("gemm.load", "1.0.0");
PL_PARAMS(Gemm3LoadParams, a, b, a_sc, b_sc, K);
PL_ROLE(load, gemm_load_role, 1);
GEMM3_TOPOLOGY();
PL_ENDPOINT(operands, gemm3::operands(pl::produce, "load"));
PL_CLAIM_WARPS(pipelink_gemm_warp_load, load, 1, 1);
GEMM3_CLAIM_OPERANDS();

#ifndef PIPELINK_EMIT
extern "C" __device__ void gemm_load_role(const void* raw_params, unsigned) {
  using namespace gemm3;
  const Gemm3LoadParams& p = *static_cast<const Gemm3LoadParams*>(raw_params);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  if ((threadIdx.x & 31) != 0) return;
  const uint32_t smem = plb::smem_u32(pl_smem);
  const int depth = pipelink_gemm_depth();
  const int k_steps = p.K / TileK;
  const int m_blk = blockIdx.x, n_blk = blockIdx.y;
  for (int k = 0; k < k_steps; ++k) {
    const int slot = k % depth;
    const uint32_t full = barrier_addr(smem, pipelink_gemm_full(), slot);
    const uint32_t empty = barrier_addr(smem, pipelink_gemm_empty(), slot);
    if (!wait(empty, ((k / depth) & 1) ^ 1)) return;
    plb::mbar_arrive_expect_tx(full, SlotBytes);
    const uint32_t dst = smem + pipelink_gemm_operands() + slot * SlotBytes;
    plb::tma_load_2d(dst, &p.a, full, k * TileK, m_blk * TileM);
    plb::tma_load_2d(dst + OperandBytes, &p.b, full, k * TileK, n_blk * TileN);
    plb::bulk_load(dst + 2 * OperandBytes, p.a_sc + (static_cast<size_t>(m_blk) * k_steps + k) * ScaleBytes, ScaleBytes, full);
    plb::bulk_load(dst + 2 * OperandBytes + ScaleBytes, p.b_sc + (static_cast<size_t>(n_blk) * k_steps + k) * ScaleBytes, ScaleBytes, full);
  }
}
#endif  // !PIPELINK_EMIT
