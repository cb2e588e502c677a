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
  // the whole warp walks the loop (coordinates and addresses warp-uniform); one elected lane issues the copies
  const uint32_t smem = plb::smem_u32(pl_smem);
  const int depth = pipelink_gemm_depth();
  const int k_steps = p.K / TileK;
  const int m_blk = blockIdx.x, n_blk = blockIdx.y;
  for (int k = 0; k < k_steps; ++k) {
    const int slot = k % depth;
    const uint32_t full = barrier_addr(smem, pipelink_gemm_full(), slot);
    const uint32_t empty = barrier_addr(smem, pipelink_gemm_empty(), slot);
    if (!__all_sync(0xFFFFFFFFu, wait(empty, ((k / depth) & 1) ^ 1))) return;
    const uint32_t dst = smem + pipelink_gemm_operands() + slot * SlotBytes;
    const uint8_t* const sc_a = p.a_sc + (static_cast<size_t>(m_blk) * k_steps + k) * ScaleBytes;
    const uint8_t* const sc_b = p.b_sc + (static_cast<size_t>(n_blk) * k_steps + k) * ScaleBytes;
    if (plb::elect_one_sync()) {
      plb::mbar_arrive_expect_tx(full, SlotBytes);
      plb::tma_load_2d(dst, &p.a, full, k * TileK, m_blk * TileM);
      plb::tma_load_2d(dst + OperandBytes, &p.b, full, k * TileK, n_blk * TileN);
      plb::bulk_load(dst + 2 * OperandBytes, sc_a, ScaleBytes, full);
      plb::bulk_load(dst + 2 * OperandBytes + ScaleBytes, sc_b, ScaleBytes, full);
    }
    __syncwarp();
  }
}
#endif  // !PIPELINK_EMIT
