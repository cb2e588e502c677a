// Stage gemm.mma: one elected lane issues block-scaled tcgen05 MMAs into tensor memory.
#include "gemm3.cuh"

extern "C" __device__ void gemm_mma_role(const void* params, unsigned variant);
PL_STAGE("gemm.mma", "1.0.0");
PL_PARAMS(Gemm3MmaParams, K);
PL_ROLE(mma, gemm_mma_role, 1);
GEMM3_TOPOLOGY();
PL_ENDPOINT(operands, gemm3::operands(pl::consume, "mma"));
PL_ENDPOINT(accumulator, gemm3::accumulator(pl::produce, "mma"));
PL_CLAIM_WARPS(pipelink_gemm_warp_mma, mma, 1, 1);
GEMM3_CLAIM_OPERANDS();
GEMM3_CLAIM_ACCUMULATOR();
PL_CLAIM(tmem, pipelink_gemm_sf, pl::per("pipelink_gemm_depth", gemm3::ScaleColsPerSlot), 32);

#ifndef PIPELINK_EMIT
extern "C" __device__ void gemm_mma_role(const void* raw_params, unsigned) {
  using namespace gemm3;
  const Gemm3MmaParams& p = *static_cast<const Gemm3MmaParams*>(raw_params);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  // the whole warp walks the loop (operands warp-uniform, computed once per warp); one elected lane issues
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot()), 0);
  const int depth = pipelink_gemm_depth();
  const int k_steps = p.K / TileK;
  const uint32_t d_tmem = tmem + pipelink_gemm_acc();
  constexpr uint32_t idesc = plb::idesc_mxf8(TileM, TileN);
  for (int k = 0; k < k_steps; ++k) {
    const int slot = k % depth;
    if (!__all_sync(0xFFFFFFFFu, wait(barrier_addr(smem, pipelink_gemm_full(), slot), (k / depth) & 1))) return;
    plb::tc_fence_after();
    const uint32_t base = smem + pipelink_gemm_operands() + slot * SlotBytes;
    const uint32_t sfa = tmem + pipelink_gemm_sf() + slot * ScaleColsPerSlot, sfb = sfa + 4;
    const uint64_t sfd_a = plb::smem_desc(base + 2 * OperandBytes, plb::kDescScale);
    const uint64_t sfd_b = plb::smem_desc(base + 2 * OperandBytes + ScaleBytes, plb::kDescScale);
    const uint64_t adesc = plb::smem_desc(base, plb::kDescSw128KMajor);
    const uint64_t bdesc = plb::smem_desc(base + OperandBytes, plb::kDescSw128KMajor);
    const uint32_t empty = barrier_addr(smem, pipelink_gemm_empty(), slot);
    const uint32_t first = k != 0 ? 1u : 0u;
    if (plb::elect_one_sync()) {
      plb::tc_cp_32x128b_warpx4(sfa, sfd_a);
      plb::tc_cp_32x128b_warpx4(sfb, sfd_b);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        plb::tc_mma_mxf8(d_tmem, adesc + 2 * j, bdesc + 2 * j, plb::idesc_with_sf(idesc, j), sfa, sfb, j != 0 ? 1u : first);
      plb::tc_commit(empty);
    }
    __syncwarp();
  }
  if (plb::elect_one_sync()) plb::tc_commit(barrier_addr(smem, pipelink_gemm_acc_ready()));
  __syncwarp();
}
#endif  // !PIPELINK_EMIT
