// Stage moe.fwd.epilogue: the accumulator consumer of the one-launch forward. A pass-1 tile goes
// through the SwiGLU + MXFP8 requantise body into the hidden rows and then counts on the row tile's
// `hidden_ready` slot (stores, fence, one release per warp); a pass-2 tile goes through the bf16
// row-store body (local placement or the combine push to the home ranks). The reference's forward
// keeps activation and combine in the same launch as its GEMM owner (campaigns/mok/port/act/act.cu,
// campaigns/mok/port/comm/comm.cu:124-129).
#include "moe.cuh"

extern "C" __device__ void moe_fwd_epilogue_role(const void* params, unsigned variant);
PL_STAGE("moe.fwd.epilogue", "1.0.0");
PL_PARAMS(MoeFwdEpilogueParams, g1, g2, hidden, hidden_sc, out, out_peers, dest_row, peer_rank, counters, hidden_cols, out_cols,
          limit);
PL_ROLE(epilogue, moe_fwd_epilogue_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_ENDPOINT(hidden_ready, moe::hidden_ready(pl::produce, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();
MOE_CLAIM_STAGING();
MOE_CLAIM_HIDDEN_READY();

#ifndef PIPELINK_EMIT
#include "epilogue.cuh"
extern "C" __device__ void moe_fwd_epilogue_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeFwdEpilogueParams p = *static_cast<const MoeFwdEpilogueParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const EpilogueWarp e = epilogue_warp(smem, pl_smem, true);
  fwd_epilogue_tiles(p, e, smem);
}
#endif  // !PIPELINK_EMIT
