// Stage moe.fwd.epilogue.combine: moe.fwd.epilogue with the forward's tail in the same launch: when every
// CTA of this GPU has finished its down-projection tiles, and in a group every rank has said so through
// the group barrier's flags, the epilogue warps sum each token's top-k rows with its router weights. With
// this owner one launch is dispatch + gate/up + SwiGLU + down + combine push + group barrier + weighted
// epilogue: the whole device side of the reference's forward between its schedule and its return
// (campaigns/mok/port/framework/interp_fwd.cu:27-263 runs the same sequence as tasks of one launch).
#include "moe.cuh"

extern "C" __device__ void moe_fwd_epilogue_combine_role(const void* params, unsigned variant);
PL_STAGE("moe.fwd.epilogue.combine", "1.0.0");
PL_PARAMS(MoeFwdCombineParams, e, t);
PL_ROLE(epilogue, moe_fwd_epilogue_combine_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_ENDPOINT(hidden_ready, moe::hidden_ready(pl::produce, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();
MOE_CLAIM_STAGING();
MOE_CLAIM_HIDDEN_READY();
PL_CLAIM(gmem_counter, pipelink_moe_ctas_done, pl::units(1), 1);
PL_CLAIM(named_barrier, pipelink_moe_tail_barrier, pl::units(1), 1);

#ifndef PIPELINK_EMIT
#include "epilogue.cuh"
extern "C" __device__ void moe_fwd_epilogue_combine_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeFwdCombineParams& all = *static_cast<const MoeFwdCombineParams*>(raw_params);
  const MoeFwdEpilogueParams p = all.e;   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const EpilogueWarp e = epilogue_warp(smem, pl_smem, true);
  const bool ok = fwd_epilogue_tiles(p, e, smem);
  const MoeFwdTailParams t = all.t;
  fwd_tail(t, p.counters, p.g1.status, ok);
}
#endif  // !PIPELINK_EMIT
