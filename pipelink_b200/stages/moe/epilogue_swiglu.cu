// Stage moe.epilogue.swiglu-mxfp8: the gate/up projection's consumer. Eight warps per CTA (two per
// 32-lane quadrant of tensor memory) drain 128 accumulator columns each into registers, release
// the accumulator at once so the next tile's MMAs overlap the arithmetic, then compute
// hidden = bf16(silu(bf16 gate) * bf16 up), requantise 32-element blocks to MXFP8 and store 64
// E4M3 bytes and two scale bytes per row. The reference runs this arithmetic as its act owner
// (campaigns/mok/port/act/act.cu:100-178) on bf16 gate / up written by the GEMM owner; here the
// accumulator channel hands it the tile in tensor memory.
#include "moe.cuh"

extern "C" __device__ void moe_epilogue_swiglu_mxfp8_role(const void* params, unsigned variant);
PL_STAGE("moe.epilogue.swiglu-mxfp8", "1.0.0");
PL_PARAMS(MoeSwigluParams, g, out, out_sc, out_cols, limit);
PL_ROLE(epilogue, moe_epilogue_swiglu_mxfp8_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();

#ifndef PIPELINK_EMIT
#include "epilogue.cuh"
extern "C" __device__ void moe_epilogue_swiglu_mxfp8_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeSwigluParams p = *static_cast<const MoeSwigluParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const EpilogueWarp e = epilogue_warp(smem, pl_smem, false);
  const Walk w = make_walk(p.g, e.lane, false);
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  uint32_t acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < w.total_tiles && ok; tile += num_pairs) {
    const Tile t = decode(p.g, w, tile, static_cast<int>(e.cta_rank));
    if (!plb::mbar_wait(bar(smem, pipelink_moe_acc_full()), acc_phase, p.g.status, plb::ST_TIMEOUT_TMEM_FULL, 0)) ok = false;
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (!ok) break;
    plb::tc_fence_after();
    swiglu_tile(e, t, p.out, p.out_sc, p.out_cols, p.limit);
    acc_phase ^= 1u;
  }
}
#endif  // !PIPELINK_EMIT
