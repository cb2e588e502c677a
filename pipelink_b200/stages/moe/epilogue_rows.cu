// Stage moe.epilogue.rows-bf16: the down projection's consumer. Eight warps per CTA drain the
// accumulator into registers, release it, round to bf16 and store whole rows: to
// out[dest_row[p]] on this GPU, or, with a table of per-rank bases, into the home rank's buffer over
// NVLink (the combine push: the reference's combine_kernel, campaigns/mok/port/comm/comm.cu:124-129,
// fed by its GEMM owner's FWD_ROUTED_DOWN case, campaigns/mok/port/gemm/gemm.cu:158-162). Rows pass
// through 2 KiB of shared memory per warp, eight at a time, so that every store instruction of a
// warp writes two 256-byte row segments.
#include "moe.cuh"

extern "C" __device__ void moe_epilogue_rows_bf16_role(const void* params, unsigned variant);
PL_STAGE("moe.epilogue.rows-bf16", "1.0.0");
PL_PARAMS(MoeRowsParams, g, out, out_peers, dest_row, peer_rank, out_cols);
PL_ROLE(epilogue, moe_epilogue_rows_bf16_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();
MOE_CLAIM_STAGING();

#ifndef PIPELINK_EMIT
#include "epilogue.cuh"
extern "C" __device__ void moe_epilogue_rows_bf16_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeRowsParams p = *static_cast<const MoeRowsParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const EpilogueWarp e = epilogue_warp(smem, pl_smem, true);
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
    rows_tile(e, t, p.out, p.out_peers, p.dest_row, p.peer_rank, p.out_cols);
    acc_phase ^= 1u;
  }
}
#endif  // !PIPELINK_EMIT
