// Stage moe.fwd.load: the TMA producer of the one-launch forward. One tile list holds the gate/up
// projection's tiles followed by the down projection's; the operands of a pass-2 tile are the hidden
// rows this same launch wrote, so before its first read of a row tile the owner waits for the tile's
// `hidden_ready` count (every epilogue warp of every pass-1 column tile has stored and released) and
// orders its async-proxy reads after the count. The reference runs its MoE forward as one
// persistent launch the same way, its GEMM owner moving from the FWD_ROUTED_GATE_UP case to
// FWD_ROUTED_DOWN behind its activation owner (campaigns/mok/port/gemm/gemm.cu:150-170,
// campaigns/mok/port/pipelines/fwd.json).
#include "moe.cuh"

extern "C" __device__ void moe_fwd_load_role(const void* params, unsigned variant);
PL_STAGE("moe.fwd.load", "1.0.0");
PL_PARAMS(MoeFwdLoadParams, a1, b1, sfa1, sfb1, a2, b2, sfa2, sfb2, g1, g2, counters, wait_rows_ready);
PL_ROLE(load, moe_fwd_load_role, 1);
MOE_TOPOLOGY();
PL_ENDPOINT(operands, moe::operands(pl::produce, "load"));
PL_ENDPOINT(rows_ready, moe::rows_ready(pl::consume, "load"));
PL_ENDPOINT(hidden_ready, moe::hidden_ready(pl::consume, "load"));
PL_CLAIM_WARPS(pipelink_moe_warp_load, load, 1, 1);
MOE_REGS_HELPER(load);
MOE_CLAIM_OPERANDS();
MOE_CLAIM_ROWS_READY();
MOE_CLAIM_HIDDEN_READY();

#ifndef PIPELINK_EMIT
extern "C" __device__ void moe_fwd_load_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeFwdLoadParams& p = *static_cast<const MoeFwdLoadParams*>(raw_params);
  // scalars in registers (the tensor maps stay in the parameter block, where TMA wants them)
  const MoeGeometry g1 = p.g1, g2 = p.g2;
  const unsigned* const counters = p.counters;
  const bool wait_rows = p.wait_rows_ready != 0;
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const int lane = threadIdx.x & 31;
  const FwdWalk f = make_fwd_walk(g1, g2, lane, blockIdx.x == 0);
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  if (lane == 0) {
    plb::prefetch_tensormap(&p.a1);
    plb::prefetch_tensormap(&p.b1);
    plb::prefetch_tensormap(&p.sfa1);
    plb::prefetch_tensormap(&p.sfb1);
  }
  // every epilogue warp of the pair (16) counts once per pass-1 column tile
  const unsigned hidden_target = 16u * static_cast<unsigned>(g1.n_tiles);
  Ring ring;
  ring.init(smem);
  const uint32_t leader_delta = plb::mapa_shared(ring.full0, 0) - ring.full0;   // the leader CTA's copy of a barrier
  const int total = __shfl_sync(0xFFFFFFFFu, f.total, 0), tiles1 = __shfl_sync(0xFFFFFFFFu, f.tiles1, 0);
  bool ok = true;
  for (int tile = pair_id; tile < total && ok; tile += num_pairs) {
    const bool second = tile >= tiles1;
    const MoeGeometry& g = second ? g2 : g1;
    const Tile t = decode(g, second ? f.w2 : f.w1, second ? tile - tiles1 : tile, static_cast<int>(cta_rank));
    const int a_blk = __shfl_sync(0xFFFFFFFFu, t.a_blk, 0), b_blk0 = __shfl_sync(0xFFFFFFFFu, t.b_blk0, 0);
    const int b_blk = b_blk0 + static_cast<int>(cta_rank);
    const CUtensorMap* const ma = second ? &p.a2 : &p.a1;
    const CUtensorMap* const mb = second ? &p.b2 : &p.b1;
    const CUtensorMap* const msa = second ? &p.sfa2 : &p.sfa1;
    const CUtensorMap* const msb = second ? &p.sfb2 : &p.sfb1;
    if (second)
      ok = wait_count_warp(counters + pipelink_moe_hidden_ready() + (a_blk >> 1), hidden_target, g.status, 312, lane);
    else if (wait_rows)
      ok = wait_count_warp(counters + pipelink_moe_rows_ready() + (a_blk >> 1), 256u, g.status, 311, lane);
    if (!ok) break;
    ok = load_k_loop(ring, g.k_steps, leader_delta, ma, mb, msa, msb, a_blk, b_blk, b_blk0, g.status);
  }
  if (!ok) {
    // give copies already in flight time to land before this CTA can exit
    const long long t0 = clock64();
    while (clock64() - t0 < 200000LL) {
    }
  }
}
#endif  // !PIPELINK_EMIT
