// Stage moe.load: one elected lane of each CTA of a pair feeds the operands ring with TMA: its own
// 128 rows of A, its 128-row half of the pair's 256 weight rows, its A-scale block and both
// B-scale blocks; completion bytes of both CTAs are credited to the leader CTA's full barrier.
// Same role as the producer warp of csrc/grouped_gemm2.cu (the reference's GEMM owner keeps this
// role inside its package, campaigns/mok/port/gemm/gemm.cu:292-325; here it is an owner of its own).
#include "moe.cuh"

extern "C" __device__ void moe_load_role(const void* params, unsigned variant);
PL_STAGE("moe.load", "1.0.0");
PL_PARAMS(MoeLoadParams, a, b, sfa, sfb, g, counters);
PL_ROLE(load, moe_load_role, 1);
MOE_TOPOLOGY();
PL_ENDPOINT(operands, moe::operands(pl::produce, "load"));
PL_ENDPOINT(rows_ready, moe::rows_ready(pl::consume, "load"));
PL_CLAIM_WARPS(pipelink_moe_warp_load, load, 1, 1);
MOE_REGS_HELPER(load);
MOE_CLAIM_OPERANDS();
MOE_CLAIM_ROWS_READY();

#ifndef PIPELINK_EMIT
extern "C" __device__ void moe_load_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeLoadParams& p = *static_cast<const MoeLoadParams*>(raw_params);
  // the scalars are read once into registers: through the pointer the compiler would have to fetch
  // them from the parameter block again after every barrier operation of the K loop
  const MoeGeometry g = p.g;
  const unsigned* const counters = p.counters;
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const int lane = threadIdx.x & 31;
  const Walk w = make_walk(g, lane, blockIdx.x == 0);
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  if (lane == 0) {
    plb::prefetch_tensormap(&p.a);
    plb::prefetch_tensormap(&p.b);
    plb::prefetch_tensormap(&p.sfa);
    plb::prefetch_tensormap(&p.sfb);
  }
  Ring ring;
  ring.init(smem);
  const uint32_t leader_delta = plb::mapa_shared(ring.full0, 0) - ring.full0;   // the leader CTA's copy of a barrier
  const int total_tiles = __shfl_sync(0xFFFFFFFFu, w.total_tiles, 0);
  bool ok = true;
  for (int tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
    const Tile t = decode(g, w, tile, static_cast<int>(cta_rank));
    const int a_blk = __shfl_sync(0xFFFFFFFFu, t.a_blk, 0), b_blk0 = __shfl_sync(0xFFFFFFFFu, t.b_blk0, 0);
    const int b_blk = b_blk0 + static_cast<int>(cta_rank);
    if (counters != nullptr) {
      // rows pulled by the comm owner are usable once their tile's count is complete; then order
      // the TMA reads after the count was observed
      ok = wait_count_warp(counters + pipelink_moe_rows_ready() + (a_blk >> 1), 256u, g.status, 311, lane);
      if (!ok) break;
    }
    ok = load_k_loop(ring, g.k_steps, leader_delta, &p.a, &p.b, &p.sfa, &p.sfb, a_blk, b_blk, b_blk0, g.status);
  }
  if (!ok) {
    // give copies already in flight time to land before this CTA can exit
    const long long t0 = clock64();
    while (clock64() - t0 < 200000LL) {
    }
  }
}
#endif  // !PIPELINK_EMIT
