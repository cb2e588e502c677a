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
  if (lane != 0) return;
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int depth = pipelink_moe_depth();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  plb::prefetch_tensormap(&p.a);
  plb::prefetch_tensormap(&p.b);
  plb::prefetch_tensormap(&p.sfa);
  plb::prefetch_tensormap(&p.sfb);
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < w.total_tiles && ok; tile += num_pairs) {
    const Tile t = decode(g, w, tile, static_cast<int>(cta_rank));
    const int b_blk = t.b_blk0 + static_cast<int>(cta_rank);
    if (counters != nullptr) {
      // rows pulled by the comm owner are usable once their tile's count is complete; then order
      // the TMA reads after the count was observed
      const unsigned* flag = counters + pipelink_moe_rows_ready() + (t.a_blk >> 1);
      const long long t0 = clock64();
      while (plb::ld_acquire_gpu_u32(flag) < 256u) {
        if (clock64() - t0 > plb::kWaitBudgetCycles / 2 || plb::ld_volatile_i32(&g.status->code) != 0) {
          plb::report_failure(g.status, plb::ST_TIMEOUT_COUNTER, 311, plb::ld_acquire_gpu_u32(flag), 256u);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    for (int kb = 0; kb < g.k_steps; ++kb) {
      if (!plb::mbar_wait(bar(smem, pipelink_moe_empty(), stage), phase ^ 1u, g.status, plb::ST_TIMEOUT_EMPTY, stage)) {
        ok = false;
        break;
      }
      const uint32_t full = plb::mapa_shared(bar(smem, pipelink_moe_full(), stage), 0);
      plb::mbar_arrive_expect_tx_cluster(full, SlotTx);
      const uint32_t slot = smem + pipelink_moe_operands() + stage * SlotBytes;
      plb::tma_load_2d_pair(slot + OffA, &p.a, full, kb * 128, t.a_blk * 128);
      plb::tma_load_2d_pair(slot + OffB, &p.b, full, kb * 128, b_blk * 128);
      plb::tma_load_2d_pair(slot + OffSf, &p.sfa, full, 0, t.a_blk * g.k_steps + kb);
      plb::tma_load_2d_pair(slot + OffSf + SfBytes, &p.sfb, full, 0, t.b_blk0 * g.k_steps + kb);
      plb::tma_load_2d_pair(slot + OffSf + 2 * SfBytes, &p.sfb, full, 0, (t.b_blk0 + 1) * g.k_steps + kb);
      if (++stage == depth) { stage = 0; phase ^= 1u; }
    }
  }
  if (!ok) {
    // give copies already in flight time to land before this CTA can exit
    const long long t0 = clock64();
    while (clock64() - t0 < 200000LL) {
    }
  }
}
#endif  // !PIPELINK_EMIT
