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
namespace {
// wait (bounded) until a grid-scoped counter reaches `target`, then order TMA reads after it
__device__ __forceinline__ bool wait_count(const unsigned* flag, unsigned target, plb::Status* status, int where) {
  const long long t0 = clock64();
  while (plb::ld_acquire_gpu_u32(flag) < target) {
    if (clock64() - t0 > plb::kWaitBudgetCycles / 2 || plb::ld_volatile_i32(&status->code) != 0) {
      plb::report_failure(status, plb::ST_TIMEOUT_COUNTER, where, plb::ld_acquire_gpu_u32(flag), target);
      return false;
    }
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}
}  // namespace

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
  if (lane != 0) return;
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int depth = pipelink_moe_depth();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  plb::prefetch_tensormap(&p.a1);
  plb::prefetch_tensormap(&p.b1);
  plb::prefetch_tensormap(&p.sfa1);
  plb::prefetch_tensormap(&p.sfb1);
  // every epilogue warp of the pair (16) counts once per pass-1 column tile
  const unsigned hidden_target = 16u * static_cast<unsigned>(g1.n_tiles);
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < f.total && ok; tile += num_pairs) {
    const bool second = tile >= f.tiles1;
    const MoeGeometry& g = second ? g2 : g1;
    const Tile t = decode(g, second ? f.w2 : f.w1, second ? tile - f.tiles1 : tile, static_cast<int>(cta_rank));
    const int b_blk = t.b_blk0 + static_cast<int>(cta_rank);
    const CUtensorMap* const ma = second ? &p.a2 : &p.a1;
    const CUtensorMap* const mb = second ? &p.b2 : &p.b1;
    const CUtensorMap* const msa = second ? &p.sfa2 : &p.sfa1;
    const CUtensorMap* const msb = second ? &p.sfb2 : &p.sfb1;
    if (second)
      ok = wait_count(counters + pipelink_moe_hidden_ready() + (t.a_blk >> 1), hidden_target, g.status, 312);
    else if (wait_rows)
      ok = wait_count(counters + pipelink_moe_rows_ready() + (t.a_blk >> 1), 256u, g.status, 311);
    if (!ok) break;
    const int k_steps = g.k_steps;
    for (int kb = 0; kb < k_steps; ++kb) {
      if (!plb::mbar_wait(bar(smem, pipelink_moe_empty(), stage), phase ^ 1u, g.status, plb::ST_TIMEOUT_EMPTY, stage)) {
        ok = false;
        break;
      }
      const uint32_t full = plb::mapa_shared(bar(smem, pipelink_moe_full(), stage), 0);
      plb::mbar_arrive_expect_tx_cluster(full, SlotTx);
      const uint32_t slot = smem + pipelink_moe_operands() + stage * SlotBytes;
      plb::tma_load_2d_pair(slot + OffA, ma, full, kb * 128, t.a_blk * 128);
      plb::tma_load_2d_pair(slot + OffB, mb, full, kb * 128, b_blk * 128);
      plb::tma_load_2d_pair(slot + OffSf, msa, full, 0, t.a_blk * k_steps + kb);
      plb::tma_load_2d_pair(slot + OffSf + SfBytes, msb, full, 0, t.b_blk0 * k_steps + kb);
      plb::tma_load_2d_pair(slot + OffSf + 2 * SfBytes, msb, full, 0, (t.b_blk0 + 1) * k_steps + kb);
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
