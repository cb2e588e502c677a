// Stage moe.fwd.mma: the MMA issuer of the one-launch forward. The same issue loop as moe.mma over
// the two-pass tile list: K steps per tile follow the pass (H / 128 for the gate/up projection,
// I / 128 for the down projection); ring, scale columns and accumulator hand-off are unchanged.
#include "moe.cuh"

extern "C" __device__ void moe_fwd_mma_role(const void* params, unsigned variant);
PL_STAGE("moe.fwd.mma", "1.0.0");
PL_PARAMS(MoeFwdMmaParams, g1, g2);
PL_ROLE(mma, moe_fwd_mma_role, 1);
MOE_TOPOLOGY();
PL_ENDPOINT(operands, moe::operands(pl::consume, "mma"));
PL_ENDPOINT(accumulator, moe::accumulator(pl::produce, "mma"));
PL_CLAIM_WARPS(pipelink_moe_warp_mma, mma, 1, 1);
MOE_REGS_HELPER(mma);
MOE_CLAIM_OPERANDS();
MOE_CLAIM_ACCUMULATOR();
PL_CLAIM(tmem, pipelink_moe_sfcols, pl::per("pipelink_moe_depth", moe::SfColsPerSlot), 32);
PL_CLAIM_EX(mbarrier, pipelink_moe_drain, pl::units(1), 1, "init_count", 1);

#ifndef PIPELINK_EMIT
extern "C" __device__ void moe_fwd_mma_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeFwdMmaParams p = *static_cast<const MoeFwdMmaParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const int lane = threadIdx.x & 31;
  const FwdWalk f = make_fwd_walk(p.g1, p.g2, lane, false);
  if (lane != 0 || plb::cluster_ctarank() != 0) return;
  plb::Status* const status = p.g1.status;
  const int k_steps1 = p.g1.k_steps, k_steps2 = p.g2.k_steps;
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot());
  const uint32_t d_tmem = tmem + pipelink_moe_acc();
  const int depth = pipelink_moe_depth();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  constexpr uint32_t idesc = plb::idesc_mxf8(256, 256);
  const uint32_t acc_full_own = bar(smem, pipelink_moe_acc_full());
  const uint32_t acc_full_peer = plb::mapa_shared(acc_full_own, 1);
  int stage = 0;
  uint32_t phase = 0, acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < f.total && ok; tile += num_pairs) {
    const int k_steps = tile >= f.tiles1 ? k_steps2 : k_steps1;
    if (!plb::mbar_wait(bar(smem, pipelink_moe_acc_empty()), acc_phase ^ 1u, status, plb::ST_TIMEOUT_TMEM_EMPTY, 0)) {
      ok = false;
      break;
    }
    plb::tc_fence_after();
    for (int kb = 0; kb < k_steps; ++kb) {
      if (!plb::mbar_wait(bar(smem, pipelink_moe_full(), stage), phase, status, plb::ST_TIMEOUT_FULL, stage)) {
        ok = false;
        break;
      }
      plb::tc_fence_after();
      const uint32_t slot = smem + pipelink_moe_operands() + stage * SlotBytes;
      const uint32_t sfa_t = tmem + pipelink_moe_sfcols() + stage * SfColsPerSlot, sfb_t = sfa_t + 4;
      plb::tc_cp_32x128b_warpx4_pair(sfa_t, plb::smem_desc(slot + OffSf, plb::kDescScale));
      plb::tc_cp_32x128b_warpx4_pair(sfb_t, plb::smem_desc(slot + OffSf + SfBytes, plb::kDescScale));
      plb::tc_cp_32x128b_warpx4_pair(sfb_t + 4, plb::smem_desc(slot + OffSf + 2 * SfBytes, plb::kDescScale));
      const uint64_t adesc = plb::smem_desc(slot + OffA, plb::kDescSw128KMajor);
      const uint64_t bdesc = plb::smem_desc(slot + OffB, plb::kDescSw128KMajor);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        plb::tc_mma_mxf8_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, plb::idesc_with_sf(idesc, k), sfa_t, sfb_t,
                              (kb | k) != 0 ? 1u : 0u);
      const uint32_t empty_own = bar(smem, pipelink_moe_empty(), stage);
      plb::tc_commit_pair(empty_own);
      plb::tc_commit_pair(plb::mapa_shared(empty_own, 1));
      if (++stage == depth) { stage = 0; phase ^= 1u; }
    }
    if (!ok) break;
    plb::tc_commit_pair(acc_full_own);
    plb::tc_commit_pair(acc_full_peer);
    acc_phase ^= 1u;
  }
  if (!ok) {
    // MMAs in flight are committed and waited for (with a limit) before the CTA may free tensor memory
    const uint32_t drain = bar(smem, pipelink_moe_drain());
    plb::tc_commit_pair(drain);
    const long long t0 = clock64();
    while (!plb::mbar_try_wait(drain, 0)) {
      if (clock64() - t0 > 20000000LL) break;
    }
  }
}
#endif  // !PIPELINK_EMIT
