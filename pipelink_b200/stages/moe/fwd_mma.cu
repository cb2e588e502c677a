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
  if (plb::cluster_ctarank() != 0) return;
  plb::Status* const status = p.g1.status;
  const int k_steps1 = p.g1.k_steps, k_steps2 = p.g2.k_steps;
  const uint32_t smem = plb::smem_u32(pl_smem);
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot()), 0);
  const uint32_t d_tmem = tmem + pipelink_moe_acc();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t acc_full_own = bar(smem, pipelink_moe_acc_full());
  const uint32_t peer_delta = plb::mapa_shared(acc_full_own, 1) - acc_full_own;   // the same CTA-relative offset in the peer
  const uint32_t acc_empty = bar(smem, pipelink_moe_acc_empty());
  const int total = __shfl_sync(0xFFFFFFFFu, f.total, 0), tiles1 = __shfl_sync(0xFFFFFFFFu, f.tiles1, 0);
  Ring ring;
  ring.init(smem);
  uint32_t acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < total && ok; tile += num_pairs) {
    const int k_steps = tile >= tiles1 ? k_steps2 : k_steps1;
    ok = __all_sync(0xFFFFFFFFu, plb::mbar_wait(acc_empty, acc_phase ^ 1u, status, plb::ST_TIMEOUT_TMEM_EMPTY, 0));
    if (!ok) break;
    plb::tc_fence_after();
    ok = mma_k_loop(ring, k_steps, tmem, d_tmem, peer_delta, status);
    if (!ok) break;
    if (plb::elect_one_sync()) {
      plb::tc_commit_pair(acc_full_own);
      plb::tc_commit_pair(acc_full_own + peer_delta);
    }
    __syncwarp();
    acc_phase ^= 1u;
  }
  if (!ok && lane == 0) {
    // MMAs in flight are committed and waited for (with a limit) before the CTA may free tensor memory
    const uint32_t drain = bar(smem, pipelink_moe_drain());
    plb::tc_commit_pair(drain);
    const long long t0 = clock64();
    while (!plb::mbar_try_wait(drain, 0)) {
      if (clock64() - t0 > 20000000LL) break;
    }
  }
  __syncwarp();
}
#endif  // !PIPELINK_EMIT
