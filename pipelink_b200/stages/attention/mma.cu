// Stage attn.mma: the tcgen05 issuer of the prefill attention image: S_t = Q_t K^T into the scores
// slots, O_t += P_t V with P read from tensor memory, per block P0 V, Q0 K'^T, P1 V, Q1 K'^T.
#include "attention.cuh"
extern "C" __device__ void attn_mma_role(const void* params, unsigned variant);
PL_STAGE("attn.mma", "1.0.0");
PL_PARAMS(AttnRoleParams, p);
PL_ROLE(mma, attn_mma_role, 1);
ATTN_TOPOLOGY();
PL_ENDPOINT(q_tiles, attnstage::q_tiles(pl::consume, "mma"));
PL_ENDPOINT(k_tiles, attnstage::k_tiles(pl::consume, "mma"));
PL_ENDPOINT(v_tiles, attnstage::v_tiles(pl::consume, "mma"));
PL_ENDPOINT(scores, attnstage::scores(pl::produce, "mma"));
PL_ENDPOINT(output, attnstage::output(pl::produce, "mma"));
PL_CLAIM_WARPS(pipelink_attn_warp_mma, mma, 1, 1);
ATTN_CLAIM_TILES();
ATTN_CLAIM_ACCUM();
PL_CLAIM_EX(mbarrier, pipelink_attn_drain, pl::units(1), 1, "init_count", 1);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_mma_role(const void* raw, unsigned) {
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  plb::attn::mma_role<attnstage::LinkedLayout>(attnstage::params_of(static_cast<const AttnRoleParams*>(raw)->p), plb::smem_u32(pl_smem),
                                              attnstage::tmem_base(pl_smem));
}
#endif
