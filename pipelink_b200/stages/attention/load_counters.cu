// Stage attn.load.counters: the TMA producer under context parallelism: a key block is read once its
// readiness counter (written by the ranks that push the block) has reached this step's target.
#include "attention.cuh"
ATTN_LOAD_STAGE("attn.load.counters", attn_load_counters_role);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_load_counters_role(const void* raw, unsigned) {
  const AttnLoadParams& lp = *static_cast<const AttnLoadParams*>(raw);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  if (threadIdx.x % 32 == 0) {
    plb::prefetch_tensormap(&lp.map_q);
    plb::prefetch_tensormap(&lp.map_k);
    plb::prefetch_tensormap(&lp.map_v);
  }
  plb::attn::load_role<attnstage::LinkedLayout, true>(&lp.map_q, &lp.map_k, &lp.map_v, attnstage::params_of(lp.p), plb::smem_u32(pl_smem));
}
#endif
