// Stage attn.softmax: online softmax in the base-2 domain with deferred rescale, causal and
// sliding-window masks, final O / l and LSE; eight warps, four per head of the pair.
#include "attention.cuh"
ATTN_SOFTMAX_STAGE("attn.softmax", attn_softmax_role);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_softmax_role(const void* raw, unsigned) {
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  plb::attn::softmax_role<attnstage::LinkedLayout, false>(attnstage::params_of(static_cast<const AttnRoleParams*>(raw)->p),
                                                         plb::smem_u32(pl_smem), attnstage::tmem_base(pl_smem));
}
#endif
