// Stage attn.softmax.softcap: attn.softmax with the tanh soft cap on the scaled scores
// (score = c * tanh(s * scale / c); the reference's score-modifier stage variant).
#include "attention.cuh"
ATTN_SOFTMAX_STAGE("attn.softmax.softcap", attn_softmax_softcap_role);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_softmax_softcap_role(const void* raw, unsigned) {
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  plb::attn::softmax_role<attnstage::LinkedLayout, true>(attnstage::params_of(static_cast<const AttnRoleParams*>(raw)->p),
                                                        plb::smem_u32(pl_smem), attnstage::tmem_base(pl_smem));
}
#endif
