// Stage attn.gather.push: the context-parallel K/V exchange inside the attention launch: the two warps
// take tickets of one piece of one 128-token K/V block for one consumer rank from a global counter,
// copy the piece into that rank's gathered buffers and count it into its readiness counter.
#include "attention.cuh"
ATTN_GATHER_STAGE("attn.gather.push", attn_gather_push_role);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_gather_push_role(const void* raw, unsigned) {
  const plb::AttnParams& p = attnstage::params_of(static_cast<const AttnRoleParams*>(raw)->p);
  if (p.push_k != nullptr) plb::attn::gather_role(p);
}
#endif
