// Stage attn.gather.none: the two spare warps of the first warpgroup when no K/V exchange runs in the launch.
#include "attention.cuh"
ATTN_GATHER_STAGE("attn.gather.none", attn_gather_none_role);
#ifndef PIPELINK_EMIT
extern "C" __device__ void attn_gather_none_role(const void*, unsigned) {}
#endif
