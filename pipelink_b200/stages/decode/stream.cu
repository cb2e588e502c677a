// Stage decode.stream: the producer warp of the decode interpreter. One lane walks the stage
// sequence of this CTA's instruction stream and issues the copies into the weights ring (untiled
// bulk copies with an evict-first L2 policy for weight rows, two TMA boxes for 128 tokens of K and
// V), never waiting for a dependency counter. Body: csrc/decode_roles.cuh:stream_role.
#include "decode.cuh"

extern "C" __device__ void decode_stream_role(const void* params, unsigned variant);
PL_STAGE("decode.stream", "1.0.0");
PL_PARAMS(DecStreamParams, map_k, map_v, args);
PL_ROLE(stream, decode_stream_role, 1);
DEC_TOPOLOGY();
PL_ENDPOINT(weights, decstage::weights(pl::produce, "stream"));
PL_ENDPOINT(instructions, decstage::instructions(pl::consume, "stream"));
PL_CLAIM_WARPS(pipelink_dec_warp_stream, stream, 1, 1);
DEC_CLAIM_RING();
DEC_CLAIM_INSTRUCTIONS();

#ifndef PIPELINK_EMIT
extern "C" __device__ void decode_stream_role(const void* raw_params, unsigned) {
  using namespace plb;
  using namespace plb::dec;
  const DecStreamParams& p = *static_cast<const DecStreamParams*>(raw_params);
  const DecodeGlobals g = reinterpret_cast<const DecodeGlobals&>(p.args);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = smem_u32(pl_smem);
  if ((threadIdx.x & 31) != 0) return;
  const int pos = *g.pos_dev;
  // the interpreter's threads copy the instruction words; wait (bounded) until they are there
  const bool local = g.num_instructions * kInstWords * 4 <= kInstSmemBytes;
  if (local && !mbar_wait(smem + 16u * static_cast<uint32_t>(pipelink_dec_inst_ready()), 0u, g.status, ST_TIMEOUT_FULL, 990)) return;
  const int* my = local ? reinterpret_cast<const int*>(pl_smem + pipelink_dec_inst())
                        : g.instructions + static_cast<size_t>(blockIdx.x) * g.num_instructions * 32;
  stream_role<decstage::LinkedLayout>(g, &p.map_k, &p.map_v, smem, my, local ? kInstWords : 32, pos);
}
#endif  // !PIPELINK_EMIT
