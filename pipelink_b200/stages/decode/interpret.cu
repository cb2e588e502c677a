// Stage decode.interpret: the sixteen consumer warps of the decode interpreter: per instruction the
// dependency wait, the matvec partial sums out of the weights ring, the op's epilogue (RoPE + KV
// append, residual add, SiLU * up, logits + argmax), partial attention with its in-launch merge,
// the greedy sample, and the dependency signal. Body: csrc/decode_roles.cuh:interpret_role.
#include "decode.cuh"

extern "C" __device__ void decode_interpret_role(const void* params, unsigned variant);
PL_STAGE("decode.interpret", "1.0.0");
PL_PARAMS(DecInterpretParams, args);
PL_ROLE(interpret, decode_interpret_role, 16);
DEC_TOPOLOGY();
PL_ENDPOINT(weights, decstage::weights(pl::consume, "interpret"));
PL_ENDPOINT(instructions, decstage::instructions(pl::produce, "interpret"));
PL_CLAIM_WARPS(pipelink_dec_warp_interpret, interpret, 16, 4);
DEC_CLAIM_RING();
DEC_CLAIM_INSTRUCTIONS();
PL_CLAIM(smem, pipelink_dec_partial, pl::units(decstage::PartialBytes), 16);
PL_CLAIM(smem, pipelink_dec_scratch, pl::units(decstage::ScratchBytes), 16);
// the interpreter's warps meet at named barrier 1 (bar.sync 1, 512); barrier 0 is the dispatch kernel's
PL_CLAIM_EX(named_barrier, pipelink_dec_named_barrier, pl::units(1), 1, "absolute_base", 1);

#ifndef PIPELINK_EMIT
extern "C" __device__ void decode_interpret_role(const void* raw_params, unsigned) {
  using namespace plb;
  using namespace plb::dec;
  const DecodeGlobals g = reinterpret_cast<const DecodeGlobals&>(static_cast<const DecInterpretParams*>(raw_params)->args);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = smem_u32(pl_smem);
  const int pos = *g.pos_dev;
  int istride;
  const int* my = stage_instructions(g, reinterpret_cast<int*>(pl_smem + pipelink_dec_inst()), threadIdx.x, kConsumers, istride);
  consumer_sync();
  if (threadIdx.x == 0 && istride != 32) mbar_arrive(smem + 16u * static_cast<uint32_t>(pipelink_dec_inst_ready()));
  interpret_role<decstage::LinkedLayout>(g, pl_smem, smem, my, istride, pos);
}
#endif  // !PIPELINK_EMIT
