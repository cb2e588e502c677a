// Stage moe.comm.none: the comm role of a composition whose operand rows are already in place
// (single-rank forward, or a pull kernel in front of the GEMM). The two warps complete the reg
// group of the load and MMA owners and do nothing else.
#include "moe.cuh"

extern "C" __device__ void moe_comm_none_role(const void* params, unsigned variant);
PL_STAGE("moe.comm.none", "1.0.0");
PL_NO_PARAMS();
PL_ROLE(comm, moe_comm_none_role, 2);
MOE_TOPOLOGY();
PL_ENDPOINT(rows_ready, moe::rows_ready(pl::produce, "comm"));
PL_CLAIM_WARPS(pipelink_moe_warp_comm, comm, 2, 1);
MOE_REGS_HELPER(comm);
MOE_CLAIM_ROWS_READY();

#ifndef PIPELINK_EMIT
extern "C" __device__ void moe_comm_none_role(const void*, unsigned) {}
#endif  // !PIPELINK_EMIT
