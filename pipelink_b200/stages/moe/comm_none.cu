// Stage moe.comm.none: the comm role of a composition whose operand rows are already in place
// (single-rank forward, or a pull kernel in front of the GEMM). The two warps complete the reg
// group of the load and MMA owners and do nothing else.
#include "moe.cuh"

extern "C" __device__ void moe_comm_none_role(const void*, unsigned) {}
