// Stage moe.epilogue.swiglu-mxfp8: the gate/up projection's consumer. Eight warps per CTA (two per
// 32-lane quadrant of tensor memory) drain 128 accumulator columns each into registers, release
// the accumulator at once so the next tile's MMAs overlap the arithmetic, then compute
// hidden = bf16(silu(bf16 gate) * bf16 up), requantise 32-element blocks to MXFP8 and store 64
// E4M3 bytes and two scale bytes per row. The reference runs this arithmetic as its act owner
// (campaigns/mok/port/act/act.cu:100-178) on bf16 gate / up written by the GEMM owner; here the
// accumulator channel hands it the tile in tensor memory.
#include "moe.cuh"

extern "C" __device__ void moe_epilogue_swiglu_mxfp8_role(const void* params, unsigned variant);
PL_STAGE("moe.epilogue.swiglu-mxfp8", "1.0.0");
PL_PARAMS(MoeSwigluParams, g, out, out_sc, out_cols, limit);
PL_ROLE(epilogue, moe_epilogue_swiglu_mxfp8_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();

#ifndef PIPELINK_EMIT
#include "../../csrc/swiglu.cuh"
extern "C" __device__ void moe_epilogue_swiglu_mxfp8_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeSwigluParams p = *static_cast<const MoeSwigluParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const int lane = threadIdx.x & 31;
  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int ew = warp - pipelink_moe_warp_epilogue();
  const int quad = warp & 3;            // the TMEM lane quadrant a warp may read is its index mod 4
  const int ch = ew >> 2;               // which half of the gate (and up) columns
  const Walk w = make_walk(p.g, lane, false);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot());
  const uint32_t taddr = tmem + pipelink_moe_acc() + (static_cast<uint32_t>(quad * 32) << 16);
  const uint32_t acc_empty_leader = plb::mapa_shared(bar(smem, pipelink_moe_acc_empty()), 0);
  uint32_t acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < w.total_tiles && ok; tile += num_pairs) {
    const Tile t = decode(p.g, w, tile, static_cast<int>(cta_rank));
    const int64_t row = t.out_row0 + cta_rank * 128 + quad * 32 + lane;
    if (!plb::mbar_wait(bar(smem, pipelink_moe_acc_full()), acc_phase, p.g.status, plb::ST_TIMEOUT_TMEM_FULL, 0)) ok = false;
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (!ok) break;
    plb::tc_fence_after();
    uint32_t g0[32], g1[32], u0[32], u1[32];
    plb::tc_ld_32x32b_x32(taddr + ch * 64, g0);
    plb::tc_ld_32x32b_x32(taddr + ch * 64 + 32, g1);
    plb::tc_ld_32x32b_x32(taddr + 128 + ch * 64, u0);
    plb::tc_ld_32x32b_x32(taddr + 128 + ch * 64 + 32, u1);
    plb::tc_wait_ld();
    plb::tc_fence_before();
    __syncwarp();
    if (lane == 0) plb::mbar_arrive_cluster(acc_empty_leader);
    uint4 q0, q1, q2, q3;
    const uint32_t e0 = plb::swiglu_quant32(g0, u0, p.limit, q0, q1);
    const uint32_t e1 = plb::swiglu_quant32(g1, u1, p.limit, q2, q3);
    uint4* dst = reinterpret_cast<uint4*>(p.out + row * p.out_cols + t.n_tile * 128 + ch * 64);
    dst[0] = q0;
    dst[1] = q1;
    dst[2] = q2;
    dst[3] = q3;
    const size_t off = plb::scale_offset(row, t.n_tile * 4 + ch * 2, p.out_cols >> 7);
    *reinterpret_cast<uint16_t*>(p.out_sc + off) = static_cast<uint16_t>(e0 | (e1 << 8));
    acc_phase ^= 1u;
  }
}
#endif  // !PIPELINK_EMIT
