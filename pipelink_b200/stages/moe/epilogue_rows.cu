// Stage moe.epilogue.rows-bf16: the down projection's consumer. Eight warps per CTA drain the
// accumulator into registers, release it, round to bf16 and store whole rows: to
// out[dest_row[p]] on this GPU, or, with a table of per-rank bases, into the home rank's buffer over
// NVLink (the combine push: the reference's combine_kernel, campaigns/mok/port/comm/comm.cu:124-129,
// fed by its GEMM owner's FWD_ROUTED_DOWN case, campaigns/mok/port/gemm/gemm.cu:158-162). Rows pass
// through 2 KiB of shared memory per warp, eight at a time, so that every store instruction of a
// warp writes two 256-byte row segments.
#include "moe.cuh"

extern "C" __device__ void moe_epilogue_rows_bf16_role(const void* params, unsigned variant);
PL_STAGE("moe.epilogue.rows-bf16", "1.0.0");
PL_PARAMS(MoeRowsParams, g, out, out_peers, dest_row, peer_rank, out_cols);
PL_ROLE(epilogue, moe_epilogue_rows_bf16_role, 8);
MOE_TOPOLOGY();
PL_ENDPOINT(accumulator, moe::accumulator(pl::consume, "epilogue"));
PL_CLAIM_WARPS(pipelink_moe_warp_epilogue, epilogue, 8, 4);
MOE_REGS_EPILOGUE(epilogue);
MOE_CLAIM_ACCUMULATOR();
MOE_CLAIM_STAGING();

#ifndef PIPELINK_EMIT
#include "../../csrc/swiglu.cuh"
extern "C" __device__ void moe_epilogue_rows_bf16_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeRowsParams p = *static_cast<const MoeRowsParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t smem = plb::smem_u32(pl_smem);
  const int lane = threadIdx.x & 31;
  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int ew = warp - pipelink_moe_warp_epilogue();
  const int quad = warp & 3;
  const int ch = ew >> 2;               // which half of the 256 accumulator columns
  const Walk w = make_walk(p.g, lane, false);
  const uint32_t cta_rank = plb::cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot());
  const uint32_t taddr = tmem + pipelink_moe_acc() + (static_cast<uint32_t>(quad * 32) << 16);
  const uint32_t acc_empty_leader = plb::mapa_shared(bar(smem, pipelink_moe_acc_empty()), 0);
  const uint32_t stage_base = smem + pipelink_moe_staging() + ew * 2048;
  uint32_t acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < w.total_tiles && ok; tile += num_pairs) {
    const Tile t = decode(p.g, w, tile, static_cast<int>(cta_rank));
    const int64_t row = t.out_row0 + cta_rank * 128 + quad * 32 + lane;
    if (!plb::mbar_wait(bar(smem, pipelink_moe_acc_full()), acc_phase, p.g.status, plb::ST_TIMEOUT_TMEM_FULL, 0)) ok = false;
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (!ok) break;
    plb::tc_fence_after();
    uint32_t v0[32], v1[32], v2[32], v3[32];
    plb::tc_ld_32x32b_x32(taddr + ch * 128, v0);
    plb::tc_ld_32x32b_x32(taddr + ch * 128 + 32, v1);
    plb::tc_ld_32x32b_x32(taddr + ch * 128 + 64, v2);
    plb::tc_ld_32x32b_x32(taddr + ch * 128 + 96, v3);
    plb::tc_wait_ld();
    plb::tc_fence_before();
    __syncwarp();
    if (lane == 0) plb::mbar_arrive_cluster(acc_empty_leader);
    uint32_t wv[64];                      // 128 fp32 -> 64 packed bf16 pairs = 16 chunks of 16 bytes
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      wv[i] = plb::pack_bf16(v0[2 * i], v0[2 * i + 1]);
      wv[16 + i] = plb::pack_bf16(v1[2 * i], v1[2 * i + 1]);
      wv[32 + i] = plb::pack_bf16(v2[2 * i], v2[2 * i + 1]);
      wv[48 + i] = plb::pack_bf16(v3[2 * i], v3[2 * i + 1]);
    }
    const int dest = p.dest_row[row];
    const int pr = (p.out_peers != nullptr && dest >= 0) ? p.peer_rank[row] : 0;
    const size_t col_byte = (static_cast<size_t>(t.n_tile) * 256 + ch * 128) * 2;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      if ((lane >> 3) == h) {
        const uint32_t r8 = lane & 7;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t addr = stage_base + r8 * 256 + ((static_cast<uint32_t>(j) ^ r8) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(wv[4 * j]), "r"(wv[4 * j + 1]),
                       "r"(wv[4 * j + 2]), "r"(wv[4 * j + 3])
                       : "memory");
        }
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t rr = i * 2 + (lane >> 4);
        const uint32_t c = lane & 15;
        const int src_lane = h * 8 + static_cast<int>(rr);
        const int d = __shfl_sync(0xFFFFFFFFu, dest, src_lane);
        const int prr = __shfl_sync(0xFFFFFFFFu, pr, src_lane);
        uint4 val;
        const uint32_t addr = stage_base + rr * 256 + ((c ^ rr) << 4);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                     : "r"(addr)
                     : "memory");
        if (d >= 0) {
          uint8_t* base = p.out_peers != nullptr ? p.out_peers[prr] : p.out;
          *reinterpret_cast<uint4*>(base + static_cast<size_t>(d) * p.out_cols * 2 + col_byte + c * 16) = val;
        }
      }
      __syncwarp();
    }
    acc_phase ^= 1u;
  }
}
#endif  // !PIPELINK_EMIT
