// The two accumulator consumers of the MoE images as per-tile bodies, shared by the single-pass
// epilogue owners (moe.epilogue.swiglu-mxfp8, moe.epilogue.rows-bf16) and by the owner of the
// one-launch forward (moe.fwd.epilogue), which runs one or the other per tile. A body starts once
// the tile's accumulator is full: it reads its 32 lanes x 128 columns, releases the accumulator,
// does its arithmetic and stores.
#pragma once
#include "../../csrc/swiglu.cuh"
#include "moe.cuh"

namespace moe {
struct EpilogueWarp {        // what an epilogue warp knows about itself
  uint32_t taddr;            // its TMEM lane quadrant of the accumulator
  uint32_t acc_empty_leader; // the leader CTA's accumulator-empty barrier
  uint32_t stage_base;       // its 2 KiB of the staging area (row stores)
  uint32_t cta_rank;
  int lane, quad, ch;        // ch: which half of the columns
};

__device__ __forceinline__ EpilogueWarp epilogue_warp(uint32_t smem, const unsigned char* smem_generic, bool staging) {
  EpilogueWarp e;
  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int ew = warp - pipelink_moe_warp_epilogue();
  e.lane = threadIdx.x & 31;
  e.quad = warp & 3;            // the TMEM lane quadrant a warp may read is its index mod 4
  e.ch = ew >> 2;
  e.cta_rank = plb::cluster_ctarank();
  const uint32_t tmem = *reinterpret_cast<const volatile uint32_t*>(smem_generic + pipelink_tmem_slot());
  e.taddr = tmem + pipelink_moe_acc() + (static_cast<uint32_t>(e.quad * 32) << 16);
  e.acc_empty_leader = plb::mapa_shared(bar(smem, pipelink_moe_acc_empty()), 0);
  e.stage_base = staging ? smem + pipelink_moe_staging() + ew * 2048 : 0u;
  return e;
}

// gate/up projection: SwiGLU of the interleaved gate and up columns, requantised to MXFP8
__device__ __forceinline__ void swiglu_tile(const EpilogueWarp& e, const Tile& t, uint8_t* out, uint8_t* out_sc, int out_cols,
                                            float limit) {
  const int64_t row = t.out_row0 + e.cta_rank * 128 + e.quad * 32 + e.lane;
  uint32_t g0[32], g1[32], u0[32], u1[32];
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 64, g0);
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 64 + 32, g1);
  plb::tc_ld_32x32b_x32(e.taddr + 128 + e.ch * 64, u0);
  plb::tc_ld_32x32b_x32(e.taddr + 128 + e.ch * 64 + 32, u1);
  plb::tc_wait_ld();
  plb::tc_fence_before();
  __syncwarp();
  if (e.lane == 0) plb::mbar_arrive_cluster(e.acc_empty_leader);
  uint4 q0, q1, q2, q3;
  const uint32_t e0 = plb::swiglu_quant32(g0, u0, limit, q0, q1);
  const uint32_t e1 = plb::swiglu_quant32(g1, u1, limit, q2, q3);
  uint4* dst = reinterpret_cast<uint4*>(out + row * out_cols + t.n_tile * 128 + e.ch * 64);
  dst[0] = q0;
  dst[1] = q1;
  dst[2] = q2;
  dst[3] = q3;
  const size_t off = plb::scale_offset(row, t.n_tile * 4 + e.ch * 2, out_cols >> 7);
  *reinterpret_cast<uint16_t*>(out_sc + off) = static_cast<uint16_t>(e0 | (e1 << 8));
}

// down projection: bf16 rows to out[dest_row[p]] on this GPU or, with a table of per-rank bases,
// into the home rank's buffer. Rows pass through the warp's 2 KiB of shared memory, eight at a
// time, so that every store instruction of a warp writes two 256-byte row segments.
__device__ __forceinline__ void rows_tile(const EpilogueWarp& e, const Tile& t, uint8_t* out, uint8_t* const* out_peers,
                                          const int* dest_row, const int* peer_rank, int out_cols) {
  const int lane = e.lane;
  const uint32_t stage_base = e.stage_base;
  const int64_t row = t.out_row0 + e.cta_rank * 128 + e.quad * 32 + lane;
  uint32_t v0[32], v1[32], v2[32], v3[32];
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 128, v0);
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 128 + 32, v1);
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 128 + 64, v2);
  plb::tc_ld_32x32b_x32(e.taddr + e.ch * 128 + 96, v3);
  plb::tc_wait_ld();
  plb::tc_fence_before();
  __syncwarp();
  if (lane == 0) plb::mbar_arrive_cluster(e.acc_empty_leader);
  uint32_t wv[64];                      // 128 fp32 -> 64 packed bf16 pairs = 16 chunks of 16 bytes
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    wv[i] = plb::pack_bf16(v0[2 * i], v0[2 * i + 1]);
    wv[16 + i] = plb::pack_bf16(v1[2 * i], v1[2 * i + 1]);
    wv[32 + i] = plb::pack_bf16(v2[2 * i], v2[2 * i + 1]);
    wv[48 + i] = plb::pack_bf16(v3[2 * i], v3[2 * i + 1]);
  }
  const int dest = dest_row[row];
  const int pr = (out_peers != nullptr && dest >= 0) ? peer_rank[row] : 0;
  const size_t col_byte = (static_cast<size_t>(t.n_tile) * 256 + e.ch * 128) * 2;
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
        uint8_t* base = out_peers != nullptr ? out_peers[prr] : out;
        *reinterpret_cast<uint4*>(base + static_cast<size_t>(d) * out_cols * 2 + col_byte + c * 16) = val;
      }
    }
    __syncwarp();
  }
}
}  // namespace moe
