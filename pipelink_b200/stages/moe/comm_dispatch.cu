// Stage moe.comm.dispatch: expert-parallel token dispatch inside the GEMM image. Two warps per CTA
// take tickets of two schedule rows, copy each row's E4M3 bytes from the token's home rank
// (peer -> shared memory with 16-byte asynchronous copies, shared memory -> the A operand with
// plain stores) and its scale words (through registers), and count the ticket into the row tile's
// `rows_ready` counter with a release; the load owner acquires a complete tile before its first
// TMA read of it. The reference's dispatch_kernel plays this part in its forward megakernel
// (campaigns/mok/port/comm/comm.cu:105-123). Any resident CTA can serve any ticket and the warps
// wait for nothing, so the tiles the load owners wait for always complete.
#include "moe.cuh"

extern "C" __device__ void moe_comm_dispatch_role(const void* params, unsigned variant);
PL_STAGE("moe.comm.dispatch", "1.0.0");
PL_PARAMS(MoeCommParams, g, xq_peers, sc_rows_peers, peer_rank, peer_token_idx, dst, dst_sc, counters, row_bytes);
PL_ROLE(comm, moe_comm_dispatch_role, 2);
MOE_TOPOLOGY();
PL_ENDPOINT(rows_ready, moe::rows_ready(pl::produce, "comm"));
PL_CLAIM_WARPS(pipelink_moe_warp_comm, comm, 2, 1);
MOE_REGS_HELPER(comm);
PL_CLAIM(smem, pipelink_moe_dispatch_ring, pl::units(2 * 8192), 16);
MOE_CLAIM_ROWS_READY();
PL_CLAIM(gmem_counter, pipelink_moe_ticket, pl::units(1), 1);

#ifndef PIPELINK_EMIT
extern "C" __device__ void moe_comm_dispatch_role(const void* raw_params, unsigned) {
  using namespace moe;
  const MoeCommParams p = *static_cast<const MoeCommParams*>(raw_params);   // a copy in registers
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const int lane = threadIdx.x & 31;
  const int warp = static_cast<int>(threadIdx.x >> 5) - pipelink_moe_warp_comm();
  const Walk w = make_walk(p.g, lane, false);
  constexpr int kTicketRows = 2;
  const uint32_t ring = plb::smem_u32(pl_smem) + pipelink_moe_dispatch_ring() + static_cast<uint32_t>(warp) * (kTicketRows * 4096);
  const int vecs = p.row_bytes >> 4;          // <= 256
  const int col_blocks = p.row_bytes >> 7;
  const int rows_live = w.m_tiles_live * 256;
  for (;;) {
    int base = 0;
    if (lane == 0) base = static_cast<int>(atomicAdd(p.counters + pipelink_moe_ticket(), static_cast<unsigned>(kTicketRows)));
    base = __shfl_sync(0xFFFFFFFFu, base, 0);
    if (base >= rows_live) break;
    int my_src = -1, my_tok = 0;
    if (lane < kTicketRows) {
      my_src = p.peer_rank[base + lane];
      my_tok = my_src >= 0 ? p.peer_token_idx[base + lane] : 0;
    }
    uint32_t word[kTicketRows];
#pragma unroll
    for (int i = 0; i < kTicketRows; ++i) {
      const int src = __shfl_sync(0xFFFFFFFFu, my_src, i);
      const int64_t t = __shfl_sync(0xFFFFFFFFu, my_tok, i);
      word[i] = 0u;
      if (src >= 0) {
        const uint8_t* from = p.xq_peers[src] + t * p.row_bytes;
        for (int v = lane; v < vecs; v += 32)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + i * 4096 + v * 16), "l"(from + v * 16)
                       : "memory");
        if (lane < col_blocks) word[i] = p.sc_rows_peers[src][t * col_blocks + lane];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < kTicketRows; ++i) {
      const int src = __shfl_sync(0xFFFFFFFFu, my_src, i);
      const int r = base + i;
      uint4* dst = reinterpret_cast<uint4*>(p.dst + static_cast<size_t>(r) * p.row_bytes);
      for (int v = lane; v < vecs; v += 32) {       // every lane reads back the pieces it copied in
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (src >= 0)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                       : "r"(ring + i * 4096 + v * 16)
                       : "memory");
        dst[v] = val;
      }
      if (lane < col_blocks) {
        const size_t off = static_cast<size_t>(r >> 7) * col_blocks * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4;
        *reinterpret_cast<uint32_t*>(p.dst_sc + off + static_cast<size_t>(lane) * 512) = word[i];
      }
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) plb::red_release_gpu_add(p.counters + pipelink_moe_rows_ready() + (base >> 8), static_cast<unsigned>(kTicketRows));
  }
}
#endif  // !PIPELINK_EMIT
