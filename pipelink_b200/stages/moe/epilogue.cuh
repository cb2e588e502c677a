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
  if (e.lane == 0) plb::mbar_arrive_cluster_relaxed(e.acc_empty_leader);
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
  if (lane == 0) plb::mbar_arrive_cluster_relaxed(e.acc_empty_leader);
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

// The tile loop of the one-launch forward's epilogue: pass-1 tiles through the SwiGLU body (then the
// row tile's hidden_ready count), pass-2 tiles through the row-store body. False when a wait ran out.
__device__ __forceinline__ bool fwd_epilogue_tiles(const MoeFwdEpilogueParams& p, const EpilogueWarp& e, uint32_t smem) {
  const FwdWalk f = make_fwd_walk(p.g1, p.g2, e.lane, false);
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  uint32_t acc_phase = 0;
  bool ok = true;
  for (int tile = pair_id; tile < f.total && ok; tile += num_pairs) {
    const bool second = tile >= f.tiles1;
    const Tile t = decode(second ? p.g2 : p.g1, second ? f.w2 : f.w1, second ? tile - f.tiles1 : tile, static_cast<int>(e.cta_rank));
    if (!plb::mbar_wait(bar(smem, pipelink_moe_acc_full()), acc_phase, p.g1.status, plb::ST_TIMEOUT_TMEM_FULL, 0)) ok = false;
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (!ok) break;
    plb::tc_fence_after();
    if (!second) {
      swiglu_tile(e, t, p.hidden, p.hidden_sc, p.hidden_cols, p.limit);
      // the warp's stores first, then its count: the load owner acquires the count before it reads the rows
      __threadfence();
      __syncwarp();
      if (e.lane == 0) plb::red_release_gpu_add(p.counters + pipelink_moe_hidden_ready() + (t.a_blk >> 1), 1u);
    } else {
      rows_tile(e, t, p.out, p.out_peers, p.dest_row, p.peer_rank, p.out_cols);
    }
    acc_phase ^= 1u;
  }
  return ok;
}

__device__ __forceinline__ void tail_sync() {   // the eight epilogue warps of this CTA
  asm volatile("bar.sync %0, %1;" ::"r"(pipelink_moe_tail_barrier()), "r"(EpilogueWarps * 32) : "memory");
}

// The forward's tail (see MoeFwdTailParams). Every CTA counts itself done; the CTA that completes the
// count tells the group (one release per rank, as plb_ep_barrier does) and advances this rank's barrier
// generation; every CTA then waits, bounded, for all ranks' flags (one rank: for the count) and takes
// its share of the weighted sums. Arithmetic and order of weighted_combine_kernel: the same bits.
__device__ __forceinline__ void fwd_tail(const MoeFwdTailParams& t, unsigned* counters, plb::Status* status, bool ok) {
  const int tid = static_cast<int>(threadIdx.x) - 32 * pipelink_moe_warp_epilogue();      // 0 .. 255
  __shared__ int tail_failed;
  unsigned target = 0;
  if (t.flags_peers != nullptr) target = plb::ld_volatile_u32(t.barrier_state) + 1u;      // read before anyone can advance it
  if (tid == 0) tail_failed = 0;
  tail_sync();
  if (!ok) tail_failed = 1;        // a warp whose wait ran out: the CTA still counts itself done, then leaves
  __threadfence_system();          // this thread's row stores (local and to peers) before its CTA is counted done
  tail_sync();
  unsigned* done = counters + pipelink_moe_ctas_done();
  if (tid == 0) {
    __threadfence();
    const unsigned before = atomicAdd(done, 1u);
    __threadfence();
    if (before + 1u == gridDim.x && t.flags_peers != nullptr) {
      // every CTA of this GPU has pushed its rows: one release per rank, then this rank's generation
      plb::fence_acq_rel_sys();
      for (int r = 0; r < t.world; ++r) plb::red_release_sys_add(t.flags_peers[r] + t.rank, 1u);
      *reinterpret_cast<volatile unsigned*>(t.barrier_state) = target;
      __threadfence();
    }
  }
  // wait: thread i < world for rank i's flag here; one rank: thread 0 for the count
  const int waiters = t.flags_peers != nullptr ? t.world : 1;
  if (tid < waiters) {
    const unsigned* flag = t.flags_peers != nullptr ? t.flags_peers[t.rank] + tid : done;
    const unsigned want = t.flags_peers != nullptr ? target : gridDim.x;
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      const unsigned v = t.flags_peers != nullptr ? plb::ld_acquire_sys_u32(flag) : plb::ld_acquire_gpu_u32(flag);
      if (static_cast<int>(v - want) >= 0) break;
      if ((it & 63u) == 63u) {
        if (clock64() - t0 > plb::kWaitBudgetCycles || plb::ld_volatile_i32(&status->code) != 0) {
          plb::report_failure(status, plb::ST_TIMEOUT_COUNTER, 330 + tid, v, want);
          tail_failed = 1;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  tail_sync();
  if (*reinterpret_cast<volatile int*>(&tail_failed) != 0) return;
  const uint4* combine = reinterpret_cast<const uint4*>(t.combine);
  uint4* out = reinterpret_cast<uint4*>(t.output);
  const long long vec_per_row = t.hidden >> 3, total = t.tokens * vec_per_row;
  // two output vectors per thread and pass: sixteen row loads in flight (a CTA runs 256 threads here, not
  // the thousands a launch of its own would, so each thread keeps more of HBM's latency covered)
  const long long stride = static_cast<long long>(gridDim.x) * (EpilogueWarps * 32);
  const long long first = static_cast<long long>(blockIdx.x) * (EpilogueWarps * 32) + tid;
  for (long long v0 = first; v0 < total; v0 += 2 * stride) {
    const long long vs[2] = {v0, v0 + stride};
    float acc[2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int s0 = 0; s0 < t.topk; s0 += 8) {
      uint4 c[2][8];
      float ws[2][8];
      const int n = t.topk - s0 < 8 ? t.topk - s0 : 8;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (vs[u] >= total) continue;
        const long long tok = vs[u] / vec_per_row, j = vs[u] - tok * vec_per_row;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s < n) {
            const long long slot = tok * t.topk + s0 + s;
            ws[u][s] = t.router_w[slot];
            c[u][s] = combine[(t.index != nullptr ? static_cast<long long>(t.index[slot]) : slot) * vec_per_row + j];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (vs[u] >= total) continue;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s < n) {
            const uint4 cc = c[u][s];
            const float f[8] = {plb::bf16_lo(cc.x), plb::bf16_hi(cc.x), plb::bf16_lo(cc.y), plb::bf16_hi(cc.y),
                                plb::bf16_lo(cc.z), plb::bf16_hi(cc.z), plb::bf16_lo(cc.w), plb::bf16_hi(cc.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[u][i] = __fadd_rn(acc[u][i], __fmul_rn(ws[u][s], f[i]));
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (vs[u] >= total) continue;
      uint4 o;
      o.x = plb::pack_bf16(__float_as_uint(acc[u][0]), __float_as_uint(acc[u][1]));
      o.y = plb::pack_bf16(__float_as_uint(acc[u][2]), __float_as_uint(acc[u][3]));
      o.z = plb::pack_bf16(__float_as_uint(acc[u][4]), __float_as_uint(acc[u][5]));
      o.w = plb::pack_bf16(__float_as_uint(acc[u][6]), __float_as_uint(acc[u][7]));
      out[vs[u]] = o;
    }
  }
}
}  // namespace moe
