// Shared vocabulary of the MoE grouped-GEMM stages: tile geometry, per-stage parameter blocks
// and the link-time handles the stages read.
//
// The linked image is the CTA-pair grouped MXFP8 GEMM of csrc/grouped_gemm2.cu cut along its
// warp roles into separately packed owners, the way the reference cuts its MoE megakernel into
// comm / gemm / act packages joined by channel contracts (campaigns/mok/port/pipelines/fwd.json,
// campaigns/mok/port/gemm/gemm.cu:447-468 for the GEMM owner's channel list):
//   moe.load       1 warp   TMA producer of the operands ring (both CTAs of a pair)
//   moe.mma        1 warp   tcgen05 cta_group::2 MMA issuer (leader CTA), scale blocks -> TMEM
//   moe.comm.*     2 warps  dispatch: pulls routed rows from the home ranks under the mainloop
//                           (moe.comm.dispatch), or does nothing (moe.comm.none)
//   moe.epilogue.* 8 warps  accumulator -> SwiGLU + MXFP8 requantise (gate/up projection), or
//                           accumulator -> bf16 rows placed / pushed to the home rank (down projection)
// joined by an `operands` ring in shared memory whose depth is bound at link time, an
// `accumulator` channel in tensor memory and a `rows_ready` counter channel in global memory
// (comm -> load). Every pipelink_* function is resolved by the generated binding stub; after the
// LTO link each call folds to a constant.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <pipelink/stage.hpp>

#ifndef PIPELINK_EMIT
#include "../../csrc/common.cuh"
#include "../../csrc/mxfp8.cuh"
#else
namespace plb { struct Status; }   // the manifest pass needs the parameter layouts only
#endif

namespace moe {
constexpr int TileBytes = 128 * 128;                       // one CTA's A or B tile of a K step
constexpr int SfBytes = 512;                               // one 128-row x 4-group scale block
constexpr int SlotBytes = 2 * TileBytes + 3 * SfBytes + 512;   // A | B | SFA SFB0 SFB1 | pad to 1 KiB
constexpr int SlotTx = 2 * TileBytes + 3 * SfBytes;        // bytes one CTA's loads credit per K step
constexpr int OffA = 0, OffB = TileBytes, OffSf = 2 * TileBytes;
constexpr int SfColsPerSlot = 16;                          // TMEM columns: 4 (A) + 8 (B) used
constexpr int AccCols = 256;
constexpr int EpilogueWarps = 8;
constexpr int MaxRowTiles = 4096;                          // counter slots claimed for rows_ready (1 M schedule rows)
static_assert(SlotBytes % 1024 == 0, "operand tiles need 1 KiB alignment for the 128-byte swizzle");
}  // namespace moe

// What every role needs to walk the same tile list.
struct MoeGeometry {
  const int* block_expert;   // expert of each 128-row block of the schedule
  const int* num_rows_dev;   // padded rows in use (device scalar)
  plb::Status* status;
  int max_m_tiles;           // capacity / 256
  int k_steps;               // K / 128
  int n_tiles;               // weight rows per expert / 256
  int m_rotation;            // the tile loop starts this many row tiles in
  int m_stride;              // and steps this many row tiles at a time (made coprime to the live count)
  int pad;
};

struct alignas(64) MoeLoadParams {
  CUtensorMap a, b, sfa, sfb;
  MoeGeometry g;
  const unsigned* counters;     // the image's counter workspace (null: A is already in place);
                                // slot pipelink_moe_rows_ready() + m_tile reaches 256 when the tile is complete
};
struct alignas(16) MoeMmaParams {
  MoeGeometry g;
};
struct alignas(16) MoeCommParams {
  MoeGeometry g;
  const uint8_t* const* xq_peers;        // per rank: u8 [tokens, K]
  const uint32_t* const* sc_rows_peers;  // per rank: u32 [tokens, K / 128]
  const int* peer_rank;
  const int* peer_token_idx;
  uint8_t* dst;                          // the A operand
  uint8_t* dst_sc;
  unsigned* counters;                    // the image's counter workspace, zeroed before the launch:
                                         // pipelink_moe_rows_ready() + m_tile and pipelink_moe_ticket()
  int row_bytes;                         // K
  int pad;
};
struct alignas(16) MoeSwigluParams {
  MoeGeometry g;
  uint8_t* out;        // E4M3 [rows, out_cols]
  uint8_t* out_sc;
  int out_cols;        // I
  float limit;         // +inf: plain SwiGLU
};
struct alignas(16) MoeRowsParams {
  MoeGeometry g;
  uint8_t* out;                  // bf16 rows, local placement
  uint8_t* const* out_peers;     // or per-rank bases (push), null for local
  const int* dest_row;
  const int* peer_rank;
  int out_cols;                  // H
  int pad;
};

// ---- the one-launch forward: gate/up projection tiles, then down projection tiles, one tile list ----
struct alignas(64) MoeFwdLoadParams {
  CUtensorMap a1, b1, sfa1, sfb1;   // pass 1: routed rows x interleaved gate/up weights
  CUtensorMap a2, b2, sfa2, sfb2;   // pass 2: hidden rows (written by this launch) x down weights
  MoeGeometry g1, g2;               // same schedule, K steps and column tiles of each pass
  const unsigned* counters;         // slot pipelink_moe_hidden_ready() + m_tile counts epilogue warps done with the
                                    // row tile's pass-1 tiles; pipelink_moe_rows_ready() + m_tile as in MoeLoadParams
  int wait_rows_ready;              // 1 when a comm owner pulls the rows under the mainloop
  int pad;
};
struct alignas(16) MoeFwdMmaParams {
  MoeGeometry g1, g2;
};
struct alignas(16) MoeFwdEpilogueParams {
  MoeGeometry g1, g2;
  uint8_t* hidden;               // pass 1 out: E4M3 [rows, hidden_cols]
  uint8_t* hidden_sc;
  uint8_t* out;                  // pass 2 out: bf16 rows, local placement
  uint8_t* const* out_peers;     // or per-rank bases (push), null for local
  const int* dest_row;
  const int* peer_rank;
  unsigned* counters;
  int hidden_cols;               // I
  int out_cols;                  // H
  float limit;                   // +inf: plain SwiGLU
  int pad;
};

// The forward's tail inside the same launch: once every CTA of this GPU has finished its down-projection
// tiles (and, in a group, every rank has said so through the group's flags), the epilogue warps sum
// each token's top-k rows with its router weights.
struct alignas(16) MoeFwdTailParams {
  const uint8_t* combine;          // bf16 rows: the [tokens * topk, H] slots, or the receive streams
  const int* index;                // row of (token, slot) in `combine`, or null for token * topk + slot
  const float* router_w;           // [tokens, topk]
  uint8_t* output;                 // bf16 [tokens, H]
  unsigned* const* flags_peers;    // the group barrier's flags (per rank: u32 [world]), or null for one rank
  unsigned* barrier_state;         // [0]: this rank's barrier generation, advanced here
  long long tokens;
  int topk, hidden, rank, world;
};
struct alignas(16) MoeFwdCombineParams {
  MoeFwdEpilogueParams e;
  MoeFwdTailParams t;
};

extern "C" __device__ int pipelink_moe_depth();
extern "C" __device__ int pipelink_moe_operands();     // smem byte offset of the ring
extern "C" __device__ int pipelink_moe_full();         // first mbarrier slot (16 bytes each)
extern "C" __device__ int pipelink_moe_empty();
extern "C" __device__ int pipelink_moe_acc_full();
extern "C" __device__ int pipelink_moe_acc_empty();
extern "C" __device__ int pipelink_moe_drain();        // mbarrier slot the MMA owner drains through on failure
extern "C" __device__ int pipelink_moe_acc();          // first TMEM column of the accumulator
extern "C" __device__ int pipelink_moe_sfcols();       // first TMEM column of the scale slots
extern "C" __device__ int pipelink_moe_staging();      // smem byte offset: 2 KiB per epilogue warp (row stores)
extern "C" __device__ int pipelink_moe_warp_epilogue();// first warp of the epilogue role
extern "C" __device__ int pipelink_moe_warp_comm();    // first warp of the comm role
extern "C" __device__ int pipelink_moe_rows_ready();   // first counter slot of the per-row-tile counts (gmem_counter domain)
extern "C" __device__ int pipelink_moe_ticket();       // counter slot of the dispatch ticket
extern "C" __device__ int pipelink_moe_hidden_ready(); // first counter slot of the per-row-tile pass-1 completion counts
extern "C" __device__ int pipelink_moe_dispatch_ring();// smem byte offset: 8 KiB per dispatch warp
extern "C" __device__ int pipelink_moe_ctas_done();    // counter slot: CTAs of this launch that finished their tiles
extern "C" __device__ int pipelink_moe_tail_barrier(); // named barrier of the eight epilogue warps
extern "C" __device__ int pipelink_tmem_slot();        // smem byte offset where dispatch put the TMEM base

#ifndef PIPELINK_EMIT
namespace moe {
__device__ __forceinline__ uint32_t bar(uint32_t smem_base, int base, int slot = 0) {
  return smem_base + 16u * static_cast<uint32_t>(base + slot);
}

struct Walk {          // the tile list of this launch, identical for every role
  int total_tiles, m_tiles_live, m_rot, m_stride;
};
struct Tile {
  int a_blk, b_blk0, n_tile;
  int64_t out_row0;
};

// Row-tile order of a pass: start `m_rotation` tiles in, step with a stride made coprime to the live count.
__device__ __forceinline__ void order_rows(Walk& w, const MoeGeometry& g) {
  w.total_tiles = w.m_tiles_live * g.n_tiles;
  w.m_rot = w.m_tiles_live > 0 ? g.m_rotation % w.m_tiles_live : 0;
  w.m_stride = 1;
  if (g.m_stride > 1 && w.m_tiles_live > 1) {
    for (w.m_stride = g.m_stride % w.m_tiles_live == 0 ? 1 : g.m_stride % w.m_tiles_live;; ++w.m_stride) {
      int a = w.m_stride, b = w.m_tiles_live;
      while (b != 0) { const int t = a % b; a = b; b = t; }
      if (a == 1) break;
    }
  }
}

// A 256-row tile is multiplied by one expert's weights: a schedule padded to less than the tile is
// refused (every warp of every role evaluates this on its own and reaches the same answer).
__device__ __forceinline__ Walk make_walk(const MoeGeometry& g, int lane, bool report) {
  Walk w;
  const int rows = *g.num_rows_dev;
  w.m_tiles_live = rows >> 8;
  if (w.m_tiles_live > g.max_m_tiles) w.m_tiles_live = g.max_m_tiles;
  int bad = (rows & 255) != 0;
  for (int m = lane; m < w.m_tiles_live; m += 32) bad |= g.block_expert[2 * m] != g.block_expert[2 * m + 1];
  bad = __any_sync(0xFFFFFFFFu, bad);
  if (bad) {
    if (report && lane == 0) plb::report_failure(g.status, plb::ST_BAD_ARGUMENT, 320, static_cast<unsigned>(rows), 256u);
    w.m_tiles_live = 0;
  }
  order_rows(w, g);
  return w;
}

// the tile list of the one-launch forward: every pass-1 tile, then every pass-2 tile; each pass walks
// the row tiles in its own order (pass 1 in the order the dispatch warps deliver rows, pass 2 in the
// order that spreads the combine push over the home ranks)
struct FwdWalk {
  Walk w1, w2;
  int tiles1, total;
};
__device__ __forceinline__ FwdWalk make_fwd_walk(const MoeGeometry& g1, const MoeGeometry& g2, int lane, bool report) {
  FwdWalk f;
  f.w1 = make_walk(g1, lane, report);
  f.w2 = f.w1;
  order_rows(f.w2, g2);
  f.tiles1 = f.w1.total_tiles;
  f.total = f.tiles1 + f.w2.total_tiles;
  return f;
}

// ---- the two issue loops, shared by the GEMM owners and the one-launch forward owners.
// A whole warp walks each loop: ring position, descriptors, tensor-memory and barrier addresses are
// computed in convergent code, so they are warp-uniform, and one elected lane issues the copies, the
// tensor instructions and the commits. (Computed by one lane in a divergent branch the operands sit in
// per-thread registers and every such instruction pays for moving them: the issuing thread, not the
// tensor pipe, then bounds the kernel.)
struct Ring {
  uint32_t smem, operands, full0, empty0, stage, phase;
  int depth;
  __device__ __forceinline__ void init(uint32_t smem_base) {
    smem = smem_base;
    operands = smem_base + static_cast<uint32_t>(pipelink_moe_operands());
    full0 = bar(smem_base, pipelink_moe_full());
    empty0 = bar(smem_base, pipelink_moe_empty());
    depth = pipelink_moe_depth();
    stage = 0;
    phase = 0;
  }
  __device__ __forceinline__ void advance() {
    if (++stage == static_cast<uint32_t>(depth)) { stage = 0; phase ^= 1u; }
  }
};

// K steps of one tile, MMA side: scale blocks -> tensor memory, four K32 MMAs, the slot back to both CTAs.
__device__ __forceinline__ bool mma_k_loop(Ring& r, int k_steps, uint32_t tmem, uint32_t d_tmem, uint32_t empty_peer_delta,
                                           plb::Status* status) {
  constexpr uint32_t idesc = plb::idesc_mxf8(256, 256);
  const uint32_t sfcols0 = tmem + static_cast<uint32_t>(pipelink_moe_sfcols());
  for (int kb = 0; kb < k_steps; ++kb) {
    if (!__all_sync(0xFFFFFFFFu, plb::mbar_wait(r.full0 + 16u * r.stage, r.phase, status, plb::ST_TIMEOUT_FULL, static_cast<int>(r.stage))))
      return false;
    plb::tc_fence_after();
    const uint32_t slot = r.operands + r.stage * SlotBytes;
    const uint32_t sfa_t = sfcols0 + r.stage * SfColsPerSlot, sfb_t = sfa_t + 4;
    const uint64_t sfd_a = plb::smem_desc(slot + OffSf, plb::kDescScale), sfd_b0 = plb::smem_desc(slot + OffSf + SfBytes, plb::kDescScale),
                   sfd_b1 = plb::smem_desc(slot + OffSf + 2 * SfBytes, plb::kDescScale);
    const uint64_t adesc = plb::smem_desc(slot + OffA, plb::kDescSw128KMajor), bdesc = plb::smem_desc(slot + OffB, plb::kDescSw128KMajor);
    const uint32_t first = kb != 0 ? 1u : 0u;
    const uint32_t empty_own = r.empty0 + 16u * r.stage, empty_peer = empty_own + empty_peer_delta;
    if (plb::elect_one_sync()) {
      plb::tc_cp_32x128b_warpx4_pair(sfa_t, sfd_a);
      plb::tc_cp_32x128b_warpx4_pair(sfb_t, sfd_b0);
      plb::tc_cp_32x128b_warpx4_pair(sfb_t + 4, sfd_b1);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        plb::tc_mma_mxf8_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, plb::idesc_with_sf(idesc, k), sfa_t, sfb_t, k != 0 ? 1u : first);
      plb::tc_commit_pair(empty_own);
      plb::tc_commit_pair(empty_peer);
    }
    __syncwarp();
    r.advance();
  }
  return true;
}

// K steps of one tile, load side: this CTA's half of A and B and the scale blocks of every K step.
__device__ __forceinline__ bool load_k_loop(Ring& r, int k_steps, uint32_t full_leader_delta, const CUtensorMap* ma, const CUtensorMap* mb,
                                            const CUtensorMap* msa, const CUtensorMap* msb, int a_blk, int b_blk, int b_blk0,
                                            plb::Status* status) {
  for (int kb = 0; kb < k_steps; ++kb) {
    if (!__all_sync(0xFFFFFFFFu, plb::mbar_wait(r.empty0 + 16u * r.stage, r.phase ^ 1u, status, plb::ST_TIMEOUT_EMPTY, static_cast<int>(r.stage))))
      return false;
    const uint32_t full = r.full0 + 16u * r.stage + full_leader_delta;
    const uint32_t slot = r.operands + r.stage * SlotBytes;
    const int kx = kb * 128, row_a = a_blk * 128, row_b = b_blk * 128;
    const int sf_a = a_blk * k_steps + kb, sf_b0 = b_blk0 * k_steps + kb, sf_b1 = (b_blk0 + 1) * k_steps + kb;
    if (plb::elect_one_sync()) {
      plb::mbar_arrive_expect_tx_cluster(full, SlotTx);
      plb::tma_load_2d_pair(slot + OffA, ma, full, kx, row_a);
      plb::tma_load_2d_pair(slot + OffB, mb, full, kx, row_b);
      plb::tma_load_2d_pair(slot + OffSf, msa, full, 0, sf_a);
      plb::tma_load_2d_pair(slot + OffSf + SfBytes, msb, full, 0, sf_b0);
      plb::tma_load_2d_pair(slot + OffSf + 2 * SfBytes, msb, full, 0, sf_b1);
    }
    __syncwarp();
    r.advance();
  }
  return true;
}

// One lane waits (bounded) until a grid-scoped counter reaches `target` and orders TMA reads after it; the warp learns the outcome.
__device__ __forceinline__ bool wait_count_warp(const unsigned* flag, unsigned target, plb::Status* status, int where, int lane) {
  bool ok = true;
  if (lane == 0) {
    const long long t0 = clock64();
    while (plb::ld_acquire_gpu_u32(flag) < target) {
      if (clock64() - t0 > plb::kWaitBudgetCycles / 2 || plb::ld_volatile_i32(&status->code) != 0) {
        plb::report_failure(status, plb::ST_TIMEOUT_COUNTER, where, plb::ld_acquire_gpu_u32(flag), target);
        ok = false;
        break;
      }
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");
  }
  return __all_sync(0xFFFFFFFFu, ok);
}

__device__ __forceinline__ Tile decode(const MoeGeometry& g, const Walk& w, int tile, int cta_rank) {
  Tile t;
  int m_tile = tile / g.n_tiles;
  t.n_tile = tile - m_tile * g.n_tiles;
  m_tile = static_cast<int>((static_cast<long long>(m_tile) * w.m_stride + w.m_rot) % w.m_tiles_live);
  const int expert = g.block_expert[m_tile * 2];
  t.a_blk = m_tile * 2 + cta_rank;
  t.b_blk0 = (expert * g.n_tiles + t.n_tile) * 2;
  t.out_row0 = static_cast<int64_t>(m_tile) * 256;
  return t;
}
}  // namespace moe
#endif  // !PIPELINK_EMIT

// ---- the contracts the owners share, stated once (annotations: <pipelink/stage.hpp>) ----
#ifdef PIPELINK_EMIT
namespace moe {
// The ring both CTAs of a pair fill: A tile | B tile | three scale blocks per slot. The leader
// CTA's full barrier collects one arrival and one slot payload from each CTA of the pair.
inline pl::endpoint operands(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("smem").scope("cluster").proxy("async")
      .tile("e4m3+ue8m0", {2, 128, 128})
      .layout_smem(8, {2, 128, 128}, {TileBytes, 128, 1}, 3, 4, 3)
      .ring(pl::depth::handle("pipelink_moe_depth"), SlotBytes, SlotTx)
      .mbarrier(pl::arrivals("pipelink_moe_full", 2, "load", 2 * SlotTx), pl::arrivals("pipelink_moe_empty", 1, "mma"), "load")
      .bind("base", "pipelink_moe_operands").bind("full", "pipelink_moe_full").bind("empty", "pipelink_moe_empty");
}
// 128 lanes x 256 fp32 columns per CTA; the leader's commit completes both CTAs' full barriers,
// and every epilogue warp of the pair arrives on the leader's empty barrier.
inline pl::endpoint accumulator(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("tmem").scope("cluster").proxy("async")
      .tile("f32", {128, AccCols})
      .layout_tmem(32, 0, 128, AccCols)
      .ring(pl::depth::fixed(1), 128 * AccCols * 4)
      .mbarrier(pl::arrivals("pipelink_moe_acc_full", 1, "mma"),
                pl::arrivals("pipelink_moe_acc_empty", 2 * EpilogueWarps, "epilogue"), "mma")
      .bind("base", "pipelink_moe_acc").bind("full", "pipelink_moe_acc_full").bind("empty", "pipelink_moe_acc_empty");
}
// Per row tile, how many of its 256 rows the comm owner has put in place: a grid-scoped counter
// released with red.release.gpu and acquired by the load owner before its first TMA read of the tile
// (the reference's counter endpoints: docs/reference/annotations.md, "Counters").
inline pl::endpoint rows_ready(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("gmem").scope("grid").proxy("generic")
      .tile("e4m3+ue8m0", {256})
      .counter("pipelink_moe_rows_ready", "red.release.gpu", "ld.acquire.gpu")
      .bind("slot", "pipelink_moe_rows_ready");
}
// Per row tile, how many epilogue warps have stored their part of a pass-1 tile of it: the load owner
// of the one-launch forward reads the hidden rows of a row tile once all column tiles are counted.
inline pl::endpoint hidden_ready(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("gmem").scope("grid").proxy("generic")
      .tile("e4m3+ue8m0", {256})
      .counter("pipelink_moe_hidden_ready", "red.release.gpu", "ld.acquire.gpu")
      .bind("slot", "pipelink_moe_hidden_ready");
}
}  // namespace moe
#endif

#define MOE_TOPOLOGY() PL_TOPOLOGY(pl::topology().cta_group(2).cluster(2, 1, 1).persistent().scheduler("static"))
#define MOE_CLAIM_OPERANDS()                                                                   \
  PL_CLAIM(smem, pipelink_moe_operands, pl::per("pipelink_moe_depth", moe::SlotBytes), 1024);  \
  PL_CLAIM(mbarrier, pipelink_moe_full, pl::per("pipelink_moe_depth", 1), 1);                  \
  PL_CLAIM(mbarrier, pipelink_moe_empty, pl::per("pipelink_moe_depth", 1), 1)
#define MOE_CLAIM_ACCUMULATOR()                                        \
  PL_CLAIM(tmem, pipelink_moe_acc, pl::units(moe::AccCols), 32);       \
  PL_CLAIM(mbarrier, pipelink_moe_acc_full, pl::units(1), 1);          \
  PL_CLAIM(mbarrier, pipelink_moe_acc_empty, pl::units(1), 1)
#define MOE_CLAIM_STAGING() PL_CLAIM(smem, pipelink_moe_staging, pl::units(moe::EpilogueWarps * 2048), 16)
#define MOE_CLAIM_HIDDEN_READY() PL_CLAIM(gmem_counter, pipelink_moe_hidden_ready, pl::units(moe::MaxRowTiles), 1)
#define MOE_CLAIM_ROWS_READY() PL_CLAIM(gmem_counter, pipelink_moe_rows_ready, pl::units(moe::MaxRowTiles), 1)
// the two register groups of an image: load + MMA + comm warps give registers up, the epilogue takes them
#define MOE_REGS_HELPER(role) PL_CLAIM_REGS("pipelink_moe_regs_helpers", "helpers", {56}, #role)
#define MOE_REGS_EPILOGUE(role) PL_CLAIM_REGS("pipelink_moe_regs_epilogue", "epilogue", {224}, #role)

static_assert(sizeof(MoeGeometry) == 48 && sizeof(MoeLoadParams) == 576 && sizeof(MoeMmaParams) == 48 &&
              sizeof(MoeCommParams) == 112 && sizeof(MoeSwigluParams) == 80 && sizeof(MoeRowsParams) == 96 &&
              sizeof(MoeFwdLoadParams) == 1152 && sizeof(MoeFwdMmaParams) == 96 && sizeof(MoeFwdEpilogueParams) == 176 &&
              sizeof(MoeFwdTailParams) == 80 && sizeof(MoeFwdCombineParams) == 256,
              "parameter blocks: the manifests and the host image state these sizes");
