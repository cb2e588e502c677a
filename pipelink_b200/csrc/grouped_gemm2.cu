// Grouped MXFP8 GEMM on CTA pairs: tcgen05.mma.cta_group::2, 256x256 output tiles.
//
// Same contract as grouped_gemm.cu (the reference's FWD_ROUTED_GATE/UP fused with its
// SwiGLU stage, and FWD_ROUTED_DOWN with the combine placement:
// campaigns/mok/port/gemm/gemm.cu:150-162, campaigns/mok/port/act/act.cu:100-178,
// campaigns/mok/port/comm/comm.cu:124-129) and the reference's own tile geometry
// (cluster of 2, M256 x N256, gemm.cu:26-36), chosen here because a 128x128 single-CTA
// tile moves ~260 B/clk/SM through shared memory and stalls the tensor pipe below 40 %;
// the paired tile stages half as many bytes per MMA cycle.
//
// Cluster (2,1,1), 384 threads per CTA:
//   warp 0      TMA producer (both CTAs): own 128 rows of A, own 128 weight rows of B
//               (the pair's MMA reads N = 256 across the two CTAs), own 512-byte A-scale
//               block and both 512-byte B-scale blocks; completion bytes of both CTAs are
//               credited to the leader CTA's full barrier
//   warp 1      MMA issuer (leader CTA only): scale blocks -> tensor memory, four K=32
//               MMAs per 128-byte K step, commits to both CTAs' empty barriers and, per
//               tile, to both CTAs' accumulator-full barriers
//   warp 2      tensor-memory alloc / free (both CTAs)
//   warps 4-11  epilogue (both CTAs): two warps per 32-lane quadrant, each drains 128
//               accumulator columns into registers, releases the accumulator at once so
//               the next tile's MMAs overlap the epilogue math, then stores
// One 256-column fp32 accumulator per CTA (columns 0-255), scale columns behind it.
//
// Mode 0: weight rows per 256-row tile are [128 gate | 128 up] of the same hidden
// indices; out = MXFP8(bf16(silu(bf16 gate) * bf16 up)).
// Mode 1: bf16 rows to out_base[dest_row], staged through shared memory (eight rows at a time) so
// every store instruction writes two 256-byte row segments (NVLink-friendly for the push).
#include "kernels.h"
#include "mxfp8.cuh"
#include "swiglu.cuh"
#include <cstring>

namespace plb {

namespace {

constexpr int kStages = 5;
constexpr int kTileBytes = 128 * 128;                  // one CTA's A or B tile per K step
constexpr int kSfBytes = 512;
constexpr int kSfStageBytes = 3 * kSfBytes;            // A scales, B scales rows 0-127, 128-255
constexpr uint32_t kStageTx = 2 * kTileBytes + kSfStageBytes;  // per CTA per stage
constexpr int kOffA = 0;
constexpr int kOffB = kStages * kTileBytes;
constexpr int kOffSf = 2 * kStages * kTileBytes;
constexpr int kOffStaging = kOffSf + kStages * kSfStageBytes;  // 8 warps x 2 KB
constexpr int kStagingBytes = 8 * 2048;
constexpr int kOffBars = kOffStaging + kStagingBytes;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes2 = kOffBars + kBarrierBytes + 1024;
static_assert(kOffSf % 1024 == 0 && kOffStaging % 16 == 0, "shared memory layout");
static_assert(kStagingBytes / 2 >= 2 * 4096, "dispatch ring: two rows of up to 4096 bytes per dispatch warp");
static_assert(kSmemBytes2 <= 232448, "shared memory of one CTA");
constexpr int kThreads2 = 384;
// Register hand-over between the roles. ptxas gives every thread 168 registers (launch bounds of 384
// threads, one CTA per SM), the CTA's pool is what it was launched with, and setmaxnreg.inc blocks
// until the pool can serve it: warps 0-3 must therefore drop to 56 before the eight epilogue warps
// can rise to 224. Any larger value for warps 0-3 makes the kernel wait forever.
constexpr int kRegsAtLaunch = 168, kRegsHelpers = 56, kRegsEpilogue = 224;
static_assert(kThreads2 * kRegsAtLaunch - 128 * kRegsHelpers >= 256 * kRegsEpilogue, "register pool of the CTA");
constexpr int kEpilogueWarps = 8;
constexpr int kTmemCols = 512;
constexpr int kSfColBase = 256;
constexpr int kSfColsPerStage = 16;  // 4 (A) + 8 (B) used
constexpr uint32_t kIdescPair = idesc_mxf8(256, 256);
constexpr uint32_t kIdescPairBf16 = idesc_bf16(256, 256, 0, 0);

struct Barriers2 {
  uint64_t full[kStages];   // used in the leader CTA: 2 arrivals + both CTAs' bytes
  uint64_t empty[kStages];  // per CTA: 1 arrival (leader's commit)
  uint64_t acc_full;        // per CTA: 1 arrival (leader's commit)
  uint64_t acc_empty;       // used in the leader CTA: one arrival per epilogue warp of the pair
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t pad;
};
static_assert(sizeof(Barriers2) <= kBarrierBytes, "barrier block too large");

#ifdef PLB_GEMM_PROFILE
#define PROF_DECL(x) long long x = 0
#define PROF_T0(x) const long long x = clock64()
#define PROF_ADD(acc, t0) acc += clock64() - (t0)
#define PROF_WRITE(slot, v) \
  if (p.prof != nullptr) p.prof[static_cast<size_t>(blockIdx.x) * 16 + (slot)] = (v)
#else
#define PROF_DECL(x)
#define PROF_T0(x)
#define PROF_ADD(acc, t0)
#define PROF_WRITE(slot, v)
#endif

struct Params2 {
  long long* prof;          // per-CTA cycle counters; only written by profiling builds
  const int* block_expert;  // per 128-row block
  const int* num_rows_dev;
  int m_rotation;           // modes 0/1: the tile loop starts this many 256-row tiles in (wraps around)
  int m_stride;             // modes 0/1: consecutive steps of the loop are this many row tiles apart (>= 1)
  const unsigned* ready;    // mode 1: per 256-row tile of A, a counter that reaches ready_target once the
  unsigned ready_target;    //         tile's rows have all arrived (all-gather -> GEMM); null = rows are local
  // mode 0, optional in-kernel dispatch (null pull_xq = A is already in place): warps 2 and 3 of every
  // CTA take tickets of two rows, copy each row's E4M3 bytes (peer -> shared -> A) and scale words
  // (through registers), and count the ticket into its 256-row tile; the load lane acquires a tile's count
  // before the tile's first TMA read (campaigns/mok/port/comm/comm.cu:105-123 gives the
  // reference's megakernel the same dispatch role)
  const uint8_t* const* pull_xq;        // per rank: u8 [tokens, K]
  const uint32_t* const* pull_sc_rows;  // per rank: u32 [tokens, K / 128], one run of scale words per token
  const int* pull_peer_rank;
  const int* pull_token_idx;
  uint8_t* pull_dst;                    // the A operand
  uint8_t* pull_dst_sc;                 // its scale tensor
  unsigned* pull_ready;                 // [max_m_tiles] zeroed by the launcher; 256 = tile complete
  unsigned* pull_ticket;                // zeroed by the launcher
  int pull_row_bytes;                   // K
  float limit;              // mode 0: gate <= limit, |up| <= limit before the activation; +inf = unclamped
  int max_m_tiles;          // capacity / 256
  int k_steps;
  int n_tiles;              // weight rows per expert / 256
  int out_cols;             // mode 0: I, mode 1: H
  uint8_t* out;
  uint8_t* out_sc;
  const int* dest_row;
  uint8_t* const* out_peers;
  const int* peer_rank;
  Status* status;
  // mode 0, training: also keep what the backward pass reads (any of these may be null)
  uint8_t* save_gate;      // E4M3 [rows, I]
  uint8_t* save_gate_sc;
  uint8_t* save_up;
  uint8_t* save_up_sc;
  __nv_bfloat16* save_hidden;  // bf16 [rows, I], the value that was quantised
  // mode 2 (weight gradients): per expert e, out[e] = A[:, seg_e] . B[:, seg_e]^T with the
  // contraction over that expert's rows of the schedule
  const int* expert_offsets;  // [experts + 1]
  int experts;
  int m_tiles;                // A rows / 256
  int k_blocks_total;         // contraction length of the whole tensors in K steps
  int k_shift;                // log2 of the schedule rows one K step contracts: 7 (128 E4M3) or 6 (64 bf16)
};

// What one tile means for the loads and the epilogue, identical for every role.
struct Tile {
  int a_blk;     // 128-row block of A loaded by this CTA
  int b_blk0;    // first of the tile's two 128-row blocks of B
  int k_blk0;    // first 128-byte K block
  int k_steps;
  int k_pitch;   // K blocks per row block in the scale tensors
  int n_tile;    // output column tile
  int64_t out_row0;  // first output row of the pair's tile (CTA adds rank*128 + quad*32 + lane)
};

template <int MODE>
__device__ __forceinline__ Tile decode_tile(const Params2& p, int tile, int cta_rank, int m_tiles_live, int m_rot,
                                            int m_stride = 1) {
  Tile t;
  if (MODE == 2) {
    const int per_expert = p.m_tiles * p.n_tiles;
    const int e = tile / per_expert, r = tile - e * per_expert;
    const int m_tile = r / p.n_tiles;
    t.n_tile = r - m_tile * p.n_tiles;
    t.a_blk = m_tile * 2 + cta_rank;
    t.b_blk0 = t.n_tile * 2;
    t.k_blk0 = p.expert_offsets[e] >> p.k_shift;
    t.k_steps = (p.expert_offsets[e + 1] - p.expert_offsets[e]) >> p.k_shift;
    t.k_pitch = p.k_blocks_total;
    t.out_row0 = (static_cast<int64_t>(e) * p.m_tiles + m_tile) * 256;
  } else {
    int m_tile = tile / p.n_tiles;
    t.n_tile = tile - m_tile * p.n_tiles;
    // A rank that pushes rows to their home ranks starts at a different source-rank segment
    // than its peers, so the group writes all-to-all instead of all-to-one.
    // ... and walks them with a stride coprime to their count, so the tiles in flight at any time
    // belong to different source ranks: a permutation of the same tiles, results unchanged.
    m_tile = static_cast<int>((static_cast<long long>(m_tile) * m_stride + m_rot) % m_tiles_live);
    const int expert = p.block_expert[m_tile * 2];
    t.a_blk = m_tile * 2 + cta_rank;
    t.b_blk0 = (expert * p.n_tiles + t.n_tile) * 2;
    t.k_blk0 = 0;
    t.k_steps = p.k_steps;
    t.k_pitch = p.k_steps;
    t.out_row0 = static_cast<int64_t>(m_tile) * 256;
  }
  return t;
}

// hidden value of one element pair exactly as swiglu_quant32 computes it (bf16-valued float)
__device__ __forceinline__ float swiglu_bf16(uint32_t g_bits, uint32_t u_bits, float limit) {
  const float gf = bf16r(__uint_as_float(g_bits));
  const float uf = bf16r(__uint_as_float(u_bits));
  return bf16r(swiglu_clamped(gf, uf, limit));
}

// 32 accumulator values -> bf16 round -> MXFP8 block (two uint4 of E4M3 + scale byte)
__device__ __forceinline__ uint32_t quant32_bf16(const uint32_t* a, uint4& q0, uint4& q1) {
  float h[32];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    h[i] = bf16r(__uint_as_float(a[i]));
    amax = fmaxf(amax, fabsf(h[i]));
  }
  const uint32_t e = e8m0_from_amax(amax);
  const float inv = e8m0_inverse(e);
  q0.x = cvt_e4m3x4(h[0] * inv, h[1] * inv, h[2] * inv, h[3] * inv);
  q0.y = cvt_e4m3x4(h[4] * inv, h[5] * inv, h[6] * inv, h[7] * inv);
  q0.z = cvt_e4m3x4(h[8] * inv, h[9] * inv, h[10] * inv, h[11] * inv);
  q0.w = cvt_e4m3x4(h[12] * inv, h[13] * inv, h[14] * inv, h[15] * inv);
  q1.x = cvt_e4m3x4(h[16] * inv, h[17] * inv, h[18] * inv, h[19] * inv);
  q1.y = cvt_e4m3x4(h[20] * inv, h[21] * inv, h[22] * inv, h[23] * inv);
  q1.z = cvt_e4m3x4(h[24] * inv, h[25] * inv, h[26] * inv, h[27] * inv);
  q1.w = cvt_e4m3x4(h[28] * inv, h[29] * inv, h[30] * inv, h[31] * inv);
  return e;
}

// BF16 = true is the reference's bf16 routed precision (pipelink_mok_precision,
// campaigns/mok/port/act/act.cu:246-249): bf16 operands, 64-element K steps of kind::f16 MMAs, no
// scale tensors, and in mode 0 the hidden rows leave as bf16 instead of MXFP8.
template <int MODE, bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
grouped_gemm2_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_sfa,
                     const __grid_constant__ CUtensorMap map_sfb, const Params2 p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  Barriers2* bars = reinterpret_cast<Barriers2*>(smem + kOffBars);

  // warp-uniform by construction, and said so to the compiler: the operands of the tensor and copy
  // instructions below are then computed once per warp, in convergent code
  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  int total_tiles, m_tiles_live = 0;
  int rows_in_use = 0, bad_schedule = 0;
  if (MODE == 2) {
    total_tiles = p.experts * p.m_tiles * p.n_tiles;
  } else {
    rows_in_use = *p.num_rows_dev;
    m_tiles_live = rows_in_use >> 8;
    if (m_tiles_live > p.max_m_tiles) m_tiles_live = p.max_m_tiles;
    total_tiles = m_tiles_live * p.n_tiles;
    // A 256-row tile is multiplied by ONE expert's weights: a schedule padded to less than the tile
    // (a trailing 128-row block, or a tile whose two blocks belong to different experts) is refused
    // below rather than computed with the wrong weights.
    bad_schedule = (rows_in_use & 255) != 0;
    for (int m = threadIdx.x; m < m_tiles_live; m += kThreads2)
      bad_schedule |= p.block_expert[2 * m] != p.block_expert[2 * m + 1];
  }
  const int m_rot = m_tiles_live > 0 ? p.m_rotation % m_tiles_live : 0;
  int m_stride = 1;
  if (MODE != 2 && p.m_stride > 1 && m_tiles_live > 1) {
    // smallest stride >= the requested one that is coprime to the live tile count
    for (m_stride = p.m_stride % m_tiles_live == 0 ? 1 : p.m_stride % m_tiles_live;; ++m_stride) {
      int a = m_stride, b = m_tiles_live;
      while (b != 0) { const int t = a % b; a = b; b = t; }
      if (a == 1) break;
    }
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 2);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_init(smem_u32(&bars->acc_empty), 2 * kEpilogueWarps);
    mbar_init(smem_u32(&bars->drain), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (!BF16) {
      prefetch_tensormap(&map_sfa);
      prefetch_tensormap(&map_sfb);
    }
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  bad_schedule = __syncthreads_or(bad_schedule);
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base), 0);
  if (bad_schedule) {   // both CTAs of every pair see the same schedule and agree
    if (threadIdx.x == 0) report_failure(p.status, ST_BAD_ARGUMENT, 320, static_cast<unsigned>(rows_in_use), 256u);
    total_tiles = 0;
    m_tiles_live = 0;
  }

  if (warp < 4) {
    setmaxnreg_dec<kRegsHelpers>();
    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer (both CTAs)
      // Like the MMA issuer below, the whole warp walks the loop with warp-uniform coordinates and barrier
      // addresses, and one elected lane issues the copies.
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t empty0 = smem_u32(&bars->empty[0]);
      const uint32_t full0_leader = mapa_shared(smem_u32(&bars->full[0]), 0);
      const int tiles_u = __shfl_sync(0xFFFFFFFFu, total_tiles, 0);
      PROF_DECL(t_empty);
      PROF_T0(t_begin);
      for (int tile = pair_id; tile < tiles_u && ok; tile += num_pairs) {
        const Tile t = decode_tile<MODE>(p, tile, static_cast<int>(cta_rank), m_tiles_live, m_rot, m_stride);
        const int a_blk = __shfl_sync(0xFFFFFFFFu, t.a_blk, 0), b_blk0 = __shfl_sync(0xFFFFFFFFu, t.b_blk0, 0);
        const int k_steps = __shfl_sync(0xFFFFFFFFu, t.k_steps, 0), k_blk0 = __shfl_sync(0xFFFFFFFFu, t.k_blk0, 0);
        const int k_pitch = __shfl_sync(0xFFFFFFFFu, t.k_pitch, 0);
        const int b_blk = b_blk0 + static_cast<int>(cta_rank);
        if (MODE == 0 && p.pull_xq != nullptr) {
          if (lane == 0) {
            const unsigned* flag = p.pull_ready + (a_blk >> 1);
            const long long t0 = clock64();
            while (ld_acquire_gpu_u32(flag) < 256u) {
              if (clock64() - t0 > kWaitBudgetCycles / 2 || ld_volatile_i32(&p.status->code) != 0) {
                report_failure(p.status, ST_TIMEOUT_COUNTER, 311, ld_acquire_gpu_u32(flag), 256u);
                ok = false;
                break;
              }
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
        }
        if (MODE == 1 && p.ready != nullptr) {
          // rows pushed by a peer are usable once its counter increment (a release at system scope,
          // examples/comm-overlap README "AllGather protocol") is observed; then order the TMA reads after it
          if (lane == 0) {
            const unsigned* flag = p.ready + (a_blk >> 1);
            const long long t0 = clock64();
            while (static_cast<int>(ld_acquire_sys_u32(flag) - p.ready_target) < 0) {
              // half the budget of the barrier waits downstream, so the record names the cause
              if (clock64() - t0 > kWaitBudgetCycles / 2 || ld_volatile_i32(&p.status->code) != 0) {
                report_failure(p.status, ST_TIMEOUT_COUNTER, 310, ld_acquire_sys_u32(flag), p.ready_target);
                ok = false;
                break;
              }
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
        }
        for (int kb = 0; kb < k_steps; ++kb) {
          PROF_T0(t0);
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(empty0 + 8u * stage, phase ^ 1u, p.status, ST_TIMEOUT_EMPTY, static_cast<int>(stage)));
          if (!ok) break;
          PROF_ADD(t_empty, t0);
          const uint32_t full = full0_leader + 8u * stage;
          const uint32_t sf = smem_base + kOffSf + stage * kSfStageBytes;
          const uint32_t dst_a = smem_base + kOffA + stage * kTileBytes, dst_b = smem_base + kOffB + stage * kTileBytes;
          const int kk = k_blk0 + kb;
          // the x coordinate counts elements: 128 E4M3 or 64 bf16 per 128-byte K step
          const int kx = kk * (BF16 ? 64 : 128);
          const int row_a = a_blk * 128, row_b = b_blk * 128;
          const int sf_a = a_blk * k_pitch + kk, sf_b0 = b_blk0 * k_pitch + kk, sf_b1 = (b_blk0 + 1) * k_pitch + kk;
          if (elect_one_sync()) {
            mbar_arrive_expect_tx_cluster(full, BF16 ? 2u * kTileBytes : kStageTx);
            tma_load_2d_pair(dst_a, &map_a, full, kx, row_a);
            tma_load_2d_pair(dst_b, &map_b, full, kx, row_b);
            if (!BF16) {
              tma_load_2d_pair(sf, &map_sfa, full, 0, sf_a);
              tma_load_2d_pair(sf + kSfBytes, &map_sfb, full, 0, sf_b0);
              tma_load_2d_pair(sf + 2 * kSfBytes, &map_sfb, full, 0, sf_b1);
            }
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      PROF_WRITE(0, t_empty);
      PROF_WRITE(1, clock64() - t_begin);
      if (!ok) {
        // give copies already in flight time to land before this CTA can exit
        const long long t0 = clock64();
        while (clock64() - t0 < 200000LL) {
        }
      }
    } else if (warp == 1 && leader) {
      // ---------------------------------------------------------- MMA issuer (leader CTA)
      // The whole warp walks the loop and every operand of the tensor instructions (descriptors, tensor-memory
      // addresses, barrier addresses) is computed in convergent code; one elected lane issues them. Computed by a
      // single lane in a divergent branch the same operands sit in per-thread registers and each instruction pays
      // for moving them (60 - 77 cycles per tcgen05 instruction measured, nine per K step: the issuing thread, not
      // the tensor pipe, then bounds the kernel).
      const uint32_t full0 = smem_u32(&bars->full[0]);
      const uint32_t empty0 = smem_u32(&bars->empty[0]);
      const uint32_t empty0_peer = mapa_shared(empty0, 1);
      const uint32_t acc_full_own = smem_u32(&bars->acc_full);
      const uint32_t acc_full_peer = mapa_shared(acc_full_own, 1);
      const uint32_t acc_empty = smem_u32(&bars->acc_empty);
      const int tiles_u = __shfl_sync(0xFFFFFFFFu, total_tiles, 0);
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      bool ok = true;
      PROF_DECL(t_acc);
      PROF_DECL(t_full);
      PROF_T0(t_begin);
      for (int tile = pair_id; tile < tiles_u && ok; tile += num_pairs) {
        const Tile t = decode_tile<MODE>(p, tile, 0, m_tiles_live, m_rot, m_stride);
        const int k_steps = __shfl_sync(0xFFFFFFFFu, t.k_steps, 0);
        if (k_steps == 0) continue;  // empty expert: the epilogue writes zeros on its own
        PROF_T0(ta);
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(acc_empty, acc_phase ^ 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, 0));
        if (!ok) break;
        PROF_ADD(t_acc, ta);
        tc_fence_after();
        for (int kb = 0; kb < k_steps; ++kb) {
          PROF_T0(tf);
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8u * stage, phase, p.status, ST_TIMEOUT_FULL, static_cast<int>(stage)));
          if (!ok) break;
          PROF_ADD(t_full, tf);
          tc_fence_after();
          const uint32_t sf = smem_base + kOffSf + stage * kSfStageBytes;
          const uint32_t sfa_t = tmem_base + kSfColBase + stage * kSfColsPerStage;
          const uint32_t sfb_t = sfa_t + 4;
          const uint64_t sfd_a = smem_desc(sf, kDescScale), sfd_b0 = smem_desc(sf + kSfBytes, kDescScale),
                         sfd_b1 = smem_desc(sf + 2 * kSfBytes, kDescScale);
          const uint64_t adesc = smem_desc(smem_base + kOffA + stage * kTileBytes, kDescSw128KMajor);
          const uint64_t bdesc = smem_desc(smem_base + kOffB + stage * kTileBytes, kDescSw128KMajor);
          const uint32_t first = kb != 0 ? 1u : 0u;
          const uint32_t empty_own = empty0 + 8u * stage, empty_peer = empty0_peer + 8u * stage;
          if (elect_one_sync()) {
            if (!BF16) {
              tc_cp_32x128b_warpx4_pair(sfa_t, sfd_a);
              tc_cp_32x128b_warpx4_pair(sfb_t, sfd_b0);
              tc_cp_32x128b_warpx4_pair(sfb_t + 4, sfd_b1);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // 32 bytes further along K per MMA: 32 E4M3 or 16 bf16 elements
              if (BF16)
                tc_mma_f16_pair(tmem_base, adesc + 2 * k, bdesc + 2 * k, kIdescPairBf16, k != 0 ? 1u : first);
              else
                tc_mma_mxf8_pair(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc_with_sf(kIdescPair, k), sfa_t, sfb_t,
                                 k != 0 ? 1u : first);
            }
            tc_commit_pair(empty_own);
            tc_commit_pair(empty_peer);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one_sync()) {
          tc_commit_pair(acc_full_own);
          tc_commit_pair(acc_full_peer);
        }
        __syncwarp();
        acc_phase ^= 1u;
      }
      PROF_WRITE(2, t_acc);
      PROF_WRITE(3, t_full);
      PROF_WRITE(4, clock64() - t_begin);
      if (!ok && lane == 0) {
        tc_commit_pair(smem_u32(&bars->drain));
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&bars->drain), 0)) {
          if (clock64() - t0 > 20000000LL) break;
        }
      }
      __syncwarp();
    } else if (MODE == 0 && warp >= 2 && p.pull_xq != nullptr) {
      // ---------------------------------------------------------- dispatch warps (two per CTA)
      // A ticket is two consecutive rows. Their bytes cross as 16-byte asynchronous copies
      // peer -> shared memory (no registers held while the loads are in flight, so both rows,
      // up to 8 KB per warp, travel at once; the ring is the staging area of the row-store
      // epilogue, which this mode does not use), then shared -> A with plain stores, and the ticket
      // is counted into its row tile after a fence. Any resident CTA can serve any ticket, and the
      // dispatch warps wait for nothing, so the tiles the load lanes wait for always complete.
      // (Bulk copies here cost the mainloop as much as the separate pull kernel they replaced: the
      // TMA unit is what feeds the tensor pipe. The load/store path is idle in this kernel.)
      constexpr int kTicketRows = 2;
      const uint32_t ring = smem_base + kOffStaging + static_cast<uint32_t>(warp - 2) * (kStagingBytes / 2);
      const int vecs = p.pull_row_bytes >> 4;                  // <= 256
      const int col_blocks = p.pull_row_bytes >> 7;
      const int rows_live = m_tiles_live * 256;
      for (;;) {
        int base = 0;
        if (lane == 0) base = static_cast<int>(atomicAdd(p.pull_ticket, static_cast<unsigned>(kTicketRows)));
        base = __shfl_sync(0xFFFFFFFFu, base, 0);
        if (base >= rows_live) break;
        int my_src = -1, my_tok = 0;
        if (lane < kTicketRows) {
          my_src = p.pull_peer_rank[base + lane];
          my_tok = my_src >= 0 ? p.pull_token_idx[base + lane] : 0;
        }
        uint32_t word[kTicketRows];
#pragma unroll
        for (int i = 0; i < kTicketRows; ++i) {
          const int src = __shfl_sync(0xFFFFFFFFu, my_src, i);
          const int64_t t = __shfl_sync(0xFFFFFFFFu, my_tok, i);
          word[i] = 0u;
          if (src >= 0) {
            const uint8_t* from = p.pull_xq[src] + t * p.pull_row_bytes;
            for (int v = lane; v < vecs; v += 32)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + i * 4096 + v * 16), "l"(from + v * 16)
                           : "memory");
            if (lane < col_blocks) word[i] = p.pull_sc_rows[src][t * col_blocks + lane];
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
        for (int i = 0; i < kTicketRows; ++i) {
          const int src = __shfl_sync(0xFFFFFFFFu, my_src, i);
          const int r = base + i;
          uint4* dst = reinterpret_cast<uint4*>(p.pull_dst + static_cast<size_t>(r) * p.pull_row_bytes);
          // every lane reads back exactly the 16-byte pieces it copied in
          for (int v = lane; v < vecs; v += 32) {
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
            *reinterpret_cast<uint32_t*>(p.pull_dst_sc + off + static_cast<size_t>(lane) * 512) = word[i];
          }
        }
        // every lane's stores, then one release increment for the ticket
        __threadfence();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(p.pull_ready + (base >> 8), static_cast<unsigned>(kTicketRows));
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue (both CTAs)
    setmaxnreg_inc<kRegsEpilogue>();
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    const int ch = (warp - 4) >> 2;       // which half of the accumulator columns
    const uint32_t acc_empty_leader = mapa_shared(smem_u32(&bars->acc_empty), 0);
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t stage_base = smem_base + kOffStaging + (warp - 4) * 2048;
    uint32_t acc_phase = 0;
    bool ok = true;
    PROF_DECL(t_wait);
    PROF_DECL(t_drain);
    PROF_DECL(t_work);
    for (int tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
      const Tile t = decode_tile<MODE>(p, tile, static_cast<int>(cta_rank), m_tiles_live, m_rot, m_stride);
      const int n_tile = t.n_tile;
      const int64_t row = t.out_row0 + cta_rank * 128 + quad * 32 + lane;
      if (MODE == 2 && t.k_steps == 0) {
        // an expert with no rows: its weight gradient is zero; no accumulator was produced
        uint4* dst = reinterpret_cast<uint4*>(p.out + (row * p.out_cols + n_tile * 256 + ch * 128) * 2);
#pragma unroll
        for (int c = 0; c < 16; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      PROF_T0(tw);
      if (!mbar_wait(smem_u32(&bars->acc_full), acc_phase, p.status, ST_TIMEOUT_TMEM_FULL, 0))
        ok = false;
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      PROF_ADD(t_wait, tw);
      PROF_T0(td);
      tc_fence_after();
      if (MODE == 0) {
        uint32_t g0[32], g1[32], u0[32], u1[32];
        tc_ld_32x32b_x32(taddr + ch * 64, g0);
        tc_ld_32x32b_x32(taddr + ch * 64 + 32, g1);
        tc_ld_32x32b_x32(taddr + 128 + ch * 64, u0);
        tc_ld_32x32b_x32(taddr + 128 + ch * 64 + 32, u1);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty_leader);
        PROF_ADD(t_drain, td);
        PROF_T0(tm);
        if (BF16) {
          if (p.save_gate != nullptr) {
            // training: the bf16 gate and up values the backward pass differentiates through
            uint4* gd = reinterpret_cast<uint4*>(p.save_gate + (static_cast<size_t>(row) * p.out_cols + n_tile * 128 + ch * 64) * 2);
            uint4* ud = reinterpret_cast<uint4*>(p.save_up + (static_cast<size_t>(row) * p.out_cols + n_tile * 128 + ch * 64) * 2);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int i = 8 * c;
              gd[c] = make_uint4(pack_bf16(g0[i], g0[i + 1]), pack_bf16(g0[i + 2], g0[i + 3]), pack_bf16(g0[i + 4], g0[i + 5]), pack_bf16(g0[i + 6], g0[i + 7]));
              gd[4 + c] = make_uint4(pack_bf16(g1[i], g1[i + 1]), pack_bf16(g1[i + 2], g1[i + 3]), pack_bf16(g1[i + 4], g1[i + 5]), pack_bf16(g1[i + 6], g1[i + 7]));
              ud[c] = make_uint4(pack_bf16(u0[i], u0[i + 1]), pack_bf16(u0[i + 2], u0[i + 3]), pack_bf16(u0[i + 4], u0[i + 5]), pack_bf16(u0[i + 6], u0[i + 7]));
              ud[4 + c] = make_uint4(pack_bf16(u1[i], u1[i + 1]), pack_bf16(u1[i + 2], u1[i + 3]), pack_bf16(u1[i + 4], u1[i + 5]), pack_bf16(u1[i + 6], u1[i + 7]));
            }
          }
          // bf16 routed precision: 64 hidden values of this row, 128 contiguous bytes
          uint4* dst = reinterpret_cast<uint4*>(
              p.out + (static_cast<size_t>(row) * p.out_cols + n_tile * 128 + ch * 64) * 2);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t w0[4], w1[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = 8 * c + 2 * j;
              w0[j] = pack_bf16(__float_as_uint(swiglu_bf16(g0[i], u0[i], p.limit)),
                                __float_as_uint(swiglu_bf16(g0[i + 1], u0[i + 1], p.limit)));
              w1[j] = pack_bf16(__float_as_uint(swiglu_bf16(g1[i], u1[i], p.limit)),
                                __float_as_uint(swiglu_bf16(g1[i + 1], u1[i + 1], p.limit)));
            }
            dst[c] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
            dst[4 + c] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
          }
        } else {
        const size_t elem0 = static_cast<size_t>(row) * p.out_cols + n_tile * 128 + ch * 64;
        const size_t sc_off = scale_offset(row, n_tile * 4 + ch * 2, p.out_cols >> 7);
        if (p.save_gate != nullptr) {
          // training: the bf16-rounded gate and up values the backward pass differentiates through,
          // stored as MXFP8 (campaigns/mok/port/gemm/gemm.cu:150-157 emits the same tensors)
          uint4 a0, a1, a2, a3;
          const uint32_t sg0 = quant32_bf16(g0, a0, a1);
          const uint32_t sg1 = quant32_bf16(g1, a2, a3);
          uint4* gd = reinterpret_cast<uint4*>(p.save_gate + elem0);
          gd[0] = a0; gd[1] = a1; gd[2] = a2; gd[3] = a3;
          *reinterpret_cast<uint16_t*>(p.save_gate_sc + sc_off) = static_cast<uint16_t>(sg0 | (sg1 << 8));
          const uint32_t su0 = quant32_bf16(u0, a0, a1);
          const uint32_t su1 = quant32_bf16(u1, a2, a3);
          uint4* ud = reinterpret_cast<uint4*>(p.save_up + elem0);
          ud[0] = a0; ud[1] = a1; ud[2] = a2; ud[3] = a3;
          *reinterpret_cast<uint16_t*>(p.save_up_sc + sc_off) = static_cast<uint16_t>(su0 | (su1 << 8));
        }
        if (p.save_hidden != nullptr) {
          uint32_t* hd = reinterpret_cast<uint32_t*>(p.save_hidden + elem0);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            hd[i >> 1] = pack_bf16(__float_as_uint(swiglu_bf16(g0[i], u0[i], p.limit)), __float_as_uint(swiglu_bf16(g0[i + 1], u0[i + 1], p.limit)));
            hd[16 + (i >> 1)] = pack_bf16(__float_as_uint(swiglu_bf16(g1[i], u1[i], p.limit)), __float_as_uint(swiglu_bf16(g1[i + 1], u1[i + 1], p.limit)));
          }
        }
        uint4 q0, q1, q2, q3;
        const uint32_t e0 = swiglu_quant32(g0, u0, p.limit, q0, q1);
        const uint32_t e1 = swiglu_quant32(g1, u1, p.limit, q2, q3);
        uint4* dst = reinterpret_cast<uint4*>(p.out + row * p.out_cols + n_tile * 128 + ch * 64);
        dst[0] = q0;
        dst[1] = q1;
        dst[2] = q2;
        dst[3] = q3;
        const size_t off = scale_offset(row, n_tile * 4 + ch * 2, p.out_cols >> 7);
        *reinterpret_cast<uint16_t*>(p.out_sc + off) = static_cast<uint16_t>(e0 | (e1 << 8));
        }
        PROF_ADD(t_work, tm);
      } else {
        uint32_t v0[32], v1[32], v2[32], v3[32];
        tc_ld_32x32b_x32(taddr + ch * 128, v0);
        tc_ld_32x32b_x32(taddr + ch * 128 + 32, v1);
        tc_ld_32x32b_x32(taddr + ch * 128 + 64, v2);
        tc_ld_32x32b_x32(taddr + ch * 128 + 96, v3);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty_leader);
        PROF_ADD(t_drain, td);
        PROF_T0(tm);
        // 128 fp32 -> 64 packed bf16 pairs = 16 chunks of 16 bytes
        uint32_t w[64];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          w[i] = pack_bf16(v0[2 * i], v0[2 * i + 1]);
          w[16 + i] = pack_bf16(v1[2 * i], v1[2 * i + 1]);
          w[32 + i] = pack_bf16(v2[2 * i], v2[2 * i + 1]);
          w[48 + i] = pack_bf16(v3[2 * i], v3[2 * i + 1]);
        }
        const int dest = MODE == 2 ? static_cast<int>(row) : p.dest_row[row];
        const int pr = (p.out_peers != nullptr && dest >= 0) ? p.peer_rank[row] : 0;
        const size_t col_byte = (static_cast<size_t>(n_tile) * 256 + ch * 128) * 2;
        // four passes of eight rows through 2 KB of staging per warp: eight lanes park their rows
        // (chunks rotated by the row number, so neither side has bank conflicts), then every store
        // instruction of the warp writes two 256-byte row segments
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          if ((lane >> 3) == h) {
            const uint32_t r8 = lane & 7;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t addr = stage_base + r8 * 256 + ((static_cast<uint32_t>(j) ^ r8) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * j]),
                           "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
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
              *reinterpret_cast<uint4*>(base + static_cast<size_t>(d) * p.out_cols * 2 + col_byte +
                                        c * 16) = val;
            }
          }
          __syncwarp();
        }
        PROF_ADD(t_work, tm);
      }
      acc_phase ^= 1u;
    }
    if (warp == 4 && lane == 0) {
      PROF_WRITE(5, t_wait);
      PROF_WRITE(6, t_drain);
      PROF_WRITE(7, t_work);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn2() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// k counts elements; a box is 128 rows by 128 bytes of K either way.
bool encode_operand(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, bool bf16 = false) {
  EncodeTiledFn fn = encode_fn2();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {bf16 ? 2 * k : k};
  const cuuint32_t box[2] = {bf16 ? 64u : 128u, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Scale tensor seen as [blocks, 128] u32: one row per 512-byte scale block.
bool encode_scales(CUtensorMap* map, const void* base, uint64_t blocks) {
  EncodeTiledFn fn = encode_fn2();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {128, blocks};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, 1};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Requirements beyond launch_grouped_gemm: rows_capacity, every expert segment and
// n_rows are multiples of 256; mode 0 weights are interleaved in blocks of 128 rows.
// Mode 2 (weight gradients): a_fp8 is [m_rows, rows_capacity] and b_fp8 [n_rows, rows_capacity],
// both quantised along the schedule-row dimension; out is bf16 [experts, m_rows, n_rows].
cudaError_t launch_grouped_gemm_pair(const GroupedGemmArgs& a, cudaStream_t stream) {
  if (a.rows_capacity % 256 || a.n_rows % 256 || a.n_rows <= 0) return cudaErrorInvalidValue;
  if (a.mode == 2) {
    if (a.m_rows % 256 || a.m_rows <= 0 || a.expert_offsets == nullptr) return cudaErrorInvalidValue;
  } else if (a.K % 128 || a.K <= 0) {
    return cudaErrorInvalidValue;
  }
  // bf16 training keeps gate and up as bf16 rows (save_gate / save_up); its hidden output is the bf16 value itself
  if (a.bf16 && (a.save_hidden != nullptr || a.save_gate_sc != nullptr || a.save_up_sc != nullptr)) return cudaErrorInvalidValue;
  if (a.rows_capacity == 0 || a.experts == 0) return cudaSuccess;
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  memset(&map_sfa, 0, sizeof(map_sfa));
  memset(&map_sfb, 0, sizeof(map_sfb));
  const uint64_t k_len = a.mode == 2 ? static_cast<uint64_t>(a.rows_capacity) : static_cast<uint64_t>(a.K);
  const uint64_t k_steps = k_len / (a.bf16 ? 64 : 128);
  const uint64_t a_rows = a.mode == 2 ? static_cast<uint64_t>(a.m_rows) : static_cast<uint64_t>(a.rows_capacity);
  const uint64_t b_rows = a.mode == 2 ? static_cast<uint64_t>(a.n_rows) : static_cast<uint64_t>(a.experts) * a.n_rows;
  if (!encode_operand(&map_a, a.a_fp8, a_rows, k_len, a.bf16) || !encode_operand(&map_b, a.b_fp8, b_rows, k_len, a.bf16))
    return cudaErrorInvalidValue;
  if (!a.bf16 && (!encode_scales(&map_sfa, a.a_sc, (a_rows / 128) * k_steps) ||
                  !encode_scales(&map_sfb, a.b_sc, (b_rows / 128) * k_steps)))
    return cudaErrorInvalidValue;
  Params2 p;
  p.prof = static_cast<long long*>(a.profile);
  p.block_expert = a.block_expert;
  p.num_rows_dev = a.num_rows_dev;
  p.m_rotation = a.m_rotation < 0 ? 0 : a.m_rotation;
  p.m_stride = a.m_stride < 1 ? 1 : a.m_stride;
  p.ready = a.ready;
  p.ready_target = a.ready_target;
  p.pull_xq = nullptr;
  if (a.pull_xq != nullptr) {
    if (a.mode != 0 || a.bf16 || a.K > 4096 || !a.pull_sc_rows || !a.pull_peer_rank || !a.pull_token_idx ||
        !a.pull_scratch)
      return cudaErrorInvalidValue;
    const size_t tiles = static_cast<size_t>(a.rows_capacity / 256);
    cudaError_t merr = cudaMemsetAsync(a.pull_scratch, 0, (tiles + 1) * sizeof(unsigned), stream);
    if (merr != cudaSuccess) return merr;
    p.pull_xq = reinterpret_cast<const uint8_t* const*>(a.pull_xq);
    p.pull_sc_rows = reinterpret_cast<const uint32_t* const*>(a.pull_sc_rows);
    p.pull_peer_rank = a.pull_peer_rank;
    p.pull_token_idx = a.pull_token_idx;
    p.pull_dst = static_cast<uint8_t*>(const_cast<void*>(a.a_fp8));
    p.pull_dst_sc = static_cast<uint8_t*>(const_cast<void*>(a.a_sc));
    p.pull_ready = static_cast<unsigned*>(a.pull_scratch);
    p.pull_ticket = static_cast<unsigned*>(a.pull_scratch) + tiles;
    p.pull_row_bytes = a.K;
  }
  p.limit = a.swiglu_limit > 0.0f ? a.swiglu_limit : HUGE_VALF;
  p.max_m_tiles = static_cast<int>(a.rows_capacity / 256);
  p.k_steps = static_cast<int>(k_steps);
  p.n_tiles = a.n_rows / 256;
  p.out_cols = a.mode == 0 ? a.n_rows / 2 : a.n_rows;
  p.out = static_cast<uint8_t*>(a.out);
  p.out_sc = static_cast<uint8_t*>(a.out_sc);
  p.dest_row = a.dest_row;
  p.out_peers = reinterpret_cast<uint8_t* const*>(a.out_peers);
  p.peer_rank = a.peer_rank;
  p.status = a.status;
  p.save_gate = static_cast<uint8_t*>(a.save_gate);
  p.save_gate_sc = static_cast<uint8_t*>(a.save_gate_sc);
  p.save_up = static_cast<uint8_t*>(a.save_up);
  p.save_up_sc = static_cast<uint8_t*>(a.save_up_sc);
  p.save_hidden = static_cast<__nv_bfloat16*>(a.save_hidden);
  p.expert_offsets = a.expert_offsets;
  p.experts = a.experts;
  p.m_tiles = a.mode == 2 ? a.m_rows / 256 : 0;
  p.k_blocks_total = static_cast<int>(k_steps);
  p.k_shift = a.bf16 ? 6 : 7;
  const int grid = a.num_sms & ~1;
  if (grid < 2) return cudaErrorInvalidValue;
  cudaError_t err;
#define PLB_LAUNCH_PAIR(M, B)                                                                           \
  err = cudaFuncSetAttribute(grouped_gemm2_kernel<M, B>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                             kSmemBytes2);                                                              \
  if (err != cudaSuccess) return err;                                                                   \
  grouped_gemm2_kernel<M, B><<<grid, kThreads2, kSmemBytes2, stream>>>(map_a, map_b, map_sfa, map_sfb, p)
  if (a.mode == 0 && a.bf16) {
    PLB_LAUNCH_PAIR(0, true);
  } else if (a.mode == 1 && a.bf16) {
    PLB_LAUNCH_PAIR(1, true);
  } else if (a.mode == 0) {
    PLB_LAUNCH_PAIR(0, false);
  } else if (a.mode == 1) {
    PLB_LAUNCH_PAIR(1, false);
  } else if (a.bf16) {
    PLB_LAUNCH_PAIR(2, true);
  } else {
    PLB_LAUNCH_PAIR(2, false);
  }
#undef PLB_LAUNCH_PAIR
  return cudaGetLastError();
}

}  // namespace plb
