// The two-heads-per-CTA prefill attention kernel's device code as four warp roles (TMA producer, MMA
// issuer, K/V gather warps, softmax + epilogue), shared by the library kernel (attention.cu:
// attention_fwd_pair_kernel) and by the separately packed stage owners (stages/attention). Where the
// barriers, the operand tiles and the tensor-memory columns are is a layout policy L: the library
// kernel states constants, a linked image reads link-time handles. See attention.cu for what the
// kernel is and which reference files it follows.
#pragma once
#include "kernels.h"
#include "attention.h"

namespace plb {
namespace attn {
namespace {   // internal linkage: compiled into the library kernel and into each stage unit

constexpr int kD = 128;                 // head dim
constexpr int kBlk = 128;               // queries per tile, keys per block
constexpr int kAtomBytes = kBlk * 128;  // 128 rows x 128 bytes (64 bf16): one swizzle atom column
constexpr int kTileBytes = 2 * kAtomBytes;  // 128 x 128 bf16
constexpr int kKvStages = 2;
constexpr int kOffQ = 0;
constexpr int kOffK = kTileBytes;
constexpr int kOffV = kOffK + kKvStages * kTileBytes;
constexpr int kOffP = kOffV + kKvStages * kTileBytes;
constexpr int kOffBar = kOffP + kTileBytes;
constexpr int kAttnSmem = kOffBar + 256 + 1024;
constexpr int kAttnThreads = 192;
constexpr uint32_t kIdescQK = idesc_bf16(kBlk, kBlk, 0, 0);
constexpr uint32_t kIdescPV = idesc_bf16(kBlk, kD, 0, 1);       // B (= V) is MN-major
constexpr uint64_t kDescVMn = smem_desc_hi(1024, kAtomBytes, 2);  // 8-key groups 1 KB apart, d-halves 16 KB apart

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Raw score q.k -> score in the base-2 softmax domain. Plain: s * scale * log2(e). With a soft cap c
// (score_softcap_score_mod, campaigns/attention/src/sm90/stage_score_softcap.cu:10-13): the scaled
// score becomes c * tanh(s * scale / c); cap_in = scale / c, cap_out = c * log2(e).
template <bool kSoftcap>
__device__ __forceinline__ float score_log2(float s, const AttnParams& p) {
  // explicit roundings: whether a multiply fuses into the subtraction that follows is otherwise the
  // compiler's choice per build, and the library kernel and a linked image must give the same bits
  return kSoftcap ? __fmul_rn(p.cap_out, tanh_approx(__fmul_rn(s, p.cap_in))) : __fmul_rn(s, p.scale_log2);
}

constexpr int kPairThreads = 384;  // warpgroup 0: TMA, MMA, two idle warps; warpgroups 1 and 2: softmax
constexpr int kPOffQ = 0;                              // two Q tiles
constexpr int kPOffK = 2 * kTileBytes;
constexpr int kPOffV = kPOffK + kKvStages * kTileBytes;
constexpr int kPOffBar = kPOffV + kKvStages * kTileBytes;
constexpr int kPairSmem = kPOffBar + 256 + 1024;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// ------------------------------------------------------------------ TMA producer (one warp)
// Both Q tiles once per record; K and V blocks through two rings of L::kv_depth() stages. With
// kUseCounters a key block's readiness counter is acquired before its first read (context parallel).
// The whole warp walks the loop, so coordinates and barrier addresses are warp-uniform, and one
// elected lane issues the copies (see mma_role).
template <class L, bool kUseCounters>
__device__ __forceinline__ void load_role(const CUtensorMap* map_q, const CUtensorMap* map_k, const CUtensorMap* map_v,
                                          const AttnParams& p, uint32_t sb) {
  const int lane = threadIdx.x & 31;
  uint32_t q_phase = 0, k_it = 0, v_it = 0;
  bool ok = true;
  auto wait = [&](uint32_t bar, uint32_t parity, int code, int what) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, p.status, code, what)) != 0;
  };
  for (int w = blockIdx.x; w < p.num_work && ok; w += gridDim.x) {
    const AttnWork wk = p.work[w];
    const int head = __shfl_sync(0xFFFFFFFFu, wk.head, 0), q_row0 = __shfl_sync(0xFFFFFFFFu, wk.q_row0, 0);
    const int kv_row0 = __shfl_sync(0xFFFFFFFFu, wk.kv_row0, 0), kv_blocks = __shfl_sync(0xFFFFFFFFu, wk.kv_blocks, 0);
    const int col = head * kD;
    const int kv_col = (head / p.q_per_kv) * kD;
    if (!wait(L::q_empty(sb), q_phase ^ 1u, ST_TIMEOUT_EMPTY, 10)) { ok = false; break; }
    {
      const uint32_t q_full = L::q_full(sb), q_dst = sb + L::q();
      if (elect_one_sync()) {
        mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
#pragma unroll
        for (int a = 0; a < 4; ++a)  // tile t = a / 2 (head + t), 64-column half a % 2
          tma_load_2d(q_dst + a * kAtomBytes, map_q, q_full, col + a * 64, q_row0);
      }
      __syncwarp();
    }
    q_phase ^= 1u;
    for (int j = 0; j < kv_blocks && ok; ++j) {
      const int kv_row = kv_row0 + j * kBlk;
      if (kUseCounters && p.ready != nullptr) {
        if (lane == 0) {
          const unsigned* flag = p.ready + (kv_row0 / kBlk + j);
          const long long t0 = clock64();
          while (static_cast<int>(ld_acquire_sys_u32(flag) - p.ready_target) < 0) {
            if (clock64() - t0 > kWaitBudgetCycles || ld_volatile_i32(&p.status->code) != 0) {
              report_failure(p.status, ST_TIMEOUT_COUNTER, 300, ld_acquire_sys_u32(flag), p.ready_target);
              ok = false;
              break;
            }
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        ok = __all_sync(0xFFFFFFFFu, ok) != 0;
        if (!ok) break;
      }
      {
        const uint32_t s = k_it % L::kv_depth();
        if (!wait(L::k_empty(sb, s), ((k_it / L::kv_depth()) & 1u) ^ 1u, ST_TIMEOUT_EMPTY, 11)) { ok = false; break; }
        const uint32_t full = L::k_full(sb, s), dst = sb + L::k() + s * kTileBytes;
        if (elect_one_sync()) {
          mbar_arrive_expect_tx(full, kTileBytes);
          tma_load_2d(dst, map_k, full, kv_col, kv_row);
          tma_load_2d(dst + kAtomBytes, map_k, full, kv_col + 64, kv_row);
        }
        __syncwarp();
        ++k_it;
      }
      {
        const uint32_t s = v_it % L::kv_depth();
        if (!wait(L::v_empty(sb, s), ((v_it / L::kv_depth()) & 1u) ^ 1u, ST_TIMEOUT_EMPTY, 12)) { ok = false; break; }
        const uint32_t full = L::v_full(sb, s), dst = sb + L::v() + s * kTileBytes;
        if (elect_one_sync()) {
          mbar_arrive_expect_tx(full, kTileBytes);
          tma_load_2d(dst, map_v, full, kv_col, kv_row);
          tma_load_2d(dst + kAtomBytes, map_v, full, kv_col + 64, kv_row);
        }
        __syncwarp();
        ++v_it;
      }
    }
  }
  if (!ok) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000LL) {
    }
  }
}

// ------------------------------------------------------------------ MMA issuer (one warp)
// The whole warp walks the loop: ring positions, descriptors, tensor-memory and barrier addresses are
// computed in convergent code, so they are warp-uniform, and one elected lane issues the tensor
// instructions and commits. Computed by one lane in a divergent branch the operands sit in per-thread
// registers and every instruction pays for moving them: with 32 small MMAs per key block the issuing
// thread, not the tensor pipe, then bounds the kernel.
template <class L>
__device__ __forceinline__ void mma_role(const AttnParams& p, uint32_t sb, uint32_t tmem_in) {
  const int lane = threadIdx.x & 31;
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, tmem_in, 0);
  uint32_t q_phase = 0, k_it = 0, v_it = 0, blk_it = 0, item_it = 0;
  bool ok = true;
  auto wait = [&](uint32_t bar, uint32_t parity, int code, int what) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, p.status, code, what)) != 0;
  };
  // the eight K16 steps of S_t = Q_t K^T into tile t's score columns, then the score barrier
  auto issue_qk = [&](int t, uint32_t ks) {
    const uint64_t qd = smem_desc(sb + L::q() + t * kTileBytes, kDescSw128KMajor), kd = smem_desc(sb + L::k() + ks * kTileBytes, kDescSw128KMajor);
    const uint32_t s_t = tmem + L::s_col() + t * 128, s_full = L::s_full(sb, t);
    if (elect_one_sync()) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = ((k >> 2) * kAtomBytes + (k & 3) * 32) >> 4;      // descriptor address units of 16 bytes
        tc_mma_f16(s_t, qd + off, kd + off, kIdescQK, k != 0 ? 1u : 0u);
      }
      tc_commit(s_full);
    }
    __syncwarp();
  };
  auto commit = [&](uint32_t bar) {
    if (elect_one_sync()) tc_commit(bar);
    __syncwarp();
  };
  const int num_work = p.num_work;
  for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
    const int n = __shfl_sync(0xFFFFFFFFu, p.work[w].kv_blocks, 0);
    if (!wait(L::q_full(sb), q_phase, ST_TIMEOUT_FULL, 22)) { ok = false; break; }
    {
      const uint32_t ks = k_it % L::kv_depth();
      if (!wait(L::k_full(sb, ks), (k_it / L::kv_depth()) & 1u, ST_TIMEOUT_FULL, 20)) { ok = false; break; }
      tc_fence_after();
      issue_qk(0, ks);
      issue_qk(1, ks);
      commit(L::k_empty(sb, ks));
      ++k_it;
    }
    for (int j = 0; j < n && ok; ++j) {
      const bool have_next = j + 1 < n;
      const uint32_t vs = v_it % L::kv_depth(), ks = k_it % L::kv_depth();
      if (!wait(L::v_full(sb, vs), (v_it / L::kv_depth()) & 1u, ST_TIMEOUT_FULL, 23)) { ok = false; break; }
      if (have_next && !wait(L::k_full(sb, ks), (k_it / L::kv_depth()) & 1u, ST_TIMEOUT_FULL, 26)) { ok = false; break; }
      const uint64_t vd = smem_desc(sb + L::v() + vs * kTileBytes, kDescVMn);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!wait(L::p_full(sb, t), blk_it & 1u, ST_TIMEOUT_FULL, 24)) { ok = false; break; }
        // the first P V of a record overwrites O_t: the previous record's epilogue must have read it
        if (j == 0 && !wait(L::o_free(sb, t), (item_it & 1u) ^ 1u, ST_TIMEOUT_TMEM_EMPTY, 25)) { ok = false; break; }
        tc_fence_after();
        const uint32_t o_t = tmem + L::o_col() + t * 128, p_t = tmem + L::s_col() + t * 128, o_full = L::o_full(sb, t);
        const uint32_t first = j != 0 ? 1u : 0u;
        if (elect_one_sync()) {
#pragma unroll
          for (int k = 0; k < 8; ++k)  // 16 keys per step: 8 packed columns of P, 16 rows x 128 B of V
            tc_mma_f16_ts(o_t, p_t + k * 8, vd + ((k * 2048) >> 4), kIdescPV, k != 0 ? 1u : first);
          if (!have_next) tc_commit(o_full);
        }
        __syncwarp();
        if (have_next) issue_qk(t, ks);
      }
      if (!ok) break;
      commit(L::v_empty(sb, vs));
      ++v_it;
      if (have_next) {
        commit(L::k_empty(sb, ks));
        ++k_it;
      }
      ++blk_it;
    }
    if (!ok) break;
    commit(L::q_empty(sb));
    q_phase ^= 1u;
    ++item_it;
  }
  if (!ok && lane == 0) {
    tc_commit(L::drain(sb));
    const long long t0 = clock64();
    while (!mbar_try_wait(L::drain(sb), 0)) {
      if (clock64() - t0 > 20000000LL) break;
    }
  }
  __syncwarp();
}

// ------------------------------------------------------------------ K/V gather warps (two warps)
__device__ __forceinline__ void gather_role(const AttnParams& p) {
  const int lane = threadIdx.x & 31;
  // ------------------------------------------------------------------ K/V gather warps (2 and 3)
  // The context-parallel exchange inside the attention launch (the reference puts its gather warps
  // into the attention CTA the same way, campaigns/attention/src/sm90/stage_kv_gather.cu:16-78, with
  // the ticket / publish primitives of examples/comm-overlap/comm/push_gather.cuh:80-150). Tickets
  // come from one global counter, so any resident CTA serves any piece and progress never depends
  // on which CTA got which attention tile; the warps wait for nothing. Order: ascending global
  // position, the order in which every consumer's tiles read their key blocks. Zigzag ownership
  // (campaigns/attention/README.md:222-228): rank r holds chunks r and 2W-1-r of 2W; the early chunk is
  // needed by every rank, the late chunk only by ranks <= r.
  const int cb = p.push_chunk_blocks, parts = p.push_parts, W = p.push_world, r = p.push_rank;
  const int early_tasks = cb * W, late_tasks = cb * (r + 1);
  const unsigned total = static_cast<unsigned>(early_tasks + late_tasks) * static_cast<unsigned>(parts);
  for (;;) {
    unsigned tk = 0;
    if (lane == 0) tk = atomicAdd(p.push_ticket, 1u);
    tk = __shfl_sync(0xFFFFFFFFu, tk, 0);
    if (tk >= total) break;
    const int task = static_cast<int>(tk / parts), part = static_cast<int>(tk - static_cast<unsigned>(task) * parts);
    int local_block, consumer, global_block;
    if (task < early_tasks) {
      const int b = task / W;
      consumer = task - b * W;
      local_block = b;
      global_block = r * cb + b;
    } else {
      const int u = task - early_tasks;
      const int b = u / (r + 1);
      consumer = u - b * (r + 1);
      local_block = cb + b;
      global_block = (2 * W - 1 - r) * cb + b;
    }
    const size_t src_off = (static_cast<size_t>(local_block) * parts + part) * p.push_vec_per_part;
    const size_t dst_off = (static_cast<size_t>(global_block) * parts + part) * p.push_vec_per_part;
    const uint4* ks = p.push_k + src_off;
    const uint4* vs = p.push_v + src_off;
    uint4* kd = p.push_k_peers[consumer] + dst_off;
    uint4* vd = p.push_v_peers[consumer] + dst_off;
    for (int i0 = lane; i0 < p.push_vec_per_part; i0 += 128) {   // loads batched before the stores
      uint4 a[4], b4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 32;
        if (i < p.push_vec_per_part) { a[u] = ks[i]; b4[u] = vs[i]; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 32;
        if (i < p.push_vec_per_part) { kd[i] = a[u]; vd[i] = b4[u]; }
      }
    }
    __threadfence_system();       // every lane's stores, then one release increment for the piece
    __syncwarp();
    if (lane == 0)
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.push_ready_peers[consumer] + global_block), "r"(1u)
                   : "memory");
  }
}

// ------------------------------------------------------------------ softmax + epilogue (eight warps)
// Warps L::warp_softmax() .. +3 take tile 0, the next four tile 1; a warp's TMEM lane quadrant is its
// index mod 4, so the role starts on a multiple of four.
template <class L, bool kSoftcap>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t sb, uint32_t tmem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = (warp - L::warp_softmax()) >> 2;     // tile (head offset) of this warp
  const int quad = warp & 3;         // TMEM lane quadrant this warp may touch
  const int row = quad * 32 + lane;  // query row inside the tile == TMEM lane
  const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
  const uint32_t tmem_s = tmem + L::s_col() + t * 128 + lane_addr;
  const uint32_t tmem_o = tmem + L::o_col() + t * 128 + lane_addr;
  const float scale = p.scale_log2;
  uint32_t blk_it = 0, item_it = 0;
  bool ok = true;
  for (int w = blockIdx.x; w < p.num_work && ok; w += gridDim.x) {
    const AttnWork wk = p.work[w];
    const int head = wk.head + t;
    const int q_pos = wk.q_pos0 + row;
    float m_ref = -INFINITY, l = 0.0f;
    for (int j = 0; j < wk.kv_blocks; ++j) {
      if (!mbar_wait(L::s_full(sb, t), blk_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, 30)) ok = false;
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int key0 = wk.kv_pos0 + j * kBlk;
      const int valid = q_pos - key0 + 1;  // keys [lo, valid) of this block are visible to the row
      const int lo = p.window > 0 ? q_pos - p.window + 1 - key0 : 0;
      // uniform per block: some row of the tile is masked (causal edge or the window's lower edge)
      const bool diag = key0 + kBlk - 1 > wk.q_pos0 || (p.window > 0 && wk.q_pos0 + kBlk - 1 - p.window + 1 > key0);
      float bm = -INFINITY;
      {
        // pass 1: block maximum of the raw scores, two 32-column chunks in flight
        float b0 = -INFINITY, b1 = -INFINITY;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t a[32], b[32];
          tc_ld_32x32b_x32(tmem_s + h * 64, a);
          tc_ld_32x32b_x32(tmem_s + h * 64 + 32, b);
          tc_wait_ld();
          if (diag) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (h * 64 + i < valid && h * 64 + i >= lo) b0 = fmaxf(b0, __uint_as_float(a[i]));
              if (h * 64 + 32 + i < valid && h * 64 + 32 + i >= lo) b1 = fmaxf(b1, __uint_as_float(b[i]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              b0 = fmaxf(b0, __uint_as_float(a[i]));
              b1 = fmaxf(b1, __uint_as_float(b[i]));
            }
          }
        }
        bm = fmaxf(b0, b1);
      }
      bm = bm == -INFINITY ? bm : score_log2<kSoftcap>(bm, p);  // monotonic: the maximum of the scores is the score of the maximum
      const float m_new = fmaxf(m_ref, bm);
      const bool need = m_new > m_ref && (m_ref == -INFINITY || m_new - m_ref > kRescaleThreshold);
      if (__any_sync(0xFFFFFFFFu, need)) {
        if (j > 0) {
          // O_t holds the sum over blocks 0..j-1 (their P V completed before this block's scores)
          const float alpha = m_new == m_ref ? 1.0f : ex2_approx(m_ref - m_new);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            tc_ld_32x32b_x32(tmem_o + c * 32, ov);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tc_st_32x32b_x32(tmem_o + c * 32, ov);
          }
          tc_wait_st();
          l *= alpha;
        }
        m_ref = m_new;
      }
      const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
      // P = exp2(s * scale - m_ref) as bf16, two per 32-bit column, over the first 64 columns of S_t
      // pass 2: scores are read again from TMEM (cheaper than holding 128 of them in registers);
      // P of columns [64 h, 64 h + 64) lands on columns [32 h, 32 h + 32), all of them already read
      float sum0 = 0.0f, sum1 = 0.0f;
      auto half = [&](auto masked, int h) {
        uint32_t a[32], b[32], pk[32];
        tc_ld_32x32b_x32(tmem_s + h * 64, a);
        tc_ld_32x32b_x32(tmem_s + h * 64 + 32, b);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0, a1, c0, c1;
          if (kSoftcap) {
            a0 = ex2_approx(__fsub_rn(score_log2<true>(__uint_as_float(a[i]), p), m_use));
            a1 = ex2_approx(__fsub_rn(score_log2<true>(__uint_as_float(a[i + 1]), p), m_use));
            c0 = ex2_approx(__fsub_rn(score_log2<true>(__uint_as_float(b[i]), p), m_use));
            c1 = ex2_approx(__fsub_rn(score_log2<true>(__uint_as_float(b[i + 1]), p), m_use));
          } else {
            a0 = ex2_approx(fmaf(__uint_as_float(a[i]), scale, -m_use));
            a1 = ex2_approx(fmaf(__uint_as_float(a[i + 1]), scale, -m_use));
            c0 = ex2_approx(fmaf(__uint_as_float(b[i]), scale, -m_use));
            c1 = ex2_approx(fmaf(__uint_as_float(b[i + 1]), scale, -m_use));
          }
          if (decltype(masked)::value) {
            if (h * 64 + i >= valid || h * 64 + i < lo) a0 = 0.0f;
            if (h * 64 + i + 1 >= valid || h * 64 + i + 1 < lo) a1 = 0.0f;
            if (h * 64 + 32 + i >= valid || h * 64 + 32 + i < lo) c0 = 0.0f;
            if (h * 64 + 32 + i + 1 >= valid || h * 64 + 32 + i + 1 < lo) c1 = 0.0f;
          }
          sum0 += a0 + a1;
          sum1 += c0 + c1;
          __nv_bfloat162 pa = __floats2bfloat162_rn(a0, a1), pc = __floats2bfloat162_rn(c0, c1);
          pk[i >> 1] = *reinterpret_cast<uint32_t*>(&pa);
          pk[16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&pc);
        }
        tc_st_32x32b_x32(tmem_s + h * 32, pk);
      };
      if (diag) {
        half(TrueTag{}, 0);
        half(TrueTag{}, 1);
      } else {
        half(FalseTag{}, 0);
        half(FalseTag{}, 1);
      }
      tc_wait_st();
      l += sum0 + sum1;
      tc_fence_before();
      mbar_arrive(L::p_full(sb, t));
      ++blk_it;
    }
    if (!ok) break;
    // epilogue: O_t / l as bf16 and the natural-log LSE
    if (!mbar_wait(L::o_full(sb, t), item_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, 32)) ok = false;
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (!ok) break;
    tc_fence_after();
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    const size_t out_row = static_cast<size_t>(wk.q_row0 + row);
    uint4* dst = reinterpret_cast<uint4*>(p.out + (out_row * p.q_heads + head) * kD);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t ov[32];
      tc_ld_32x32b_x32(tmem_o + c * 32, ov);
      tc_wait_ld();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t wv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 tt = __floats2bfloat162_rn(__uint_as_float(ov[g * 8 + e * 2]) * inv,
                                                    __uint_as_float(ov[g * 8 + e * 2 + 1]) * inv);
          wv[e] = *reinterpret_cast<uint32_t*>(&tt);
        }
        dst[c * 4 + g] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
      }
    }
    tc_fence_before();
    mbar_arrive(L::o_free(sb, t));
    ++item_it;
    p.lse[(static_cast<size_t>(wk.batch) * p.q_heads + head) * p.seq_q + (wk.q_row0 - wk.batch * p.seq_q) + row] =
        l > 0.0f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace
}  // namespace attn
}  // namespace plb
