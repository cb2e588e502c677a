// Causal prefill flash-attention forward on tcgen05 (bf16, head_dim 128, sm_100a), with
// the context-parallel hooks of the reference's cp composition.
//
// Stands in for the reference's Hopper core (campaigns/attention/src/sm90/role_core.cuh,
// role_load.cuh, role_epilogue.cuh: M = N = 128 tiles, online softmax, normalised bf16 O and
// LSE = log l + scale * m, src/sm90/README.md:164-165) and for its cp load stage
// (campaigns/attention/src/sm90/cp_load.cuh:19-218): work is a list of descriptors
// {first row of the query tile in Q/O, global position of its first query, KV blocks to
// visit, head, batch} like the reference's WorkDesc (src/sm90/README.md:107-122); keys and
// values are read from buffers laid out in global sequence order, and a KV block can carry a
// readiness counter that the load lane acquires (ld.acquire.sys, bounded) and follows with
// fence.proxy.async before the first TMA of that block (cp_load.cuh:124-137).
//
// Per CTA (192 threads), persistent over the work list:
//   warp 0     TMA: Q tile once per item; K and V blocks through two 2-deep rings
//   warp 1     MMA: S = Q K^T (M128 N128 K16 x 8, both operands K-major, fp32 into one of two
//              128-column TMEM buffers), then O_blk = P V (A = P from shared memory, B = V
//              MN-major) into a third 128-column buffer; QK^T of block j+1 is issued before
//              PV of block j so the tensor pipe works while block j's softmax runs
//   warps 2-5  one query row per thread: scale, causal mask, online max/sum in base 2, P as
//              bf16 into the 128-byte-swizzled A-operand layout, O kept in registers and
//              rescaled per block (O = O * alpha + O_blk), final O / l and LSE
// All peer/global traffic is TMA loads of LOCAL memory and plain stores; nothing is multicast.
#include <cstddef>

#include "attention_roles.cuh"

namespace plb {

using namespace attn;

namespace {

struct AttnBars {
  uint64_t q_full, q_empty;
  uint64_t k_full[kKvStages], k_empty[kKvStages];
  uint64_t v_full[kKvStages], v_empty[kKvStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty;
  uint64_t o_full, o_empty;
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t pad;
};
static_assert(sizeof(AttnBars) <= 256, "barrier block");


template <bool kUseCounters, bool kSoftcap>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sb = raw_addr + pad;
  AttnBars* bars = reinterpret_cast<AttnBars*>(smem + kOffBar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    mbar_init(smem_u32(&bars->q_empty), 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(smem_u32(&bars->k_full[s]), 1);
      mbar_init(smem_u32(&bars->k_empty[s]), 1);
      mbar_init(smem_u32(&bars->v_full[s]), 1);
      mbar_init(smem_u32(&bars->v_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bars->s_full[s]), 1);
      mbar_init(smem_u32(&bars->s_empty[s]), 128);
    }
    mbar_init(smem_u32(&bars->p_full), 128);
    mbar_init(smem_u32(&bars->p_empty), 1);
    mbar_init(smem_u32(&bars->o_full), 1);
    mbar_init(smem_u32(&bars->o_empty), 128);
    mbar_init(smem_u32(&bars->drain), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t q_phase = 0, k_it = 0, v_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.num_work && ok; w += gridDim.x) {
        const AttnWork wk = p.work[w];
        const int col = wk.head * kD;
        const int kv_col = (wk.head / p.q_per_kv) * kD;
        if (!mbar_wait(smem_u32(&bars->q_empty), q_phase ^ 1u, p.status, ST_TIMEOUT_EMPTY, 10)) { ok = false; break; }
        mbar_arrive_expect_tx(smem_u32(&bars->q_full), kTileBytes);
        tma_load_2d(sb + kOffQ, &map_q, smem_u32(&bars->q_full), col, wk.q_row0);
        tma_load_2d(sb + kOffQ + kAtomBytes, &map_q, smem_u32(&bars->q_full), col + 64, wk.q_row0);
        q_phase ^= 1u;
        // K runs one block ahead of V so that QK^T of the next block can be issued early
        for (int j = 0; j < wk.kv_blocks && ok; ++j) {
          const int kv_row = wk.kv_row0 + j * kBlk;
          if (kUseCounters && p.ready != nullptr) {
            // context parallel: a remote block is usable once its pusher published it
            const unsigned* flag = p.ready + (wk.kv_row0 / kBlk + j);
            const long long t0 = clock64();
            while (static_cast<int>(ld_acquire_sys_u32(flag) - p.ready_target) < 0) {
              if (clock64() - t0 > kWaitBudgetCycles || ld_volatile_i32(&p.status->code) != 0) {
                report_failure(p.status, ST_TIMEOUT_COUNTER, 300, ld_acquire_sys_u32(flag), p.ready_target);
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
          {
            const int s = k_it % kKvStages;
            if (!mbar_wait(smem_u32(&bars->k_empty[s]), ((k_it / kKvStages) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, 11)) { ok = false; break; }
            const uint32_t full = smem_u32(&bars->k_full[s]);
            mbar_arrive_expect_tx(full, kTileBytes);
            tma_load_2d(sb + kOffK + s * kTileBytes, &map_k, full, kv_col, kv_row);
            tma_load_2d(sb + kOffK + s * kTileBytes + kAtomBytes, &map_k, full, kv_col + 64, kv_row);
            ++k_it;
          }
          {
            const int s = v_it % kKvStages;
            if (!mbar_wait(smem_u32(&bars->v_empty[s]), ((v_it / kKvStages) & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, 12)) { ok = false; break; }
            const uint32_t full = smem_u32(&bars->v_full[s]);
            mbar_arrive_expect_tx(full, kTileBytes);
            tma_load_2d(sb + kOffV + s * kTileBytes, &map_v, full, kv_col, kv_row);
            tma_load_2d(sb + kOffV + s * kTileBytes + kAtomBytes, &map_v, full, kv_col + 64, kv_row);
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
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t q_phase = 0, k_it = 0, v_it = 0, s_it = 0, pv_it = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t buf) -> bool {
        const int s = k_it % kKvStages;
        if (!mbar_wait(smem_u32(&bars->k_full[s]), (k_it / kKvStages) & 1u, p.status, ST_TIMEOUT_FULL, 20)) return false;
        if (!mbar_wait(smem_u32(&bars->s_empty[buf]), ((s_it >> 1) & 1u) ^ 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, 21)) return false;
        tc_fence_after();
        const uint32_t qa = sb + kOffQ, ka = sb + kOffK + s * kTileBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          tc_mma_f16(tmem_s0 + buf * 128, smem_desc(qa + off, kDescSw128KMajor), smem_desc(ka + off, kDescSw128KMajor),
                     kIdescQK, k != 0 ? 1u : 0u);
        }
        tc_commit(smem_u32(&bars->k_empty[s]));
        tc_commit(smem_u32(&bars->s_full[buf]));
        ++k_it;
        ++s_it;
        return true;
      };
      for (int w = blockIdx.x; w < p.num_work && ok; w += gridDim.x) {
        const AttnWork wk = p.work[w];
        if (!mbar_wait(smem_u32(&bars->q_full), q_phase, p.status, ST_TIMEOUT_FULL, 22)) { ok = false; break; }
        tc_fence_after();
        if (!issue_qk(s_it & 1u)) { ok = false; break; }
        for (int j = 0; j < wk.kv_blocks; ++j) {
          if (j + 1 < wk.kv_blocks) {
            if (!issue_qk(s_it & 1u)) { ok = false; break; }
          }
          const int s = v_it % kKvStages;
          if (!mbar_wait(smem_u32(&bars->v_full[s]), (v_it / kKvStages) & 1u, p.status, ST_TIMEOUT_FULL, 23)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&bars->p_full), pv_it & 1u, p.status, ST_TIMEOUT_FULL, 24)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&bars->o_empty), (pv_it & 1u) ^ 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, 25)) { ok = false; break; }
          tc_fence_after();
          const uint32_t pa = sb + kOffP, va = sb + kOffV + s * kTileBytes;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // A = P: K-major, keys along K (two 64-key atoms); B = V: 16 keys further = 16 rows x 128 B
            const uint32_t a_off = (k >> 2) * kAtomBytes + (k & 3) * 32;
            tc_mma_f16(tmem_o, smem_desc(pa + a_off, kDescSw128KMajor), smem_desc(va + k * 2048, kDescVMn), kIdescPV,
                       k != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&bars->v_empty[s]));
          tc_commit(smem_u32(&bars->p_empty));
          tc_commit(smem_u32(&bars->o_full));
          ++v_it;
          ++pv_it;
        }
        if (!ok) break;
        // Q may be overwritten once every QK^T of this item has completed
        tc_commit(smem_u32(&bars->q_empty));
        q_phase ^= 1u;
      }
      if (!ok) {
        tc_commit(smem_u32(&bars->drain));
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&bars->drain), 0)) {
          if (clock64() - t0 > 20000000LL) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t s_it = 0, pv_it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.num_work && ok; w += gridDim.x) {
      const AttnWork wk = p.work[w];
      const int q_pos = wk.q_pos0 + row;
      float o[kD];
#pragma unroll
      for (int i = 0; i < kD; ++i) o[i] = 0.0f;
      float m = -INFINITY, l = 0.0f;
      for (int j = 0; j < wk.kv_blocks; ++j) {
        const uint32_t buf = s_it & 1u;
        if (!mbar_wait(smem_u32(&bars->s_full[buf]), (s_it >> 1) & 1u, p.status, ST_TIMEOUT_TMEM_FULL, 30)) ok = false;
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after();
        // pass 1 over the 128 scores of this row: block maximum (scaled, causal mask applied)
        const int key0 = wk.kv_pos0 + j * kBlk;
        // visible keys of the row inside this block: [lo, hi); the sliding window keeps
        // kv_pos > q_pos - window (mask_window_mask_mod, campaigns/attention/src/sm90/stage_mask_window.cu:8-11)
        const int hi = q_pos - key0 + 1;
        const int lo = p.window > 0 ? q_pos - p.window + 1 - key0 : 0;
        const bool diag = hi < kBlk || lo > 0;
        float bm = m;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tc_ld_32x32b_x32(tmem_s0 + buf * 128 + lane_addr + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float sv = score_log2<kSoftcap>(__uint_as_float(v[i]), p);
            if (!diag || (c * 32 + i < hi && c * 32 + i >= lo)) bm = fmaxf(bm, sv);
          }
        }
        const float alpha = m == -INFINITY ? 0.0f : exp2f(m - bm);
        // the P buffer is free once P V of the previous block has completed
        if (!mbar_wait(smem_u32(&bars->p_empty), (pv_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, 31)) ok = false;
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        // pass 2: p = exp2(s - max) as bf16 straight into the A-operand layout of P V
        // (two 64-key atoms, 128-byte swizzle); the row sum uses the rounded values
        float sum = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tc_ld_32x32b_x32(tmem_s0 + buf * 128 + lane_addr + c * 32, v);
          tc_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = 0.0f, p1 = 0.0f;
            if (bm != -INFINITY) {
              if (!diag || (c * 32 + i < hi && c * 32 + i >= lo)) p0 = exp2f(score_log2<kSoftcap>(__uint_as_float(v[i]), p) - bm);
              if (!diag || (c * 32 + i + 1 < hi && c * 32 + i + 1 >= lo)) p1 = exp2f(score_log2<kSoftcap>(__uint_as_float(v[i + 1]), p) - bm);
            }
            __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
            sum += __bfloat162float(t.x) + __bfloat162float(t.y);
            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&t);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int cc = c * 4 + q4;  // 16-byte chunk of the row: 8 keys
            const uint32_t addr = sb + kOffP + (cc >> 3) * kAtomBytes + row * 128 + (((cc & 7) ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[q4 * 4]), "r"(pk[q4 * 4 + 1]),
                         "r"(pk[q4 * 4 + 2]), "r"(pk[q4 * 4 + 3])
                         : "memory");
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bars->s_empty[buf]));
        ++s_it;
        l = l * alpha + sum;
        m = bm;
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&bars->p_full));
        // O_blk = P V of this block, folded into the running output
        if (!mbar_wait(smem_u32(&bars->o_full), pv_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, 32)) ok = false;
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tc_ld_32x32b_x32(tmem_o + lane_addr + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(v[i]));
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bars->o_empty));
        ++pv_it;
      }
      if (!ok) break;
      // epilogue: normalise, store bf16 O row and the natural-log LSE
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const size_t out_row = static_cast<size_t>(wk.q_row0 + row);
      uint4* dst = reinterpret_cast<uint4*>(p.out + (out_row * p.q_heads + wk.head) * kD);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint32_t wv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 t = __floats2bfloat162_rn(o[c * 8 + e * 2] * inv, o[c * 8 + e * 2 + 1] * inv);
          wv[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        dst[c] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
      }
      p.lse[(static_cast<size_t>(wk.batch) * p.q_heads + wk.head) * p.seq_q + (wk.q_row0 - wk.batch * p.seq_q) + row] =
          l > 0.0f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Two query heads per CTA. When the number of query heads per KV head is even, one work record
// covers heads h and h+1 of the same 128-query tile: both read the same K/V blocks under the
// same mask, so every K/V tile is fetched once for two S/O tiles and the tensor pipe alternates
// between them while the other tile's softmax runs.
//
// Per CTA (384 threads), persistent over the work list:
//   warp 0     TMA: both Q tiles once per record; K and V blocks through two 2-deep rings
//   warp 1     MMA: S_t = Q_t K^T into TMEM columns [128 t, 128 t + 128); O_t += P_t V with the A
//              operand P_t read from TMEM (bf16, written over the first 64 columns of S_t by the
//              softmax warps) and O_t accumulated in TMEM columns [256 + 128 t, +128) across all
//              blocks of the record. Issue order per block: P0 V, Q0 K'^T, P1 V, Q1 K'^T (K' the
//              next block), so each tile's next scores are queued right behind its P V.
//   warps 4-7  softmax of tile 0, warps 8-11 of tile 1, one query row per thread: the running
//              maximum is only advanced (and O_t, l rescaled in TMEM) when a block raises it by
//              more than 2^8; otherwise exponentials stay relative to the older maximum, which
//              fp32 sums and bf16 P tolerate. Final O_t / l and LSE.
struct PairBars {
  uint64_t q_full, q_empty;
  uint64_t k_full[kKvStages], k_empty[kKvStages];
  uint64_t v_full[kKvStages], v_empty[kKvStages];
  uint64_t s_full[2], p_full[2];
  uint64_t o_full[2], o_free[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t pad;
};
static_assert(sizeof(PairBars) <= 256, "barrier block");

// The library kernel's shared-memory and tensor-memory map, as constants.
#define PLB_PAIR_BAR(name) \
  __device__ static uint32_t name(uint32_t sb, int i = 0) { return sb + kPOffBar + offsetof(PairBars, name) + 8 * i; }
struct LibPairLayout {
  __device__ static constexpr int kv_depth() { return kKvStages; }
  __device__ static constexpr int q() { return kPOffQ; }
  __device__ static constexpr int k() { return kPOffK; }
  __device__ static constexpr int v() { return kPOffV; }
  __device__ static constexpr int s_col() { return 0; }
  __device__ static constexpr int o_col() { return 256; }
  __device__ static constexpr int warp_softmax() { return 4; }
  PLB_PAIR_BAR(q_full) PLB_PAIR_BAR(q_empty) PLB_PAIR_BAR(k_full) PLB_PAIR_BAR(k_empty) PLB_PAIR_BAR(v_full)
  PLB_PAIR_BAR(v_empty) PLB_PAIR_BAR(s_full) PLB_PAIR_BAR(p_full) PLB_PAIR_BAR(o_full) PLB_PAIR_BAR(o_free) PLB_PAIR_BAR(drain)
};
#undef PLB_PAIR_BAR

template <bool kUseCounters, bool kSoftcap>
__global__ void __launch_bounds__(kPairThreads, 1)
attention_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sb = raw_addr + pad;
  PairBars* bars = reinterpret_cast<PairBars*>(smem + kPOffBar);
  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);   // warp-uniform, and said so to the compiler
  using L = LibPairLayout;

  if (threadIdx.x == 0) {
    mbar_init(L::q_full(sb), 1);
    mbar_init(L::q_empty(sb), 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(L::k_full(sb, s), 1);
      mbar_init(L::k_empty(sb, s), 1);
      mbar_init(L::v_full(sb, s), 1);
      mbar_init(L::v_empty(sb, s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(L::s_full(sb, t), 1);
      mbar_init(L::p_full(sb, t), 128);
      mbar_init(L::o_full(sb, t), 1);
      mbar_init(L::o_free(sb, t), 128);
    }
    mbar_init(L::drain(sb), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    load_role<L, kUseCounters>(&map_q, &map_k, &map_v, p, sb);
  } else if (warp == 1) {
    mma_role<L>(p, sb, tmem);
  } else if (warp < 4) {
    if (kUseCounters && p.push_k != nullptr) gather_role(p);
  } else {
    softmax_role<L, kSoftcap>(p, sb, tmem);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, cols] bf16 row-major; box = 128 rows x 64 columns (128 bytes), 128-byte swizzle.
bool encode_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return false;
    fn = reinterpret_cast<EncodeFn>(sym);
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_attention_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.num_work == 0) return cudaSuccess;
  CUtensorMap mq, mk, mv;
  if (!encode_bf16(&mq, a.q, a.q_rows, static_cast<uint64_t>(a.q_heads) * kD) ||
      !encode_bf16(&mk, a.k, a.kv_rows, static_cast<uint64_t>(a.kv_heads) * kD) ||
      !encode_bf16(&mv, a.v, a.kv_rows, static_cast<uint64_t>(a.kv_heads) * kD))
    return cudaErrorInvalidValue;
  AttnParams p;
  p.work = a.work;
  p.num_work = a.num_work;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.lse = a.lse;
  p.q_heads = a.q_heads;
  p.q_per_kv = a.q_heads / a.kv_heads;
  p.seq_q = a.seq_q;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.ready = a.ready;
  p.ready_target = a.ready_target;
  p.status = a.status;
  p.push_k = nullptr;
  if (a.push_k != nullptr) {
    // the gather warps live in the two-heads-per-CTA kernel; a piece is a whole number of 16-byte words
    if (a.heads_per_work != 2 || a.ready == nullptr || !a.push_v || !a.push_k_peers || !a.push_v_peers ||
        !a.push_ready_peers || !a.push_ticket || a.push_parts < 1 || a.push_world < 1 || a.push_rank < 0 ||
        a.push_rank >= a.push_world || a.push_chunk_blocks < 0 || a.push_block_bytes <= 0 ||
        a.push_block_bytes % (16 * a.push_parts))
      return cudaErrorInvalidValue;
    cudaError_t merr = cudaMemsetAsync(a.push_ticket, 0, sizeof(unsigned), stream);
    if (merr != cudaSuccess) return merr;
    p.push_k = static_cast<const uint4*>(a.push_k);
    p.push_v = static_cast<const uint4*>(a.push_v);
    p.push_k_peers = reinterpret_cast<uint4* const*>(a.push_k_peers);
    p.push_v_peers = reinterpret_cast<uint4* const*>(a.push_v_peers);
    p.push_ready_peers = a.push_ready_peers;
    p.push_ticket = a.push_ticket;
    p.push_chunk_blocks = a.push_chunk_blocks;
    p.push_parts = a.push_parts;
    p.push_vec_per_part = static_cast<int>((a.push_block_bytes / a.push_parts) >> 4);
    p.push_rank = a.push_rank;
    p.push_world = a.push_world;
  }
  int grid = a.num_sms < a.num_work ? a.num_sms : a.num_work;
  cudaError_t err;
  p.window = a.window;
  p.cap_in = a.softcap > 0.0f ? a.scale / a.softcap : 0.0f;
  p.cap_out = a.softcap * 1.4426950408889634f;
  const bool counters = a.ready != nullptr, cap = a.softcap > 0.0f;
  if (a.heads_per_work == 2) {
    if (p.q_per_kv % 2 != 0) return cudaErrorInvalidValue;
    auto kern = counters ? (cap ? attention_fwd_pair_kernel<true, true> : attention_fwd_pair_kernel<true, false>)
                         : (cap ? attention_fwd_pair_kernel<false, true> : attention_fwd_pair_kernel<false, false>);
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (err != cudaSuccess) return err;
    kern<<<grid, kPairThreads, kPairSmem, stream>>>(mq, mk, mv, p);
  } else {
    auto kern = counters ? (cap ? attention_fwd_kernel<true, true> : attention_fwd_kernel<true, false>)
                         : (cap ? attention_fwd_kernel<false, true> : attention_fwd_kernel<false, false>);
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (err != cudaSuccess) return err;
    kern<<<grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, p);
  }
  return cudaGetLastError();
}

}  // namespace plb
