// Grouped MXFP8 GEMM for MoE experts on tcgen05 block-scaled MMA (sm_100a).
//
// Replaces the reference's expert_grouped_gemm_kernel cases FWD_ROUTED_GATE/UP and
// FWD_ROUTED_DOWN (campaigns/mok/port/gemm/gemm.cu:150-162) and, in mode 0, also the
// SwiGLU + requantise stage that follows it there (campaigns/mok/port/act/act.cu:100-178):
// the accumulator goes from tensor memory straight through silu(gate)*up, the bf16
// rounding the reference applies between the two stages, and MXFP8 quantisation.
//
// One persistent CTA per SM, 256 threads:
//   warp 0      TMA producer: per 128-byte K step one A tile (128 rows), one B tile
//               (128 weight rows) and the two 512-byte scale blocks into a 6-deep ring
//   warp 1      MMA issuer: copies the scale blocks into tensor memory, issues four
//               K=32 kind::mxf8f6f4.block_scale MMAs per step, commits to the ring's
//               empty barrier and, per tile, to the accumulator's full barrier
//   warp 2      allocates / frees tensor memory
//   warps 4-7   epilogue: each warp drains its own 32-lane quadrant of one of the two
//               128-column accumulators while the MMA warp fills the other one
//
// Tiles are (128-row block of the padded schedule) x (128 weight rows of that
// block's expert); tile index = m_block * n_tiles + n_tile, strided over the grid so
// CTAs running together share one expert's weights in L2.
#include "kernels.h"
#include "mxfp8.cuh"

namespace plb {

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;  // bytes == E4M3 elements per K step; one 128-byte swizzle atom
constexpr int kStages = 6;
constexpr int kABytes = BM * BK;
constexpr int kBBytes = BN * BK;
constexpr int kSfBytes = 512;
constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;  // 33,792 = 33 * 1024
constexpr int kTmemCols = 512;
constexpr int kAccCols = BN;           // fp32 accumulator: one column per output column
constexpr int kSfColBase = 2 * kAccCols;  // scale columns start after the two accumulators
constexpr int kThreadsGemm = 256;
constexpr int kEpilogueThreads = 128;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack

constexpr uint32_t kIdesc = idesc_mxf8(BM, BN);

struct Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

struct KernelParams {
  const uint8_t* a_sc;
  const uint8_t* b_sc;
  const int* block_expert;
  const int* num_rows_dev;
  int max_m_blocks;
  int k_steps;     // K / 128
  int n_tiles;     // weight rows per expert / 128
  int out_cols;    // mode 0: intermediate size I; mode 1: hidden size H
  uint8_t* out;
  uint8_t* out_sc;
  const int* dest_row;
  uint8_t* const* out_peers;  // mode 1, optional: output base per source rank (peer-mapped)
  const int* peer_rank;       // mode 1 with out_peers: which base row p goes to
  Status* status;
  float limit;  // mode 0: SwiGLU clamp bound, +inf when off
};

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

template <int MODE>
__global__ void __launch_bounds__(kThreadsGemm, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int live_rows = *p.num_rows_dev;
  int m_blocks = live_rows >> 7;
  if (m_blocks > p.max_m_blocks) m_blocks = p.max_m_blocks;
  const int total_tiles = m_blocks * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->acc_full[i]), 1);
      mbar_init(smem_u32(&bars->acc_empty[i]), kEpilogueThreads);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / p.n_tiles;
        const int n_blk = tile - m_blk * p.n_tiles;
        const int expert = p.block_expert[m_blk];
        const int b_row_blk = expert * p.n_tiles + n_blk;
        const uint8_t* sfa = p.a_sc + static_cast<size_t>(m_blk) * p.k_steps * kSfBytes;
        const uint8_t* sfb = p.b_sc + static_cast<size_t>(b_row_blk) * p.k_steps * kSfBytes;
        for (int kb = 0; kb < p.k_steps; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, p.status, ST_TIMEOUT_EMPTY,
                         stage)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t base = smem_base + stage * kStageBytes;
          mbar_arrive_expect_tx(full, kStageBytes);
          tma_load_2d(base, &map_a, full, kb * BK, m_blk * BM);
          tma_load_2d(base + kABytes, &map_b, full, kb * BK, b_row_blk * BN);
          bulk_load(base + kABytes + kBBytes, sfa + static_cast<size_t>(kb) * kSfBytes, kSfBytes,
                    full);
          bulk_load(base + kABytes + kBBytes + kSfBytes, sfb + static_cast<size_t>(kb) * kSfBytes,
                    kSfBytes, full);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let every copy this thread started land before the CTA can exit
        for (int s = 0; s < kStages; ++s) {
          const uint32_t par = s < stage ? phase : (phase ^ 1u);
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&bars->full[s]), par)) {
            if (clock64() - t0 > 20000000LL) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase ^ 1u, p.status,
                       ST_TIMEOUT_TMEM_EMPTY, acc)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < p.k_steps; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, p.status, ST_TIMEOUT_FULL, stage)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t base = smem_base + stage * kStageBytes;
          const uint32_t sfa_t = tmem_base + kSfColBase + stage * 8;
          const uint32_t sfb_t = sfa_t + 4;
          tc_cp_32x128b_warpx4(sfa_t, smem_desc(base + kABytes + kBBytes, kDescScale));
          tc_cp_32x128b_warpx4(sfb_t, smem_desc(base + kABytes + kBBytes + kSfBytes, kDescScale));
          const uint64_t adesc = smem_desc(base, kDescSw128KMajor);
          const uint64_t bdesc = smem_desc(base + kABytes, kDescSw128KMajor);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes further along K inside the swizzle atom = +2 in the address field
            tc_mma_mxf8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_with_sf(kIdesc, k), sfa_t,
                        sfb_t, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&bars->empty[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(smem_u32(&bars->acc_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        // wait for the MMAs already issued so tensor memory can be freed safely
        tc_commit(smem_u32(&bars->drain));
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&bars->drain), 0)) {
          if (clock64() - t0 > 20000000LL) break;
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp - 4;  // == warp % 4: the TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.n_tiles;
      const int n_blk = tile - m_blk * p.n_tiles;
      if (!mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase, p.status, ST_TIMEOUT_TMEM_FULL,
                     acc)) {
        ok = false;
      }
      // all lanes of a warp must agree before the warp-wide tensor memory loads
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccCols;
      const int64_t row = static_cast<int64_t>(m_blk) * BM + quad * 32 + lane;
      if (MODE == 0) {
        // columns [0,64) gate, [64,128) up of hidden columns [n_blk*64, n_blk*64+64)
        uint32_t scale_pair = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t g[32], u[32];
          tc_ld_32x32b_x32(taddr + half * 32, g);
          tc_ld_32x32b_x32(taddr + 64 + half * 32, u);
          tc_wait_ld();
          float h[32];
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float gf = bf16_round(__uint_as_float(g[i]));
            const float uf = bf16_round(__uint_as_float(u[i]));
            const float gc = fminf(gf, p.limit);
            const float uc = fminf(fmaxf(uf, -p.limit), p.limit);
            const float s = __fdividef(gc, 1.0f + __expf(-gc));
            h[i] = bf16_round(s * uc);
            amax = fmaxf(amax, fabsf(h[i]));
          }
          const uint32_t e = e8m0_from_amax(amax);
          const float inv = e8m0_inverse(e);
          scale_pair |= e << (8 * half);
          uint4 q0, q1;
          q0.x = cvt_e4m3x4(h[0] * inv, h[1] * inv, h[2] * inv, h[3] * inv);
          q0.y = cvt_e4m3x4(h[4] * inv, h[5] * inv, h[6] * inv, h[7] * inv);
          q0.z = cvt_e4m3x4(h[8] * inv, h[9] * inv, h[10] * inv, h[11] * inv);
          q0.w = cvt_e4m3x4(h[12] * inv, h[13] * inv, h[14] * inv, h[15] * inv);
          q1.x = cvt_e4m3x4(h[16] * inv, h[17] * inv, h[18] * inv, h[19] * inv);
          q1.y = cvt_e4m3x4(h[20] * inv, h[21] * inv, h[22] * inv, h[23] * inv);
          q1.z = cvt_e4m3x4(h[24] * inv, h[25] * inv, h[26] * inv, h[27] * inv);
          q1.w = cvt_e4m3x4(h[28] * inv, h[29] * inv, h[30] * inv, h[31] * inv);
          uint4* dst = reinterpret_cast<uint4*>(p.out + row * p.out_cols + n_blk * 64 + half * 32);
          dst[0] = q0;
          dst[1] = q1;
        }
        // two adjacent scale bytes: 32-column groups (n_blk*2) and (n_blk*2 + 1)
        const size_t off = scale_offset(row, n_blk * 2, p.out_cols >> 7);
        *reinterpret_cast<uint16_t*>(p.out_sc + off) = static_cast<uint16_t>(scale_pair);
      } else {
        const int dest = p.dest_row[row];
        // combine push: the row goes to its home rank's buffer (plain stores over NVLink)
        uint8_t* out_base = p.out;
        if (p.out_peers != nullptr && dest >= 0) out_base = p.out_peers[p.peer_rank[row]];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tc_ld_32x32b_x32(taddr + c * 32, v);
          tc_wait_ld();
          if (dest >= 0) {
            uint4* dst = reinterpret_cast<uint4*>(
                out_base + (static_cast<size_t>(dest) * p.out_cols + n_blk * BN + c * 32) * 2);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              __nv_bfloat162 t;
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
              o.x = *reinterpret_cast<uint32_t*>(&t);
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
              o.y = *reinterpret_cast<uint32_t*>(&t);
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
              o.z = *reinterpret_cast<uint32_t*>(&t);
              t = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
              o.w = *reinterpret_cast<uint32_t*>(&t);
              dst[q] = o;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->acc_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

// [rows, K] u8 row-major, box = 128 rows x 128 bytes, 128-byte swizzle.
bool encode_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int grouped_gemm_smem_bytes() { return kSmemBytes; }

cudaError_t launch_grouped_gemm(const GroupedGemmArgs& a, cudaStream_t stream) {
  if (a.rows_capacity % BM || a.n_rows % BN || a.K % BK || a.K <= 0 || a.n_rows <= 0)
    return cudaErrorInvalidValue;
  if (a.rows_capacity == 0 || a.experts == 0) return cudaSuccess;
  CUtensorMap map_a, map_b;
  if (!encode_u8_2d(&map_a, a.a_fp8, static_cast<uint64_t>(a.rows_capacity), a.K) ||
      !encode_u8_2d(&map_b, a.b_fp8, static_cast<uint64_t>(a.experts) * a.n_rows, a.K))
    return cudaErrorInvalidValue;
  KernelParams p;
  p.a_sc = static_cast<const uint8_t*>(a.a_sc);
  p.b_sc = static_cast<const uint8_t*>(a.b_sc);
  p.block_expert = a.block_expert;
  p.num_rows_dev = a.num_rows_dev;
  p.max_m_blocks = static_cast<int>(a.rows_capacity / BM);
  p.k_steps = a.K / BK;
  p.n_tiles = a.n_rows / BN;
  p.out_cols = a.mode == 0 ? a.n_rows / 2 : a.n_rows;
  p.out = static_cast<uint8_t*>(a.out);
  p.out_sc = static_cast<uint8_t*>(a.out_sc);
  p.dest_row = a.dest_row;
  p.out_peers = reinterpret_cast<uint8_t* const*>(a.out_peers);
  p.peer_rank = a.peer_rank;
  p.status = a.status;
  p.limit = a.swiglu_limit > 0.0f ? a.swiglu_limit : HUGE_VALF;
  static bool attr_set[2] = {false, false};
  cudaError_t err;
  if (a.mode == 0) {
    if (!attr_set[0]) {
      err = cudaFuncSetAttribute(grouped_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemBytes);
      if (err != cudaSuccess) return err;
      attr_set[0] = true;
    }
    grouped_gemm_kernel<0><<<a.num_sms, kThreadsGemm, kSmemBytes, stream>>>(map_a, map_b, p);
  } else {
    if (!attr_set[1]) {
      err = cudaFuncSetAttribute(grouped_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemBytes);
      if (err != cudaSuccess) return err;
      attr_set[1] = true;
    }
    grouped_gemm_kernel<1><<<a.num_sms, kThreadsGemm, kSmemBytes, stream>>>(map_a, map_b, p);
  }
  return cudaGetLastError();
}

}  // namespace plb
