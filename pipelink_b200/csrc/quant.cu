// HBM-bound byte/element kernels either side of the grouped GEMM:
//   * MXFP8 quantisation of bf16 rows, optionally gathered through the routing
//     schedule from peer-addressable token buffers (the dispatch stage,
//     campaigns/mok/port/comm/comm.cu:105-123: x_routed[p] = quant(x_buffer[peer_rank[p]][peer_token_idx[p]])),
//   * the transposed orientation (scales along the original row dimension) that the
//     backward GEMMs contract over (campaigns/mok/host/resources.py:62-77),
//   * dequantisation (checker use), gate/up weight interleave, and the weighted
//     top-k reduction  out = y_shared + sum_j w[t,j] * combine[t*k+j]
//     (ops.fwd_epilogue, campaigns/mok/host/mok_port_host.py:204).
// All are sized as grid-stride loops over 16-byte vectors with a grid that is a
// multiple of the SM count.
#include "kernels.h"
#include "mxfp8.cuh"

namespace plb {

namespace {

constexpr int kThreads = 256;


// One thread owns 8 consecutive elements; 4 adjacent lanes own one 32-element block.
template <bool GATHER>
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const void* const* __restrict__ src_peers, const uint4* __restrict__ src_plain,
                     const int* __restrict__ peer_rank, const int* __restrict__ peer_token_idx,
                     const int* __restrict__ num_rows_dev, int64_t rows, int64_t cols,
                     uint2* __restrict__ dst_fp8, uint8_t* __restrict__ dst_sc) {
  const int64_t vec_per_row = cols >> 3;
  int64_t nrows = rows;
  if (num_rows_dev != nullptr) {
    const int64_t live = *num_rows_dev;
    nrows = live < rows ? live : rows;
  }
  const int64_t total = nrows * vec_per_row;               // multiple of 16
  const int64_t total_warp = (total + 31) & ~int64_t(31);  // keep whole warps in the loop
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t col_blocks = cols >> 7;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total_warp;
       v += stride) {
    const bool active = v < total;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    int64_t row = 0, j = 0;
    if (active) {
      row = v / vec_per_row;
      j = v - row * vec_per_row;
      if (GATHER) {
        const int pr = peer_rank[row];
        if (pr >= 0) {
          const uint4* base = static_cast<const uint4*>(src_peers[pr]);
          raw = base[static_cast<int64_t>(peer_token_idx[row]) * vec_per_row + j];
        }
      } else {
        raw = src_plain[v];
      }
    }
    float f[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                  bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const uint32_t e = e8m0_from_amax(amax);
    const float inv = e8m0_inverse(e);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t base_lane = lane & ~15u;
    uint32_t word = __shfl_sync(0xFFFFFFFFu, e, base_lane);
    word |= __shfl_sync(0xFFFFFFFFu, e, base_lane + 4) << 8;
    word |= __shfl_sync(0xFFFFFFFFu, e, base_lane + 8) << 16;
    word |= __shfl_sync(0xFFFFFFFFu, e, base_lane + 12) << 24;
    if (active) {
      uint2 out;
      out.x = cvt_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
      out.y = cvt_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
      dst_fp8[v] = out;
      if ((lane & 15u) == 0u) {
        const size_t off = scale_offset(row, j >> 2, col_blocks);
        *reinterpret_cast<uint32_t*>(dst_sc + off) = word;
      }
    }
  }
}

// Transposed orientation: dst_t[c, r] = quant(src[r, c]) with blocks of 32 along r.
// One thread owns two adjacent source columns and one 32-row block.
__global__ void __launch_bounds__(kThreads)
quantize_transposed_kernel(const uint32_t* __restrict__ src, int64_t rows, int64_t cols,
                           uint8_t* __restrict__ dst_fp8, uint8_t* __restrict__ dst_sc) {
  const int64_t col_pairs = cols >> 1;
  const int64_t row_blocks = rows >> 5;
  const int64_t total = col_pairs * row_blocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t dst_col_blocks = rows >> 7;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += stride) {
    const int64_t rb = v / col_pairs;
    const int64_t cp = v - rb * col_pairs;
    float lo[32], hi[32];
    float amax_lo = 0.0f, amax_hi = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t w = src[(rb * 32 + i) * col_pairs + cp];
      lo[i] = bf16_lo(w);
      hi[i] = bf16_hi(w);
      amax_lo = fmaxf(amax_lo, fabsf(lo[i]));
      amax_hi = fmaxf(amax_hi, fabsf(hi[i]));
    }
    const uint32_t e_lo = e8m0_from_amax(amax_lo), e_hi = e8m0_from_amax(amax_hi);
    const float inv_lo = e8m0_inverse(e_lo), inv_hi = e8m0_inverse(e_hi);
    uint4* out_lo = reinterpret_cast<uint4*>(dst_fp8 + (2 * cp) * rows + rb * 32);
    uint4* out_hi = reinterpret_cast<uint4*>(dst_fp8 + (2 * cp + 1) * rows + rb * 32);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint4 a, b;
      a.x = cvt_e4m3x4(lo[q * 16 + 0] * inv_lo, lo[q * 16 + 1] * inv_lo, lo[q * 16 + 2] * inv_lo, lo[q * 16 + 3] * inv_lo);
      a.y = cvt_e4m3x4(lo[q * 16 + 4] * inv_lo, lo[q * 16 + 5] * inv_lo, lo[q * 16 + 6] * inv_lo, lo[q * 16 + 7] * inv_lo);
      a.z = cvt_e4m3x4(lo[q * 16 + 8] * inv_lo, lo[q * 16 + 9] * inv_lo, lo[q * 16 + 10] * inv_lo, lo[q * 16 + 11] * inv_lo);
      a.w = cvt_e4m3x4(lo[q * 16 + 12] * inv_lo, lo[q * 16 + 13] * inv_lo, lo[q * 16 + 14] * inv_lo, lo[q * 16 + 15] * inv_lo);
      b.x = cvt_e4m3x4(hi[q * 16 + 0] * inv_hi, hi[q * 16 + 1] * inv_hi, hi[q * 16 + 2] * inv_hi, hi[q * 16 + 3] * inv_hi);
      b.y = cvt_e4m3x4(hi[q * 16 + 4] * inv_hi, hi[q * 16 + 5] * inv_hi, hi[q * 16 + 6] * inv_hi, hi[q * 16 + 7] * inv_hi);
      b.z = cvt_e4m3x4(hi[q * 16 + 8] * inv_hi, hi[q * 16 + 9] * inv_hi, hi[q * 16 + 10] * inv_hi, hi[q * 16 + 11] * inv_hi);
      b.w = cvt_e4m3x4(hi[q * 16 + 12] * inv_hi, hi[q * 16 + 13] * inv_hi, hi[q * 16 + 14] * inv_hi, hi[q * 16 + 15] * inv_hi);
      out_lo[q] = a;
      out_hi[q] = b;
    }
    dst_sc[scale_offset(2 * cp, rb, dst_col_blocks)] = static_cast<uint8_t>(e_lo);
    dst_sc[scale_offset(2 * cp + 1, rb, dst_col_blocks)] = static_cast<uint8_t>(e_hi);
  }
}

// One pass over the input for both orientations: a CTA stages a 128 x 128 bf16 tile in shared
// memory (coalesced 16-byte loads), then quantises it along the columns (row orientation: 32
// consecutive columns per block, four threads of a warp finish 128 contiguous output bytes of a
// row) and along the rows (transposed orientation: 32 consecutive rows per block, the four row
// blocks of a column are written by the same CTA so L2 sees whole 128-byte lines). Either output
// may be absent. Same arithmetic as the two kernels above, so the same bytes.
constexpr int kTile = 128;
constexpr int kTilePitch = kTile * 2 + 16;   // bytes per staged row; the pad keeps 16-byte alignment

__device__ __forceinline__ float bf16_at(const uint8_t* row, int col) {
  return __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(row + col * 2)) << 16);
}

__global__ void __launch_bounds__(kThreads)
quantize_tile_kernel(const uint4* __restrict__ src, int64_t rows, int64_t cols, const int* __restrict__ live_rows_dev,
                     uint8_t* __restrict__ dst_fp8, uint8_t* __restrict__ dst_sc, uint8_t* __restrict__ dst_t_fp8,
                     uint8_t* __restrict__ dst_t_sc) {
  extern __shared__ __align__(16) uint8_t tile[];
  const int64_t col_tiles = cols >> 7, row_tiles = rows >> 7;
  // a routed buffer is sized for the worst case; only the row tiles in use are read and written
  // (the tensors keep the full `rows` as their leading dimension)
  int64_t row_tiles_live = row_tiles;
  if (live_rows_dev != nullptr) {
    const int64_t live = (static_cast<int64_t>(*live_rows_dev) + kTile - 1) >> 7;
    if (live < row_tiles_live) row_tiles_live = live < 0 ? 0 : live;
  }
  for (int64_t tid = blockIdx.x; tid < row_tiles_live * col_tiles; tid += gridDim.x) {
    const int64_t tr = tid / col_tiles, tc = tid - tr * col_tiles;
    const int64_t r0 = tr * kTile, c0 = tc * kTile;
    // stage: 16 threads per row, 16 rows per pass
    for (int i = threadIdx.x; i < kTile * 16; i += kThreads) {
      const int r = i >> 4, v = i & 15;
      *reinterpret_cast<uint4*>(tile + r * kTilePitch + v * 16) = src[((r0 + r) * cols + c0) / 8 + v];
    }
    __syncthreads();
    if (dst_fp8 != nullptr) {
      for (int i = threadIdx.x; i < kTile * 4; i += kThreads) {
        const int r = i >> 2, blk = i & 3;   // a warp covers 8 rows x 4 blocks
        const uint8_t* row = tile + r * kTilePitch + blk * 64;
        float x[32];
        float amax = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 w = *reinterpret_cast<const uint4*>(row + q * 16);
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            x[q * 8 + e * 2] = bf16_lo(ws[e]);
            x[q * 8 + e * 2 + 1] = bf16_hi(ws[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(x[e]));
        const uint32_t eb = e8m0_from_amax(amax);
        const float inv = e8m0_inverse(eb);
        uint4 o[2];
        uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          ow[q] = cvt_e4m3x4(x[q * 4] * inv, x[q * 4 + 1] * inv, x[q * 4 + 2] * inv, x[q * 4 + 3] * inv);
        uint4* out = reinterpret_cast<uint4*>(dst_fp8 + (r0 + r) * cols + c0 + blk * 32);
        out[0] = o[0];
        out[1] = o[1];
        dst_sc[scale_offset(r0 + r, (c0 >> 5) + blk, col_tiles)] = static_cast<uint8_t>(eb);
      }
    }
    if (dst_t_fp8 != nullptr) {
      for (int i = threadIdx.x; i < kTile * 4; i += kThreads) {
        const int col = i & 127, rb = i >> 7;   // a warp covers 32 consecutive columns of one row block
        const uint8_t* base = tile + (rb * 32) * kTilePitch;
        float x[32];
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          x[e] = bf16_at(base + e * kTilePitch, col);
          amax = fmaxf(amax, fabsf(x[e]));
        }
        const uint32_t eb = e8m0_from_amax(amax);
        const float inv = e8m0_inverse(eb);
        uint4 o[2];
        uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          ow[q] = cvt_e4m3x4(x[q * 4] * inv, x[q * 4 + 1] * inv, x[q * 4 + 2] * inv, x[q * 4 + 3] * inv);
        uint4* out = reinterpret_cast<uint4*>(dst_t_fp8 + (c0 + col) * rows + r0 + rb * 32);
        out[0] = o[0];
        out[1] = o[1];
        dst_t_sc[scale_offset(c0 + col, (r0 >> 5) + rb, row_tiles)] = static_cast<uint8_t>(eb);
      }
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
dequantize_kernel(const uint8_t* __restrict__ src, const uint8_t* __restrict__ sc, int64_t rows,
                  int64_t cols, float* __restrict__ dst) {
  const int64_t total = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t col_blocks = cols >> 7;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t r = i / cols, c = i - r * cols;
    const uint32_t s = sc[scale_offset(r, c >> 5, col_blocks)];
    dst[i] = e4m3_to_float(src[i]) * e8m0_value(s);
  }
}

// w13 row order per expert, for interleave block B (64 or 128):
// [gate 0..B-1 | up 0..B-1 | gate B..2B-1 | up B..2B-1 | ...] so that one 2B-row weight
// tile yields B gate and B up columns of the same hidden index range and its scale
// blocks are ordinary 512-byte blocks.
__global__ void __launch_bounds__(kThreads)
pack_gate_up_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ gate_sc,
                    const uint8_t* __restrict__ up, const uint8_t* __restrict__ up_sc, int experts,
                    int inter, int hidden, int block, uint8_t* __restrict__ w13,
                    uint8_t* __restrict__ w13_sc) {
  const int64_t vec_per_row = hidden >> 4;  // 16-byte vectors
  const int64_t dst_rows = static_cast<int64_t>(experts) * 2 * inter;
  const int64_t total = dst_rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t col_blocks = hidden >> 7;
  const int64_t groups = hidden >> 5;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += stride) {
    const int64_t dr = v / vec_per_row, j = v - dr * vec_per_row;
    const int64_t e = dr / (2 * inter), within = dr - e * 2 * inter;
    const int64_t tile = within / (2 * block), r = within - tile * 2 * block;
    const bool is_up = r >= block;
    const int64_t sr = e * inter + tile * block + (is_up ? r - block : r);
    const uint8_t* src = is_up ? up : gate;
    reinterpret_cast<uint4*>(w13)[v] = reinterpret_cast<const uint4*>(src)[sr * vec_per_row + j];
    // this thread also moves the scale bytes of the 32-column groups it starts
    if ((j & 1) == 0) {
      const int64_t g = j >> 1;
      if (g < groups) {
        const uint8_t* ssrc = is_up ? up_sc : gate_sc;
        w13_sc[scale_offset(dr, g, col_blocks)] = ssrc[scale_offset(sr, g, col_blocks)];
      }
    }
  }
}

// out[t, c] = bf16( (y_shared ? y_shared[t,c] : 0) + sum_{j<k} w[t,j] * combine[t*k+j, c] )
// (`index` non-null: the row of slot t*k+j is combine[index[t*k+j]], rows received in arrival order)
// with every multiply and add rounded separately in fp32 and j ascending, so the
// result is a pure function of its inputs (deterministic combine order).
template <int TOPK>  // 0 = runtime top-k; otherwise the loads of all slots are issued together
__global__ void __launch_bounds__(kThreads)
weighted_combine_kernel(const uint4* __restrict__ combine, const float* __restrict__ w,
                        const uint4* __restrict__ y_shared, int64_t tokens, int topk_rt,
                        int64_t hidden, uint4* __restrict__ out, const int* __restrict__ index) {
  const int topk = TOPK > 0 ? TOPK : topk_rt;
  const int64_t vec_per_row = hidden >> 3;
  const int64_t total = tokens * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += stride) {
    const int64_t t = v / vec_per_row, j = v - t * vec_per_row;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (y_shared != nullptr) {
      const uint4 y = y_shared[v];
      acc[0] = bf16_lo(y.x); acc[1] = bf16_hi(y.x); acc[2] = bf16_lo(y.y); acc[3] = bf16_hi(y.y);
      acc[4] = bf16_lo(y.z); acc[5] = bf16_hi(y.z); acc[6] = bf16_lo(y.w); acc[7] = bf16_hi(y.w);
    }
    if (TOPK > 0) {
      uint4 c[TOPK > 0 ? TOPK : 1];
      float ws[TOPK > 0 ? TOPK : 1];
#pragma unroll
      for (int s = 0; s < TOPK; ++s) {
        ws[s] = w[t * TOPK + s];
        c[s] = combine[static_cast<int64_t>(index != nullptr ? index[t * TOPK + s] : t * TOPK + s) * vec_per_row + j];
      }
#pragma unroll
      for (int s = 0; s < TOPK; ++s) {
        const float f[8] = {bf16_lo(c[s].x), bf16_hi(c[s].x), bf16_lo(c[s].y), bf16_hi(c[s].y),
                            bf16_lo(c[s].z), bf16_hi(c[s].z), bf16_lo(c[s].w), bf16_hi(c[s].w)};
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(ws[s], f[i]));
      }
    } else
    for (int s = 0; s < topk; ++s) {
      const float ws = w[t * topk + s];
      const uint4 c = combine[static_cast<int64_t>(index != nullptr ? index[t * topk + s] : t * topk + s) * vec_per_row + j];
      const float f[8] = {bf16_lo(c.x), bf16_hi(c.x), bf16_lo(c.y), bf16_hi(c.y),
                          bf16_lo(c.z), bf16_hi(c.z), bf16_lo(c.w), bf16_hi(c.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(ws, f[i]));
    }
    uint4 o;
    __nv_bfloat162 p;
    p = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&p);
    p = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&p);
    p = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&p);
    p = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&p);
    out[v] = o;
  }
}

int grid_for(int64_t work_items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  int64_t g = want < cap ? want : cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

cudaError_t launch_quantize_rows(const void* const* src_peers, const int* peer_rank,
                                 const int* peer_token_idx, const int* num_rows_dev, int64_t rows,
                                 int64_t cols, void* dst_fp8, void* dst_sc, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  quantize_rows_kernel<true><<<grid_for(rows * (cols >> 3)), kThreads, 0, stream>>>(
      src_peers, nullptr, peer_rank, peer_token_idx, num_rows_dev, rows, cols,
      static_cast<uint2*>(dst_fp8), static_cast<uint8_t*>(dst_sc));
  return cudaGetLastError();
}

cudaError_t launch_quantize_plain(const void* src_bf16, int64_t rows, int64_t cols, void* dst_fp8,
                                  void* dst_sc, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  quantize_rows_kernel<false><<<grid_for(rows * (cols >> 3)), kThreads, 0, stream>>>(
      nullptr, static_cast<const uint4*>(src_bf16), nullptr, nullptr, nullptr, rows, cols,
      static_cast<uint2*>(dst_fp8), static_cast<uint8_t*>(dst_sc));
  return cudaGetLastError();
}

cudaError_t launch_quantize_transposed(const void* src_bf16, int64_t rows, int64_t cols,
                                       void* dst_t_fp8, void* dst_t_sc, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  quantize_transposed_kernel<<<grid_for((rows >> 5) * (cols >> 1)), kThreads, 0, stream>>>(
      static_cast<const uint32_t*>(src_bf16), rows, cols, static_cast<uint8_t*>(dst_t_fp8),
      static_cast<uint8_t*>(dst_t_sc));
  return cudaGetLastError();
}

cudaError_t launch_quantize_tile(const void* src_bf16, int64_t rows, int64_t cols, const int* live_rows_dev, void* dst_fp8,
                                 void* dst_sc, void* dst_t_fp8, void* dst_t_sc, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const int smem = kTile * kTilePitch;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(quantize_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    configured = true;
  }
  const int64_t tiles = (rows >> 7) * (cols >> 7);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t resident = static_cast<int64_t>(sms > 0 ? sms : 148) * 6;   // 34 KB of shared memory per CTA
  quantize_tile_kernel<<<static_cast<unsigned>(tiles < resident ? tiles : resident), kThreads, smem, stream>>>(
      static_cast<const uint4*>(src_bf16), rows, cols, live_rows_dev, static_cast<uint8_t*>(dst_fp8),
      static_cast<uint8_t*>(dst_sc), static_cast<uint8_t*>(dst_t_fp8), static_cast<uint8_t*>(dst_t_sc));
  return cudaGetLastError();
}

cudaError_t launch_dequantize(const void* src_fp8, const void* src_sc, int64_t rows, int64_t cols,
                              float* dst, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  dequantize_kernel<<<grid_for(rows * cols), kThreads, 0, stream>>>(
      static_cast<const uint8_t*>(src_fp8), static_cast<const uint8_t*>(src_sc), rows, cols, dst);
  return cudaGetLastError();
}

cudaError_t launch_pack_gate_up(const void* gate_fp8, const void* gate_sc, const void* up_fp8,
                                const void* up_sc, int experts, int inter, int hidden, int block,
                                void* w13_fp8, void* w13_sc, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(experts) * 2 * inter * (hidden >> 4);
  pack_gate_up_kernel<<<grid_for(total), kThreads, 0, stream>>>(
      static_cast<const uint8_t*>(gate_fp8), static_cast<const uint8_t*>(gate_sc),
      static_cast<const uint8_t*>(up_fp8), static_cast<const uint8_t*>(up_sc), experts, inter,
      hidden, block, static_cast<uint8_t*>(w13_fp8), static_cast<uint8_t*>(w13_sc));
  return cudaGetLastError();
}

cudaError_t launch_weighted_combine(const void* combine_bf16, const float* router_weights,
                                    const void* y_shared_bf16, int64_t tokens, int topk,
                                    int64_t hidden, void* out_bf16, cudaStream_t stream, const int* index) {
  if (tokens == 0) return cudaSuccess;
  const int grid = grid_for(tokens * (hidden >> 3));
  const uint4* c = static_cast<const uint4*>(combine_bf16);
  const uint4* y = static_cast<const uint4*>(y_shared_bf16);
  uint4* o = static_cast<uint4*>(out_bf16);
#define PLB_COMBINE(K) \
  weighted_combine_kernel<K><<<grid, kThreads, 0, stream>>>(c, router_weights, y, tokens, topk, hidden, o, index)
  switch (topk) {
    case 1: PLB_COMBINE(1); break;
    case 2: PLB_COMBINE(2); break;
    case 4: PLB_COMBINE(4); break;
    case 6: PLB_COMBINE(6); break;
    case 8: PLB_COMBINE(8); break;
    default: PLB_COMBINE(0); break;
  }
#undef PLB_COMBINE
  return cudaGetLastError();
}

}  // namespace plb
