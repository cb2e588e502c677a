// HBM-bound stages of the MoE backward pass around the grouped GEMMs:
//   * d_y rows: d_y[p] = w[t, slot] * d_out[t] for every scheduled row (the backward of the
//     weighted combine, ops.bwd path of campaigns/mok/host/mok_port_host.py:207-219) and the
//     router-weight gradient d_w[t, slot] = <d_out[t], y[t, slot]>;
//   * SwiGLU backward (campaigns/mok/port/act_gptoss/swiglu.cuh:4-43,219-558, default variant
//     silu(g) * u): dequantise the saved MXFP8 gate / up, d_up = d_h * silu(g),
//     d_gate = d_h * u * sig(g) * (1 + g * (1 - sig(g))), written as bf16 [rows, 2I] = [d_gate | d_up];
//   * row gather of bf16 tokens into schedule order (the operand of the gate/up weight gradient).
// The quantisations these feed (both orientations) are plb_mxfp8_quantize calls on the host side.
#include "kernels.h"
#include "mxfp8.cuh"

namespace plb {

namespace {

__device__ __forceinline__ float lo16(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi16(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// One warp per scheduled row.
__global__ void __launch_bounds__(256)
bwd_dy_kernel(const uint4* __restrict__ d_out, const uint4* __restrict__ y, const float* __restrict__ router_w,
              const int* __restrict__ peer_rank, const int* __restrict__ peer_token_idx,
              const int* __restrict__ dest_row, const int* __restrict__ num_rows_dev, int64_t capacity,
              int hidden, int topk, uint4* __restrict__ dy, float* __restrict__ d_router_w) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int vecs = hidden >> 3;
  for (int64_t p = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    uint4* dst = dy + p * vecs;
    if (peer_rank[p] < 0) {
      for (int v = lane; v < vecs; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int64_t t = peer_token_idx[p];
    const int64_t d = dest_row[p];
    const float w = router_w[d];  // router weights are [tokens, topk] = indexed by token * topk + slot
    const uint4* src = d_out + t * vecs;
    const uint4* yr = y + d * vecs;
    float dot = 0.0f;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 g = src[v], yy = yr[v];
      const float gf[8] = {lo16(g.x), hi16(g.x), lo16(g.y), hi16(g.y), lo16(g.z), hi16(g.z), lo16(g.w), hi16(g.w)};
      const float yf[8] = {lo16(yy.x), hi16(yy.x), lo16(yy.y), hi16(yy.y), lo16(yy.z), hi16(yy.z), lo16(yy.w), hi16(yy.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) dot = fmaf(gf[i], yf[i], dot);
      uint4 o;
      o.x = pack2(__fmul_rn(w, gf[0]), __fmul_rn(w, gf[1]));
      o.y = pack2(__fmul_rn(w, gf[2]), __fmul_rn(w, gf[3]));
      o.z = pack2(__fmul_rn(w, gf[4]), __fmul_rn(w, gf[5]));
      o.w = pack2(__fmul_rn(w, gf[6]), __fmul_rn(w, gf[7]));
      dst[v] = o;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, s);
    if (lane == 0) d_router_w[d] = dot;
    (void)topk;
  }
}

// One thread per 8 consecutive intermediate columns of one row.
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ gate_sc,
                  const uint8_t* __restrict__ up, const uint8_t* __restrict__ up_sc,
                  const uint4* __restrict__ d_hidden, const int* __restrict__ num_rows_dev, int64_t capacity,
                  int inter, float limit, uint4* __restrict__ dgu) {
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int vecs = inter >> 3;
  const int64_t total = rows * vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t col_blocks = inter >> 7;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total; v += stride) {
    const int64_t r = v / vecs, j = v - r * vecs;
    const size_t so = scale_offset(r, j >> 2, col_blocks);
    const float gs = e8m0_value(gate_sc[so]), us = e8m0_value(up_sc[so]);
    const uint2 gq = *reinterpret_cast<const uint2*>(gate + r * inter + j * 8);
    const uint2 uq = *reinterpret_cast<const uint2*>(up + r * inter + j * 8);
    const uint4 dh = d_hidden[v];
    const float dhf[8] = {lo16(dh.x), hi16(dh.x), lo16(dh.y), hi16(dh.y), lo16(dh.z), hi16(dh.z), lo16(dh.w), hi16(dh.w)};
    float dg[8], du[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t gb = ((i < 4 ? gq.x : gq.y) >> (8 * (i & 3))) & 0xFFu;
      const uint32_t ub = ((i < 4 ? uq.x : uq.y) >> (8 * (i & 3))) & 0xFFu;
      const float g_raw = e4m3_to_float(gb) * gs, u_raw = e4m3_to_float(ub) * us;
      // clamped variant: the bounds of the forward pass, and no gradient through a bound that is
      // active or met with equality (swiglu.cuh:13-21); limit = +inf keeps every gradient
      const bool g_open = g_raw < limit, u_open = u_raw > -limit && u_raw < limit;
      const float g = fminf(g_raw, limit), u = fminf(fmaxf(u_raw, -limit), limit);
      const float sg = 1.0f / (1.0f + __expf(-g));
      du[i] = u_open ? dhf[i] * (g * sg) : 0.0f;
      dg[i] = g_open ? dhf[i] * u * sg * (1.0f + g * (1.0f - sg)) : 0.0f;
    }
    uint4 og, ou;
    og.x = pack2(dg[0], dg[1]); og.y = pack2(dg[2], dg[3]); og.z = pack2(dg[4], dg[5]); og.w = pack2(dg[6], dg[7]);
    ou.x = pack2(du[0], du[1]); ou.y = pack2(du[2], du[3]); ou.z = pack2(du[4], du[5]); ou.w = pack2(du[6], du[7]);
    dgu[r * (2 * vecs) + j] = og;
    dgu[r * (2 * vecs) + vecs + j] = ou;
  }
}

// Padding rows inside the schedule become zeros; rows beyond it are left alone (the transposed
// quantisation that follows stops at the rows in use).
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ peer_rank,
                   const int* __restrict__ peer_token_idx, const int* __restrict__ num_rows_dev,
                   int64_t capacity, int vecs, uint4* __restrict__ dst) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  for (int64_t p = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    const bool live = peer_rank[p] >= 0;
    const uint4* s = live ? src + static_cast<int64_t>(peer_token_idx[p]) * vecs : nullptr;
    for (int v = lane; v < vecs; v += 32) dst[p * vecs + v] = live ? s[v] : make_uint4(0u, 0u, 0u, 0u);
  }
}

// Expert-parallel forms of the two kernels above: the row's source rank picks the base pointer.
// d_y[p] = w_peers[r][dest_row[p]] * d_out_peers[r][token]; the router gradient is computed at
// the token's home rank instead (router_grad_kernel), where the combine rows already are.
__global__ void __launch_bounds__(256)
ep_bwd_dy_kernel(const uint4* const* __restrict__ d_out_peers, const float* const* __restrict__ router_w_peers,
                 const int* __restrict__ peer_rank, const int* __restrict__ peer_token_idx,
                 const int* __restrict__ dest_row, const int* __restrict__ num_rows_dev, int64_t capacity,
                 int hidden, uint4* __restrict__ dy) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int vecs = hidden >> 3;
  for (int64_t p = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    uint4* dst = dy + p * vecs;
    const int r = peer_rank[p];
    if (r < 0) {
      for (int v = lane; v < vecs; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float w = router_w_peers[r][dest_row[p]];
    const uint4* src = d_out_peers[r] + static_cast<int64_t>(peer_token_idx[p]) * vecs;
    for (int v0 = lane; v0 < vecs; v0 += 128) {   // four 16-byte loads in flight per lane
      uint4 g[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) g[u] = src[v0 + u * 32];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + u * 32 >= vecs) break;
        uint4 o;
        o.x = pack2(__fmul_rn(w, lo16(g[u].x)), __fmul_rn(w, hi16(g[u].x)));
        o.y = pack2(__fmul_rn(w, lo16(g[u].y)), __fmul_rn(w, hi16(g[u].y)));
        o.z = pack2(__fmul_rn(w, lo16(g[u].z)), __fmul_rn(w, hi16(g[u].z)));
        o.w = pack2(__fmul_rn(w, lo16(g[u].w)), __fmul_rn(w, hi16(g[u].w)));
        dst[v0 + u * 32] = o;
      }
    }
  }
}

// bf16 routed precision: the saved gate / up are bf16 rows, everything else as above.
__global__ void __launch_bounds__(256)
swiglu_bwd_bf16_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, const uint4* __restrict__ d_hidden,
                       const int* __restrict__ num_rows_dev, int64_t capacity, int inter, float limit,
                       uint4* __restrict__ dgu) {
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  const int vecs = inter >> 3;
  const int64_t total = rows * vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total; v += stride) {
    const int64_t r = v / vecs, j = v - r * vecs;
    const uint4 gq = gate[v], uq = up[v], dh = d_hidden[v];
    const float gf[8] = {lo16(gq.x), hi16(gq.x), lo16(gq.y), hi16(gq.y), lo16(gq.z), hi16(gq.z), lo16(gq.w), hi16(gq.w)};
    const float uf[8] = {lo16(uq.x), hi16(uq.x), lo16(uq.y), hi16(uq.y), lo16(uq.z), hi16(uq.z), lo16(uq.w), hi16(uq.w)};
    const float dhf[8] = {lo16(dh.x), hi16(dh.x), lo16(dh.y), hi16(dh.y), lo16(dh.z), hi16(dh.z), lo16(dh.w), hi16(dh.w)};
    float dg[8], du[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool g_open = gf[i] < limit, u_open = uf[i] > -limit && uf[i] < limit;
      const float g = fminf(gf[i], limit), u = fminf(fmaxf(uf[i], -limit), limit);
      const float sg = 1.0f / (1.0f + __expf(-g));
      du[i] = u_open ? dhf[i] * (g * sg) : 0.0f;
      dg[i] = g_open ? dhf[i] * u * sg * (1.0f + g * (1.0f - sg)) : 0.0f;
    }
    uint4 og, ou;
    og.x = pack2(dg[0], dg[1]); og.y = pack2(dg[2], dg[3]); og.z = pack2(dg[4], dg[5]); og.w = pack2(dg[6], dg[7]);
    ou.x = pack2(du[0], du[1]); ou.y = pack2(du[2], du[3]); ou.z = pack2(du[4], du[5]); ou.w = pack2(du[6], du[7]);
    dgu[r * (2 * vecs) + j] = og;
    dgu[r * (2 * vecs) + vecs + j] = ou;
  }
}

// out[c, r] = in[r, c] for a bf16 [rows, cols] tensor (both multiples of 64): 64 x 64 tiles through
// shared memory, 128-byte segments on both sides. The bf16 weight-gradient GEMMs contract over the
// schedule rows, so their operands are the transposes of the row-major activations.
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, int64_t rows, int64_t cols, const int* __restrict__ live_rows_dev,
                      __nv_bfloat16* __restrict__ out) {
  __shared__ __nv_bfloat16 tile[64][66];
  // a routed buffer is sized for the worst case: only the 64-row tiles in use are moved (`rows` stays
  // the leading dimension of the transpose)
  int64_t row_tiles = rows >> 6;
  if (live_rows_dev != nullptr) {
    const int64_t live = (static_cast<int64_t>(*live_rows_dev) + 63) >> 6;
    if (live < row_tiles) row_tiles = live < 0 ? 0 : live;
  }
  const int64_t tiles_c = cols >> 6, total = row_tiles * tiles_c;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t r0 = (t / tiles_c) << 6, c0 = (t % tiles_c) << 6;
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {       // 32 pairs per row
      const int r = i >> 5, c2 = (i & 31) << 1;
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(in + (r0 + r) * cols + c0 + c2);
      tile[r][c2] = v.x;
      tile[r][c2 + 1] = v.y;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int c = i >> 5, r2 = (i & 31) << 1;
      __nv_bfloat162 v;
      v.x = tile[r2][c];
      v.y = tile[r2 + 1][c];
      *reinterpret_cast<__nv_bfloat162*>(out + (c0 + c) * rows + r0 + r2) = v;
    }
    __syncthreads();
  }
}

// d_router_w[t * topk + j] = <d_out[t], combine[t * topk + j]>: one warp per (token, slot), the
// same lane partition, fma order and shuffle tree as bwd_dy_kernel, so both give the same bits.
__global__ void __launch_bounds__(256)
router_grad_kernel(const uint4* __restrict__ d_out, const uint4* __restrict__ y, const int* __restrict__ row_index,
                   int64_t tokens, int topk, int hidden, float* __restrict__ d_router_w) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int vecs = hidden >> 3;
  for (int64_t d = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; d < tokens * topk; d += warps) {
    const uint4* src = d_out + (d / topk) * vecs;
    // row_index: where the (token, slot) row sits when the combine rows were pushed into receive streams
    const uint4* yr = y + (row_index != nullptr ? static_cast<int64_t>(row_index[d]) : d) * vecs;
    float dot = 0.0f;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 g = src[v], yy = yr[v];
      const float gf[8] = {lo16(g.x), hi16(g.x), lo16(g.y), hi16(g.y), lo16(g.z), hi16(g.z), lo16(g.w), hi16(g.w)};
      const float yf[8] = {lo16(yy.x), hi16(yy.x), lo16(yy.y), hi16(yy.y), lo16(yy.z), hi16(yy.z), lo16(yy.w), hi16(yy.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) dot = fmaf(gf[i], yf[i], dot);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, s);
    if (lane == 0) d_router_w[d] = dot;
  }
}

__global__ void __launch_bounds__(256)
ep_gather_rows_kernel(const uint4* const* __restrict__ src_peers, const int* __restrict__ peer_rank,
                      const int* __restrict__ peer_token_idx, const int* __restrict__ num_rows_dev,
                      int64_t capacity, int vecs, uint4* __restrict__ dst) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  int64_t rows = *num_rows_dev;
  if (rows > capacity) rows = capacity;
  for (int64_t p = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    const int r = peer_rank[p];
    const uint4* s = r >= 0 ? src_peers[r] + static_cast<int64_t>(peer_token_idx[p]) * vecs : nullptr;
    for (int v0 = lane; v0 < vecs; v0 += 128) {
      uint4 g[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) g[u] = (r >= 0 && v0 + u * 32 < vecs) ? s[v0 + u * 32] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) dst[p * vecs + v0 + u * 32] = g[u];
    }
  }
}

int sm_grid(int mult) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * mult;
}

}  // namespace

cudaError_t launch_bwd_dy(const void* d_out, const void* y, const float* router_w, const int* peer_rank,
                          const int* peer_token_idx, const int* dest_row, const int* num_rows_dev,
                          int64_t capacity, int hidden, int topk, void* dy, float* d_router_w,
                          cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  bwd_dy_kernel<<<sm_grid(8), 256, 0, stream>>>(static_cast<const uint4*>(d_out), static_cast<const uint4*>(y),
                                                router_w, peer_rank, peer_token_idx, dest_row, num_rows_dev,
                                                capacity, hidden, topk, static_cast<uint4*>(dy), d_router_w);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* gate, const void* gate_sc, const void* up, const void* up_sc,
                              const void* d_hidden, const int* num_rows_dev, int64_t capacity, int inter,
                              float limit, void* dgu, cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  const float bound = limit > 0.0f ? limit : HUGE_VALF;
  swiglu_bwd_kernel<<<sm_grid(8), 256, 0, stream>>>(
      static_cast<const uint8_t*>(gate), static_cast<const uint8_t*>(gate_sc), static_cast<const uint8_t*>(up),
      static_cast<const uint8_t*>(up_sc), static_cast<const uint4*>(d_hidden), num_rows_dev, capacity, inter,
      bound, static_cast<uint4*>(dgu));
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* src, const int* peer_rank, const int* peer_token_idx,
                               const int* num_rows_dev, int64_t capacity, int cols, void* dst,
                               cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  gather_rows_kernel<<<sm_grid(8), 256, 0, stream>>>(static_cast<const uint4*>(src), peer_rank, peer_token_idx,
                                                     num_rows_dev, capacity, cols >> 3, static_cast<uint4*>(dst));
  return cudaGetLastError();
}

cudaError_t launch_ep_bwd_dy(const void* const* d_out_peers, const float* const* router_w_peers, const int* peer_rank,
                             const int* peer_token_idx, const int* dest_row, const int* num_rows_dev, int64_t capacity,
                             int hidden, void* dy, cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  ep_bwd_dy_kernel<<<sm_grid(8), 256, 0, stream>>>(reinterpret_cast<const uint4* const*>(d_out_peers), router_w_peers,
                                                   peer_rank, peer_token_idx, dest_row, num_rows_dev, capacity, hidden,
                                                   static_cast<uint4*>(dy));
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd_bf16(const void* gate, const void* up, const void* d_hidden, const int* num_rows_dev,
                                   int64_t capacity, int inter, float limit, void* dgu, cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  swiglu_bwd_bf16_kernel<<<sm_grid(8), 256, 0, stream>>>(static_cast<const uint4*>(gate), static_cast<const uint4*>(up),
                                                         static_cast<const uint4*>(d_hidden), num_rows_dev, capacity, inter,
                                                         limit > 0.0f ? limit : HUGE_VALF, static_cast<uint4*>(dgu));
  return cudaGetLastError();
}

cudaError_t launch_transpose_bf16(const void* in, int64_t rows, int64_t cols, const int* live_rows_dev, void* out,
                                  cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  transpose_bf16_kernel<<<sm_grid(8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), rows, cols, live_rows_dev,
                                                        static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError();
}

cudaError_t launch_router_grad(const void* d_out, const void* combine, int64_t tokens, int topk, int hidden,
                               float* d_router_w, cudaStream_t stream, const int* row_index) {
  if (tokens == 0) return cudaSuccess;
  router_grad_kernel<<<sm_grid(8), 256, 0, stream>>>(static_cast<const uint4*>(d_out), static_cast<const uint4*>(combine),
                                                     row_index, tokens, topk, hidden, d_router_w);
  return cudaGetLastError();
}

cudaError_t launch_ep_gather_rows(const void* const* src_peers, const int* peer_rank, const int* peer_token_idx,
                                  const int* num_rows_dev, int64_t capacity, int cols, void* dst, cudaStream_t stream) {
  if (capacity == 0) return cudaSuccess;
  ep_gather_rows_kernel<<<sm_grid(8), 256, 0, stream>>>(reinterpret_cast<const uint4* const*>(src_peers), peer_rank,
                                                        peer_token_idx, num_rows_dev, capacity, cols >> 3,
                                                        static_cast<uint4*>(dst));
  return cudaGetLastError();
}

}  // namespace plb
