// Batch-1 Llama-shaped decode as one persistent interpreter kernel (sm_100a).
//
// Stands in for the reference's decode megakernel: a per-SM instruction stream
// (instructions [num_sms, n, 32] i32, campaigns/megakernel/host/mk_host_abi.h:37), the
// opcodes of campaigns/megakernel/host/export_inputs.py:49-58
//   1 RMSNorm + QKV matvec + interleaved RoPE + KV append     4 O projection + residual
//   2 partial attention (4 query heads of one KV head)        5 RMSNorm + gate/up + SiLU*up
//   3 attention reduction (LSE-weighted merge of partials)    6 down projection + residual
//   7 RMSNorm + LM head
// plus 8 (greedy sample: argmax, next embedding row, position + 1) so a decode loop needs
// no host round trip, and cross-SM ordering through global counters that a consumer polls
// and a producer bumps after a fence (port/src/ops/attn_partial_cute.cu:66-80,129-136).
// The arithmetic of ops 1 and 3-7 is in the reference's absent Megakernels submodule
// (port/src/mono.cu:14-20); this file implements the published Llama math directly.
// Op 2 follows the contract of port/src/ops/cute_attention.cuh:70-225: scores in the
// base-2 domain, online max/sum, normalised fp32 partial output, LSE2 = max + log2(sum),
// 16-token KV blocks split as blocks_per_partition = ceil(ceil(len/16)/partitions).
//
// Decode at batch 1 streams 2.47 GB of weights per token and does ~2 FLOP per byte, so
// every op is an HBM-bound matvec: one warp per pair of weight rows, 16-byte
// non-allocating loads, eight in flight per lane (64 KB per SM), fp32 accumulation,
// activations staged once per instruction in shared memory. While an instruction waits
// for its producers it prefetches its weight rows into L2.
//
// Every wait is bounded (cycle budget -> status record, all other waits give up).
#include "kernels.h"
#include "decode.h"

namespace plb {

namespace {

constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kHidden = 2048;
constexpr int kHeadDim = 64;
constexpr int kQHeads = 32;
constexpr int kKvHeads = 8;
constexpr int kFfn = 8192;
constexpr int kQkvRows = (kQHeads + 2 * kKvHeads) * kHeadDim;  // 3072

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Coherent read of a bf16 another SM may have written earlier in this launch.
__device__ __forceinline__ float ld_bf16_coherent(const __nv_bfloat16* p) {
  unsigned short raw;
  asm volatile("ld.volatile.global.u16 %0, [%1];" : "=h"(raw) : "l"(p) : "memory");
  return __uint_as_float(static_cast<uint32_t>(raw) << 16);
}
__device__ __forceinline__ float blo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bhi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
  return v;
}

__device__ __forceinline__ float dot8(uint4 w, const float* x) {
  const float4 a = *reinterpret_cast<const float4*>(x);
  const float4 b = *reinterpret_cast<const float4*>(x + 4);
  float s = blo(w.x) * a.x;
  s = fmaf(bhi(w.x), a.y, s);
  s = fmaf(blo(w.y), a.z, s);
  s = fmaf(bhi(w.y), a.w, s);
  s = fmaf(blo(w.z), b.x, s);
  s = fmaf(bhi(w.z), b.y, s);
  s = fmaf(blo(w.w), b.z, s);
  s = fmaf(bhi(w.w), b.w, s);
  return s;
}

// Two weight rows (each `chunks` 16-byte vectors) against the staged fp32 vector.
// chunks is a multiple of 128 (2048 or 8192 columns).
__device__ __forceinline__ void warp_dot2(const uint4* __restrict__ row_a,
                                          const uint4* __restrict__ row_b,
                                          const float* __restrict__ x, int chunks, int lane,
                                          float& sum_a, float& sum_b) {
  float sa = 0.0f, sb = 0.0f;
  for (int c0 = 0; c0 < chunks; c0 += 128) {
    uint4 wa[4], wb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      wa[u] = ldg_stream(row_a + c0 + u * 32 + lane);
      wb[u] = ldg_stream(row_b + c0 + u * 32 + lane);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float* xs = x + (c0 + u * 32 + lane) * 8;
      sa += dot8(wa[u], xs);
      sb += dot8(wb[u], xs);
    }
  }
  sum_a = warp_sum(sa);
  sum_b = warp_sum(sb);
}

// Stage a bf16 vector of n elements into shared fp32; optionally RMS-normalise with weight.
__device__ void stage_vector(const __nv_bfloat16* __restrict__ src,
                             const __nv_bfloat16* __restrict__ norm_w, int n, float eps,
                             float* x, float* red) {
  float ss = 0.0f;
  // coherent 16-byte loads: these activations were written by other SMs in this launch
  for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
    uint4 raw;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                 : "l"(src + i)
                 : "memory");
    const float f[8] = {blo(raw.x), bhi(raw.x), blo(raw.y), bhi(raw.y),
                        blo(raw.z), bhi(raw.z), blo(raw.w), bhi(raw.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      x[i + j] = f[j];
      ss += f[j] * f[j];
    }
  }
  if (norm_w == nullptr) {
    __syncthreads();
    return;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) total += red[w];
  const float inv = rsqrtf(total / static_cast<float>(n) + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] = x[i] * inv * __bfloat162float(norm_w[i]);
  __syncthreads();
}

// Bounded wait until counter >= target. Returns false after recording a failure.
__device__ bool wait_counter(const unsigned* counter, unsigned target, Status* st, int what) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      if (ld_acquire_gpu(counter) >= target) break;
      if ((it & 63u) == 63u) {
        if (ld_volatile_i32(&st->code) != 0) { ok = 0; break; }
        if (clock64() - t0 > kWaitBudgetCycles) {
          report_failure(st, ST_TIMEOUT_COUNTER, what, ld_acquire_gpu(counter), target);
          ok = 0;
          break;
        }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  const bool ok = ok_flag != 0;
  __syncthreads();
  return ok;
}

__device__ __forceinline__ void signal_counter(unsigned* counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}

// ---------------------------------------------------------------- partial attention
// One CTA: 4 query heads of one KV head over tokens [begin, end). Warps take 32-token
// tiles round-robin; a lane scores one token, then owns two output dims for the P.V sum.
// q: bf16 [4][64] (this KV head's heads); k, v: first token's row of this KV head;
// kv_stride: elements between consecutive tokens. Results: out [4][64] normalised, lse2 [4].
__device__ void attention_partial(const __nv_bfloat16* __restrict__ q,
                                  const __nv_bfloat16* __restrict__ k,
                                  const __nv_bfloat16* __restrict__ v, int kv_stride, int begin,
                                  int end, float scale_log2, float* smem, float* out,
                                  float* lse) {
  float* qs = smem;                         // [4][64]
  float* part_m = smem + 256;               // [warps][4]
  float* part_l = part_m + kDecWarps * 4;   // [warps][4]
  float* part_o = part_l + kDecWarps * 4;   // [warps][4][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 256; i += blockDim.x)
    qs[i] = ld_bf16_coherent(q + i) * scale_log2;
  __syncthreads();
  float m[4], l[4], acc[4][2];
#pragma unroll
  for (int h = 0; h < 4; ++h) { m[h] = -INFINITY; l[h] = 0.0f; acc[h][0] = acc[h][1] = 0.0f; }
  for (int t0 = begin + warp * 32; t0 < end; t0 += kDecWarps * 32) {
    const int t = t0 + lane;
    float s[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (t < end) {
      const uint4* krow = reinterpret_cast<const uint4*>(k + static_cast<size_t>(t) * kv_stride);
      uint4 kk[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) kk[c] = krow[c];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float d = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) d += dot8(kk[c], qs + h * 64 + c * 8);
        s[h] = d;
      }
    }
    float p[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float tile_max = warp_max(s[h]);
      const float new_m = fmaxf(m[h], tile_max);
      const float corr = m[h] == -INFINITY ? 0.0f : exp2f(m[h] - new_m);
      p[h] = t < end ? exp2f(s[h] - new_m) : 0.0f;
      l[h] = l[h] * corr + warp_sum(p[h]);
      acc[h][0] *= corr;
      acc[h][1] *= corr;
      m[h] = new_m;
    }
    const int n = min(32, end - t0);
    for (int j = 0; j < n; ++j) {
      const uint32_t vv = *reinterpret_cast<const uint32_t*>(
          v + static_cast<size_t>(t0 + j) * kv_stride + 2 * lane);
      const float v0 = blo(vv), v1 = bhi(vv);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float pj = __shfl_sync(0xFFFFFFFFu, p[h], j);
        acc[h][0] = fmaf(pj, v0, acc[h][0]);
        acc[h][1] = fmaf(pj, v1, acc[h][1]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    if (lane == 0) { part_m[warp * 4 + h] = m[h]; part_l[warp * 4 + h] = l[h]; }
    part_o[(warp * 4 + h) * 64 + 2 * lane] = acc[h][0];
    part_o[(warp * 4 + h) * 64 + 2 * lane + 1] = acc[h][1];
  }
  __syncthreads();
  // merge the warps: thread (h, d) for h < 4, d < 64
  if (threadIdx.x < 256) {
    const int h = threadIdx.x >> 6, d = threadIdx.x & 63;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mx = fmaxf(mx, part_m[w * 4 + h]);
    float denom = 0.0f, val = 0.0f;
    if (mx != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float mw = part_m[w * 4 + h];
        const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mx);
        denom += part_l[w * 4 + h] * f;
        val += part_o[(w * 4 + h) * 64 + d] * f;
      }
    }
    out[h * 64 + d] = denom > 0.0f ? val / denom : 0.0f;
    if (d == 0) lse[h] = denom > 0.0f ? mx + log2f(denom) : -INFINITY;
  }
  __syncthreads();
}

__device__ __forceinline__ void partition_range(int length, int partitions, int part, int& begin,
                                                int& end) {
  const int blocks = (length + 15) / 16;
  const int per = (blocks + partitions - 1) / partitions;
  begin = part * per * 16;
  end = min(length, begin + per * 16);
  if (begin > end) begin = end;
}

// L2 prefetch of the weight rows an instruction will stream.
__device__ void prefetch_weights(const DecodeGlobals& g, const int* in) {
  const int op = in[0], layer = in[1], a0 = in[2], a1 = in[3];
  const __nv_bfloat16* wbase = nullptr;
  const __nv_bfloat16* wbase2 = nullptr;
  size_t wbytes = 0;
  if (op == 1) { wbase = g.qkv_w + (static_cast<size_t>(layer) * kQkvRows + a0) * kHidden; wbytes = static_cast<size_t>(a1) * kHidden * 2; }
  if (op == 4) { wbase = g.o_w + (static_cast<size_t>(layer) * kHidden + a0) * kHidden; wbytes = static_cast<size_t>(a1) * kHidden * 2; }
  if (op == 5) {
    wbase = g.gate_w + (static_cast<size_t>(layer) * kFfn + a0) * kHidden;
    wbase2 = g.up_w + (static_cast<size_t>(layer) * kFfn + a0) * kHidden;
    wbytes = static_cast<size_t>(a1) * kHidden * 2;
  }
  if (op == 6) { wbase = g.down_w + (static_cast<size_t>(layer) * kHidden + a0) * kFfn; wbytes = static_cast<size_t>(a1) * kFfn * 2; }
  if (op == 7) {  // the LM head (525 MB) exceeds L2: only its first 512 KB per SM is worth prefetching
    wbase = g.lm_head + static_cast<size_t>(a0) * kHidden;
    wbytes = static_cast<size_t>(a1) * kHidden * 2;
    if (wbytes > (512u << 10)) wbytes = 512u << 10;
  }
  if (wbase == nullptr) return;
  const char* pa = reinterpret_cast<const char*>(wbase);
  for (size_t off = static_cast<size_t>(threadIdx.x) * 128; off < wbytes; off += kDecThreads * 128) {
    prefetch_l2(pa + off);
    if (wbase2 != nullptr) prefetch_l2(reinterpret_cast<const char*>(wbase2) + off);
  }
}

// ---------------------------------------------------------------- the interpreter
__global__ void __launch_bounds__(kDecThreads, 1) decode_kernel(const DecodeGlobals g) {
  extern __shared__ __align__(16) float dsm[];
  float* x = dsm;                 // up to 8192 floats
  float* red = dsm + kFfn;        // 64 floats
  float* scratch = red + 64;      // attention workspace / argmax
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = *g.pos_dev;
  const int* my = g.instructions + static_cast<size_t>(blockIdx.x) * g.num_instructions * 32;

  for (int ip = 0; ip < g.num_instructions; ++ip) {
    const int* in = my + ip * 32;
    const int op = in[0];
    if (op == 0) continue;
    const int layer = in[1], a0 = in[2], a1 = in[3], a2 = in[4];
    const int dep = in[6], sig = in[8];
    const unsigned dep_target = static_cast<unsigned>(in[7]);

    // Keep HBM busy across the dependency stalls: the first instruction prefetches its own
    // weight rows into L2, every instruction prefetches the rows of the next one before it
    // starts computing, so a matvec mostly reads L2 while HBM streams the following slice.
    if (ip == 0) prefetch_weights(g, in);
    if (ip + 1 < g.num_instructions) prefetch_weights(g, in + 32);
    if (dep >= 0) {
      if (!wait_counter(g.bars + dep, dep_target, g.status, op * 100 + layer)) return;
    }

    if (op == 1) {
      // RMSNorm(hidden) -> rows [a0, a0+a1) of W_qkv -> RoPE on q/k pairs -> q_post_rope / KV append
      stage_vector(g.hidden, g.attn_norm + static_cast<size_t>(layer) * kHidden, kHidden, g.eps, x, red);
      const uint4* W = reinterpret_cast<const uint4*>(g.qkv_w + static_cast<size_t>(layer) * kQkvRows * kHidden);
      for (int pr = warp; pr < a1 / 2; pr += kDecWarps) {
        const int r = a0 + 2 * pr;
        float s0, s1;
        warp_dot2(W + static_cast<size_t>(r) * (kHidden / 8), W + static_cast<size_t>(r + 1) * (kHidden / 8), x, kHidden / 8, lane, s0, s1);
        if (lane == 0) {
          const size_t cache_row = (static_cast<size_t>(layer) * g.max_seq_len + pos) * (kKvHeads * kHeadDim);
          if (r < (kQHeads + kKvHeads) * kHeadDim) {
            const int pair = (r & (kHeadDim - 1)) >> 1;
            const float c = g.rope_cos[static_cast<size_t>(pos) * 32 + pair];
            const float sn = g.rope_sin[static_cast<size_t>(pos) * 32 + pair];
            const float o0 = s0 * c - s1 * sn, o1 = s1 * c + s0 * sn;
            if (r < kQHeads * kHeadDim) {
              g.q_post_rope[r] = __float2bfloat16_rn(o0);
              g.q_post_rope[r + 1] = __float2bfloat16_rn(o1);
            } else {
              const int kr = r - kQHeads * kHeadDim;
              g.k_cache[cache_row + kr] = __float2bfloat16_rn(o0);
              g.k_cache[cache_row + kr + 1] = __float2bfloat16_rn(o1);
            }
          } else {
            const int vr = r - (kQHeads + kKvHeads) * kHeadDim;
            g.v_cache[cache_row + vr] = __float2bfloat16_rn(s0);
            g.v_cache[cache_row + vr + 1] = __float2bfloat16_rn(s1);
          }
        }
      }
    } else if (op == 2) {
      // a0 = kv head, a1 = partitions, a2 = partition index
      int begin, end;
      partition_range(pos + 1, a1, a2, begin, end);
      const size_t kv_base = static_cast<size_t>(layer) * g.max_seq_len * (kKvHeads * kHeadDim) + a0 * kHeadDim;
      // partial layout: [head][part][64]; heads of this KV head are a0*4 .. a0*4+3
      float* tmp_out = scratch + 256 + kDecWarps * 8 + kDecWarps * 256;
      float* tmp_lse = tmp_out + 256;
      attention_partial(g.q_post_rope + a0 * 4 * kHeadDim, g.k_cache + kv_base, g.v_cache + kv_base,
                        kKvHeads * kHeadDim, begin, end, g.attn_scale * 1.4426950408889634f, scratch,
                        tmp_out, tmp_lse);
      if (threadIdx.x < 256) {
        const int h = threadIdx.x >> 6, d = threadIdx.x & 63;
        g.attn_out_partial[(static_cast<size_t>(a0 * 4 + h) * g.max_parts + a2) * 64 + d] = tmp_out[h * 64 + d];
        if (d == 0) g.attn_lse_partial[static_cast<size_t>(a0 * 4 + h) * g.max_parts + a2] = tmp_lse[h];
      }
    } else if (op == 3) {
      // merge partials of heads [a0, a0+a1): a2 = partitions
      for (int idx = threadIdx.x; idx < a1 * 64; idx += blockDim.x) {
        const int head = a0 + idx / 64, d = idx & 63;
        const volatile float* lse = g.attn_lse_partial + static_cast<size_t>(head) * g.max_parts;
        float mx = -INFINITY;
        for (int p = 0; p < a2; ++p) mx = fmaxf(mx, lse[p]);
        float sum = 0.0f, val = 0.0f;
        if (mx != -INFINITY) {
          for (int p = 0; p < a2; ++p) {
            const float lp = lse[p];
            const float w = lp == -INFINITY ? 0.0f : exp2f(lp - mx);
            sum += w;
            val += w * *reinterpret_cast<const volatile float*>(
                           g.attn_out_partial + (static_cast<size_t>(head) * g.max_parts + p) * 64 + d);
          }
        }
        g.attn_out[head * 64 + d] = __float2bfloat16_rn(sum > 0.0f ? val / sum : 0.0f);
      }
    } else if (op == 4 || op == 6) {
      // hidden[r] += W[r, :] . v   (v = attn_out for 4, silu_out for 6)
      const int K = op == 4 ? kHidden : kFfn;
      stage_vector(op == 4 ? g.attn_out : g.silu_out, nullptr, K, g.eps, x, red);
      const __nv_bfloat16* Wb = op == 4 ? g.o_w + static_cast<size_t>(layer) * kHidden * kHidden
                                        : g.down_w + static_cast<size_t>(layer) * kHidden * kFfn;
      const uint4* W = reinterpret_cast<const uint4*>(Wb);
      for (int pr = warp; pr < a1 / 2; pr += kDecWarps) {
        const int r = a0 + 2 * pr;
        float s0, s1;
        warp_dot2(W + static_cast<size_t>(r) * (K / 8), W + static_cast<size_t>(r + 1) * (K / 8), x, K / 8, lane, s0, s1);
        if (lane == 0) {
          g.hidden[r] = __float2bfloat16_rn(ld_bf16_coherent(g.hidden + r) + s0);
          g.hidden[r + 1] = __float2bfloat16_rn(ld_bf16_coherent(g.hidden + r + 1) + s1);
        }
      }
    } else if (op == 5) {
      stage_vector(g.hidden, g.mlp_norm + static_cast<size_t>(layer) * kHidden, kHidden, g.eps, x, red);
      const uint4* G = reinterpret_cast<const uint4*>(g.gate_w + static_cast<size_t>(layer) * kFfn * kHidden);
      const uint4* U = reinterpret_cast<const uint4*>(g.up_w + static_cast<size_t>(layer) * kFfn * kHidden);
      for (int i = warp; i < a1; i += kDecWarps) {
        const int r = a0 + i;
        float sg, su;
        warp_dot2(G + static_cast<size_t>(r) * (kHidden / 8), U + static_cast<size_t>(r) * (kHidden / 8), x, kHidden / 8, lane, sg, su);
        if (lane == 0) g.silu_out[r] = __float2bfloat16_rn(sg / (1.0f + __expf(-sg)) * su);
      }
    } else if (op == 7) {
      stage_vector(g.hidden, g.lm_norm, kHidden, g.eps, x, red);
      const uint4* W = reinterpret_cast<const uint4*>(g.lm_head);
      float best = -INFINITY;
      int best_idx = 0x7FFFFFFF;
      for (int pr = warp; pr < a1 / 2; pr += kDecWarps) {
        const int r = a0 + 2 * pr;
        float s0, s1;
        warp_dot2(W + static_cast<size_t>(r) * (kHidden / 8), W + static_cast<size_t>(r + 1) * (kHidden / 8), x, kHidden / 8, lane, s0, s1);
        if (lane == 0) {
          const __nv_bfloat16 b0 = __float2bfloat16_rn(s0), b1 = __float2bfloat16_rn(s1);
          g.logits[r] = b0;
          g.logits[r + 1] = b1;
          const float f0 = __bfloat162float(b0), f1 = __bfloat162float(b1);
          if (f0 > best || (f0 == best && r < best_idx)) { best = f0; best_idx = r; }
          if (f1 > best || (f1 == best && r + 1 < best_idx)) { best = f1; best_idx = r + 1; }
        }
      }
      float* bv = scratch;
      int* bi = reinterpret_cast<int*>(scratch + kDecWarps);
      if (lane == 0) { bv[warp] = best; bi[warp] = best_idx; }
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int w = 1; w < kDecWarps; ++w)
          if (bv[w] > best || (bv[w] == best && bi[w] < best_idx)) { best = bv[w]; best_idx = bi[w]; }
        g.argmax_val[blockIdx.x] = best;
        g.argmax_idx[blockIdx.x] = best_idx;
      }
    } else if (op == 8) {
      // greedy sample over the per-SM candidates (a0 = how many), next embedding row, position + 1
      __shared__ int token;
      if (threadIdx.x == 0) {
        float best = -INFINITY;
        int best_idx = 0x7FFFFFFF;
        for (int i = 0; i < a0; ++i) {
          const float v = *reinterpret_cast<const volatile float*>(g.argmax_val + i);
          const int id = *reinterpret_cast<const volatile int*>(g.argmax_idx + i);
          if (v > best || (v == best && id < best_idx)) { best = v; best_idx = id; }
        }
        token = best_idx;
        g.token_out[pos + 1] = best_idx;
        *g.pos_dev = pos + 1;
      }
      __syncthreads();
      const __nv_bfloat16* row = g.lm_head + static_cast<size_t>(token) * kHidden;
      for (int i = threadIdx.x; i < kHidden; i += blockDim.x) g.hidden[i] = row[i];
    }
    if (sig >= 0) signal_counter(g.bars + sig);
    __syncthreads();
  }
}

// Standalone harness for op 2 with the layout of the reference's checker
// (campaigns/megakernel/host/check_cute_attention.cu:16-45): grid = 8 * partitions CTAs,
// q bf16 [32][64], k/v bf16 [length][8][64], out f32 [(head*partitions+part)*4 + h][64].
__global__ void __launch_bounds__(kDecThreads, 1)
attention_partial_kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                         float* out, float* lse, int length, int partitions, float scale) {
  extern __shared__ __align__(16) float dsm[];
  const int head = blockIdx.x / partitions, part = blockIdx.x % partitions;
  int begin, end;
  partition_range(length, partitions, part, begin, end);
  float* tmp_out = dsm + 256 + kDecWarps * 8 + kDecWarps * 256;
  float* tmp_lse = tmp_out + 256;
  attention_partial(q + head * 4 * kHeadDim, k + head * kHeadDim, v + head * kHeadDim,
                    kKvHeads * kHeadDim, begin, end, scale * 1.4426950408889634f, dsm, tmp_out,
                    tmp_lse);
  if (threadIdx.x < 256) {
    const int h = threadIdx.x >> 6, d = threadIdx.x & 63;
    const int index = (head * partitions + part) * 4 + h;
    out[static_cast<size_t>(index) * 64 + d] = tmp_out[h * 64 + d];
    if (d == 0) lse[index] = tmp_lse[h];
  }
}

constexpr int kDecodeSmemFloats = kFfn + 64 + 256 + kDecWarps * 8 + kDecWarps * 256 + 256 + 8;
constexpr int kAttnSmemFloats = 256 + kDecWarps * 8 + kDecWarps * 256 + 256 + 8;

}  // namespace

cudaError_t launch_decode_step(const DecodeGlobals& g, int num_sms, cudaStream_t stream) {
  const int smem = kDecodeSmemFloats * 4;
  cudaError_t err = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  DecodeGlobals copy = g;
  void* args[] = {&copy};
  // cooperative launch: every CTA of the grid is resident, which the counter waits rely on
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_kernel), dim3(num_sms),
                                     dim3(kDecThreads), args, smem, stream);
}

cudaError_t launch_attention_partial(const void* q, const void* k, const void* v, float* out,
                                     float* lse, int length, int partitions, float scale,
                                     cudaStream_t stream) {
  const int smem = kAttnSmemFloats * 4;
  cudaError_t err = cudaFuncSetAttribute(attention_partial_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  attention_partial_kernel<<<kKvHeads * partitions, kDecThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
      static_cast<const __nv_bfloat16*>(v), out, lse, length, partitions, scale);
  return cudaGetLastError();
}

}  // namespace plb
