// The decode interpreter's device code: helpers, the producer (stream) role and the consumer
// (interpret) role, shared by the library kernel (decode.cu) and by the separately packed stage
// owners (stages/decode). See decode.cu for what the kernel is and which reference files it follows.
#pragma once
#include "kernels.h"
#include "decode.h"

namespace plb {
namespace dec {
namespace {   // internal linkage: the header is compiled into the library kernel and into each stage unit

constexpr int kConsumers = 512;              // 16 consumer warps
constexpr int kDecWarps = kConsumers / 32;
constexpr int kDecThreads = kConsumers + 32;  // + the producer warp
constexpr int kStageBytes = 32768;
constexpr int kStages = 6;
constexpr int kTaskBytes = 2048;              // one warp task: 1024 bf16 of one weight row
constexpr int kPartialFloats = 2048;          // per-row partial sums of one block of rows
constexpr int kAttnSmemFloats = 256 + kDecWarps * 8 + kDecWarps * 256 + 256 + 8;  // attention workspace
constexpr int kInstWords = 12;                // words 0-8 of an instruction are used; kept 16-byte aligned
constexpr int kInstSmemBytes = 6144;          // streams of up to 128 instructions are copied to shared memory
// Ring copies mark their lines evict-first in L2: a weight byte is used once per token. (Measured
// on B200: asking L2 to prefetch slices ahead of the ring made a token 4-12 % slower, and bounding
// the copies in flight changed nothing, so neither is done.)
constexpr bool kEvictFirst = true;
constexpr int kHidden = 2048;
constexpr int kHeadDim = 64;
constexpr int kQHeads = 32;
constexpr int kKvHeads = 8;
constexpr int kFfn = 8192;
constexpr int kQkvRows = (kQHeads + 2 * kKvHeads) * kHeadDim;  // 3072

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

// All consumer threads (the producer warp never joins).
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
}

// 16-byte load of bf16 activations another SM wrote earlier in this launch.
__device__ __forceinline__ uint4 ld_coherent_v4(const void* p) {
  uint4 raw;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
               : "l"(p)
               : "memory");
  return raw;
}
__device__ __forceinline__ void unpack8(uint4 raw, float* f) {
  f[0] = blo(raw.x); f[1] = bhi(raw.x); f[2] = blo(raw.y); f[3] = bhi(raw.y);
  f[4] = blo(raw.z); f[5] = bhi(raw.z); f[6] = blo(raw.w); f[7] = bhi(raw.w);
}
__device__ __forceinline__ float dot8r(uint4 w, const float* x) {
  float s = blo(w.x) * x[0];
  s = fmaf(bhi(w.x), x[1], s);
  s = fmaf(blo(w.y), x[2], s);
  s = fmaf(bhi(w.y), x[3], s);
  s = fmaf(blo(w.z), x[4], s);
  s = fmaf(bhi(w.z), x[5], s);
  s = fmaf(blo(w.w), x[6], s);
  s = fmaf(bhi(w.w), x[7], s);
  return s;
}

// The activations one lane multiplies for a whole instruction: section `sec` of the input vector
// (1024 elements), chunks lane, lane + 32, lane + 64, lane + 96 of it. With `norm_w` the vector
// (2048 long) is RMS-normalised first: every warp reads all of it once, computes the sum of
// squares itself and keeps its own section.
__device__ __forceinline__ void load_norm_w(const __nv_bfloat16* __restrict__ norm_w, int sec, int lane,
                                            uint4 (&wn)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) wn[i] = *reinterpret_cast<const uint4*>(norm_w + sec * 1024 + (lane + 32 * i) * 8);
}
// `wn`: this lane's norm weights (load_norm_w; constants, so they are fetched before the
// instruction's dependency wait), ignored when `normed` is false. A 2048-long input is read from
// global memory once per CTA (256 threads, one 16-byte chunk each) and shared through `xs`
// (4 KB + 8 floats): 16 warps each reading all of it from the same few L2 lines on every SM
// made those lines a hot spot. An 8192-long input is read directly, every warp its own 2 KB.
__device__ __forceinline__ void load_x(const __nv_bfloat16* __restrict__ src, int K, bool normed,
                                       const uint4 (&wn)[4], int sec, int lane, float eps,
                                       float* xs, float (&xr)[32]) {
  if (K == kHidden) {
    uint4* xs4 = reinterpret_cast<uint4*>(xs);
    float* red = xs + 1024;
    if (threadIdx.x < 256) {
      const uint4 raw = ld_coherent_v4(src + threadIdx.x * 8);
      xs4[threadIdx.x] = raw;
      if (normed) {
        float f[8], ss = 0.0f;
        unpack8(raw, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        ss = warp_sum(ss);
        if (lane == 0) red[threadIdx.x >> 5] = ss;
      }
    }
    consumer_sync();
    float inv = 1.0f;
    if (normed) {
      float ss = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) ss += red[w];
      inv = rsqrtf(ss / static_cast<float>(kHidden) + eps);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
      unpack8(xs4[sec * 128 + lane + 32 * i], f);
      if (normed) {
        float w[8];
        unpack8(wn[i], w);
#pragma unroll
        for (int e = 0; e < 8; ++e) xr[i * 8 + e] = f[e] * inv * w[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xr[i * 8 + e] = f[e];
      }
    }
  } else {
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = ld_coherent_v4(src + sec * 1024 + (lane + 32 * i) * 8);
#pragma unroll
    for (int i = 0; i < 4; ++i) unpack8(raw[i], &xr[i * 8]);
  }
}

// Which weight rows an instruction streams: up to two matrices (gate, up) of `rows` rows of K.
struct Plan {
  const char* base[2];
  int nmat;
  int rows;
  int K;
};
__device__ __forceinline__ Plan plan_of(const DecodeGlobals& g, const int* in) {
  Plan p;
  p.base[0] = p.base[1] = nullptr;
  p.nmat = 0;
  p.rows = 0;
  p.K = kHidden;
  const int op = in[0], layer = in[1], a0 = in[2], a1 = in[3];
  if (op == 1) { p.base[0] = reinterpret_cast<const char*>(g.qkv_w + (static_cast<size_t>(layer) * kQkvRows + a0) * kHidden); p.nmat = 1; p.rows = a1; }
  if (op == 4) { p.base[0] = reinterpret_cast<const char*>(g.o_w + (static_cast<size_t>(layer) * kHidden + a0) * kHidden); p.nmat = 1; p.rows = a1; }
  if (op == 5) {
    p.base[0] = reinterpret_cast<const char*>(g.gate_w + (static_cast<size_t>(layer) * kFfn + a0) * kHidden);
    p.base[1] = reinterpret_cast<const char*>(g.up_w + (static_cast<size_t>(layer) * kFfn + a0) * kHidden);
    p.nmat = 2;
    p.rows = a1;
  }
  if (op == 6) { p.base[0] = reinterpret_cast<const char*>(g.down_w + (static_cast<size_t>(layer) * kHidden + a0) * kFfn); p.nmat = 1; p.rows = a1; p.K = kFfn; }
  if (op == 7) { p.base[0] = reinterpret_cast<const char*>(g.lm_head + static_cast<size_t>(a0) * kHidden); p.nmat = 1; p.rows = a1; }
  return p;
}
// Rows of one block: its partial sums (rows x matrices x warps per row) fit kPartialFloats.
__device__ __forceinline__ int block_rows_of(const Plan& p) {
  return kPartialFloats / ((p.K / 1024) * p.nmat);
}

// Bounded wait until counter >= target. Returns false after recording a failure.
__device__ bool wait_counter(const unsigned* counter, unsigned target, Status* st, int what) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      if (ld_acquire_gpu(counter) >= target) break;
      __nanosleep(40);   // 148 CTAs poll one line: back off so the bumps get through
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
  consumer_sync();
  const bool ok = ok_flag != 0;
  consumer_sync();
  return ok;
}

__device__ __forceinline__ void signal_counter(unsigned* counter) {
  consumer_sync();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}

// ---------------------------------------------------------------- partial attention
// One CTA: 4 query heads of one KV head over tokens [begin, end). A warp takes 32-token tiles;
// a lane scores one token against the 4 heads, then owns two output dims for the P.V sum.
// Results: out [4][64] normalised, lse2 [4] (base 2).
struct AttnAcc {
  float m[4], l[4], acc[4][2];
};
__device__ __forceinline__ void attn_init(AttnAcc& a) {
#pragma unroll
  for (int h = 0; h < 4; ++h) { a.m[h] = -INFINITY; a.l[h] = 0.0f; a.acc[h][0] = a.acc[h][1] = 0.0f; }
}

// One tile of n <= 32 tokens. kchunk(c): 16-byte chunk c (8 dims) of THIS lane's token's key row;
// vword(j): dims 2*lane, 2*lane+1 of token j's value row. qs: [4][64] queries, pre-scaled, in
// shared memory.
template <class KChunk, class VWord>
__device__ __forceinline__ void attn_tile(AttnAcc& a, const float* qs, int n, int lane, KChunk kchunk,
                                          VWord vword) {
  float s[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  if (lane < n) {
#pragma unroll
    for (int h = 0; h < 4; ++h) s[h] = 0.0f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 kk = kchunk(c);
#pragma unroll
      for (int h = 0; h < 4; ++h) s[h] += dot8(kk, qs + h * 64 + c * 8);
    }
  }
  float p[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const float tile_max = warp_max(s[h]);
    const float new_m = fmaxf(a.m[h], tile_max);
    const float corr = a.m[h] == -INFINITY ? 0.0f : exp2f(a.m[h] - new_m);
    p[h] = lane < n ? exp2f(s[h] - new_m) : 0.0f;
    a.l[h] = a.l[h] * corr + warp_sum(p[h]);
    a.acc[h][0] *= corr;
    a.acc[h][1] *= corr;
    a.m[h] = new_m;
  }
  // the value rows are fetched as two batches of 16 independent loads so their latencies overlap
#pragma unroll
  for (int jb = 0; jb < 32; jb += 16) {
    if (jb >= n) break;
    uint32_t vv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) vv[j] = jb + j < n ? vword(jb + j) : 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float v0 = blo(vv[j]), v1 = bhi(vv[j]);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float pj = __shfl_sync(0xFFFFFFFFu, p[h], jb + j);
        a.acc[h][0] = fmaf(pj, v0, a.acc[h][0]);
        a.acc[h][1] = fmaf(pj, v1, a.acc[h][1]);
      }
    }
  }
}

// smem floats: qs [256] | part_m [warps*4] | part_l [warps*4] | part_o [warps*4*64]
__device__ __forceinline__ void attn_stage_q(const __nv_bfloat16* __restrict__ q, float scale_log2, float* smem) {
  for (int i = threadIdx.x; i < 256; i += kConsumers) smem[i] = ld_bf16_coherent(q + i) * scale_log2;
  consumer_sync();
}

// Merge the 16 warps' states into out [4][64], lse [4].
__device__ void attn_merge(const AttnAcc& a, float* smem, float* out, float* lse) {
  float* part_m = smem + 256;               // [warps][4]
  float* part_l = part_m + kDecWarps * 4;   // [warps][4]
  float* part_o = part_l + kDecWarps * 4;   // [warps][4][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    if (lane == 0) { part_m[warp * 4 + h] = a.m[h]; part_l[warp * 4 + h] = a.l[h]; }
    part_o[(warp * 4 + h) * 64 + 2 * lane] = a.acc[h][0];
    part_o[(warp * 4 + h) * 64 + 2 * lane + 1] = a.acc[h][1];
  }
  consumer_sync();
  // thread (h, d) for h < 4, d < 64
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
  consumer_sync();
}

// Tokens [begin, end) straight from global memory (coherent loads: rows may have been written
// by other SMs earlier in this launch). k, v: first token's row of this KV head; kv_stride:
// elements between consecutive tokens.
__device__ __forceinline__ void attn_tiles_global(AttnAcc& a, const float* qs, const __nv_bfloat16* k,
                                                  const __nv_bfloat16* v, int kv_stride, int begin, int end,
                                                  int first_warp, int num_warps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < first_warp || warp >= first_warp + num_warps) return;
  for (int t0 = begin + (warp - first_warp) * 32; t0 < end; t0 += num_warps * 32) {
    const int n = min(32, end - t0);
    const __nv_bfloat16* krow = k + static_cast<size_t>(t0 + min(lane, n - 1)) * kv_stride;
    attn_tile(a, qs, n, lane,
              [&](int c) { return ld_coherent_v4(krow + c * 8); },
              [&](int j) {
                uint32_t w;
                asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(w) : "l"(v + static_cast<size_t>(t0 + j) * kv_stride + 2 * lane) : "memory");
                return w;
              });
  }
}

__device__ void attention_partial(const __nv_bfloat16* __restrict__ q,
                                  const __nv_bfloat16* __restrict__ k,
                                  const __nv_bfloat16* __restrict__ v, int kv_stride, int begin,
                                  int end, float scale_log2, float* smem, float* out,
                                  float* lse) {
  attn_stage_q(q, scale_log2, smem);
  AttnAcc a;
  attn_init(a);
  attn_tiles_global(a, smem, k, v, kv_stride, begin, end, 0, kDecWarps);
  attn_merge(a, smem, out, lse);
}

__device__ __forceinline__ void partition_range(int length, int partitions, int part, int& begin,
                                                int& end) {
  const int blocks = (length + 15) / 16;
  const int per = (blocks + partitions - 1) / partitions;
  begin = part * per * 16;
  end = min(length, begin + per * 16);
  if (begin > end) begin = end;
}

#ifdef PLB_DECODE_PROFILE
// Profiling builds: per CTA and opcode, cycles spent waiting for the dependency, working, and
// signalling, accumulated by thread 0 into [grid][9][8] i64 (slot 7: instruction count).
__device__ long long* g_decode_profile = nullptr;
#define DEC_PROF_T(var) const long long var = clock64()
#define DEC_PROF_MARK(var) var = clock64()
#define DEC_PROF_ADD(op, slot, cycles)                                                        \
  if (threadIdx.x == 0 && g_decode_profile != nullptr)                                        \
  g_decode_profile[(static_cast<size_t>(blockIdx.x) * 9 + (op)) * 8 + (slot)] += (cycles)
#else
#define DEC_PROF_T(var)
#define DEC_PROF_MARK(var)
#define DEC_PROF_ADD(op, slot, cycles)
#endif

// Op 3: merge the partials of heads [head0, head0 + nheads) over `parts` partitions. One warp
// per (head, 16 output dims); lanes take partitions, so every load of the merge is issued at once.
__device__ void merge_heads(const DecodeGlobals& g, int a0, int a1, int a2) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int task = warp; task < a1 * 4; task += kDecWarps) {
    const int head = a0 + (task >> 2), d0 = (task & 3) * 16;
    const volatile float* lse = g.attn_lse_partial + static_cast<size_t>(head) * g.max_parts;
    float mx = -INFINITY;
    for (int p = lane; p < a2; p += 32) mx = fmaxf(mx, lse[p]);
    mx = warp_max(mx);
    float sum = 0.0f, val[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) val[e] = 0.0f;
    if (mx != -INFINITY) {
      for (int p = lane; p < a2; p += 32) {
        const float lp = lse[p];
        const float w = lp == -INFINITY ? 0.0f : exp2f(lp - mx);
        sum += w;
        const float* src = g.attn_out_partial + (static_cast<size_t>(head) * g.max_parts + p) * 64 + d0;
        float4 o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(o[q].x), "=f"(o[q].y), "=f"(o[q].z), "=f"(o[q].w)
                       : "l"(src + q * 4)
                       : "memory");
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          val[q * 4 + 0] = fmaf(w, o[q].x, val[q * 4 + 0]);
          val[q * 4 + 1] = fmaf(w, o[q].y, val[q * 4 + 1]);
          val[q * 4 + 2] = fmaf(w, o[q].z, val[q * 4 + 2]);
          val[q * 4 + 3] = fmaf(w, o[q].w, val[q * 4 + 3]);
        }
      }
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int e = 0; e < 16; ++e) val[e] = warp_sum(val[e]);
    if (lane < 16) {
      float mine = 0.0f;
#pragma unroll
      for (int e = 0; e < 16; ++e) mine = lane == e ? val[e] : mine;
      g.attn_out[head * 64 + d0 + lane] = __float2bfloat16_rn(sum > 0.0f ? mine / sum : 0.0f);
    }
  }
}

// Ring stages of a partial-attention instruction: tokens [begin, lim) of one KV head, 128 per
// stage (16 KB of keys then 16 KB of values, rows of 128 bytes with the 128-byte swizzle). The
// token being decoded (row `pos`, written earlier in this launch) never goes through the ring.
struct AttnPlan {
  int begin, end, lim, stages;
};
__device__ __forceinline__ AttnPlan attn_plan_of(const int* in, int pos) {
  AttnPlan a;
  partition_range(pos + 1, in[3], in[4], a.begin, a.end);
  a.lim = min(a.end, pos);
  a.stages = a.lim > a.begin ? (a.lim - a.begin + 127) / 128 : 0;
  return a;
}

// One ring stage as the producer sees it.
struct StageDesc {
  const char* src;   // weights: first byte
  uint32_t bytes;    // bytes the stage's barrier expects
  int attn;          // 1: K and V boxes of 128 tokens through the tensor maps
  int head, token, layer;
  int op;
};

// Enumerates the stages of a CTA's instruction stream in the order the consumers take them.
struct StageCursor {
  int ip, sub, b0, m, r0;
  __device__ void reset() { ip = 0; sub = 0; b0 = 0; m = 0; r0 = 0; }
  __device__ bool next(const DecodeGlobals& g, const int* my, int stride, int pos, StageDesc& d) {
    for (; ip < g.num_instructions; ++ip, sub = 0, b0 = 0, m = 0, r0 = 0) {
      const int* in = my + ip * stride;
      d.op = in[0];
      if (in[0] == 2) {
        const AttnPlan ap = attn_plan_of(in, pos);
        if (sub >= ap.stages) continue;
        d.attn = 1;
        d.bytes = kStageBytes;
        d.head = in[2];
        d.token = ap.begin + sub * 128;
        d.layer = in[1];
        d.src = nullptr;
        ++sub;
        return true;
      }
      const Plan pl = plan_of(g, in);
      if (pl.nmat == 0 || b0 >= pl.rows) continue;
      const int row_bytes = pl.K * 2, rps = kStageBytes / row_bytes, brows = block_rows_of(pl);
      const int nb = min(brows, pl.rows - b0);
      d.attn = 0;
      d.bytes = static_cast<uint32_t>(min(rps, nb - r0)) * row_bytes;
      d.src = pl.base[m] + static_cast<size_t>(b0 + r0) * row_bytes;
      r0 += rps;
      if (r0 >= nb) {
        r0 = 0;
        if (++m >= pl.nmat) {
          m = 0;
          b0 += brows;   // past the last block the next call moves on to the next instruction
        }
      }
      return true;
    }
    return false;
  }
};


// ---------------------------------------------------------------- the two roles of a decode CTA
// Where things are in the CTA's dynamic shared memory is a policy L: the library kernel states
// constants (LibLayout in decode.cu), the linked image reads link-time handles. L::depth() ring
// stages of 32 KB at L::ring(), their full / empty barriers, the partial-sum block, the attention
// workspace and the copy of the instruction stream.

// Copies the used words of this CTA's instruction stream to shared memory (a miss on an instruction
// word would cost a full memory latency per instruction); longer streams are read in place. The
// caller synchronises the copying threads before anyone reads `local`.
__device__ __forceinline__ const int* stage_instructions(const DecodeGlobals& g, int* local, int tid, int nthreads, int& istride) {
  const int* my = g.instructions + static_cast<size_t>(blockIdx.x) * g.num_instructions * 32;
  istride = 32;
  if (g.num_instructions * kInstWords * 4 <= kInstSmemBytes) {
    for (int i = tid; i < g.num_instructions * kInstWords; i += nthreads)
      local[i] = my[(i / kInstWords) * 32 + i % kInstWords];
    my = local;
    istride = kInstWords;
  }
  return my;
}

// The producer: one lane walks the stage sequence of this CTA's instructions and issues the copies
// into the ring, never waiting for a dependency: HBM keeps streaming while the consumers sit at a counter.
template <class L>
__device__ __forceinline__ void stream_role(const DecodeGlobals& g, const CUtensorMap* map_k, const CUtensorMap* map_v,
                                            uint32_t smem, const int* my, int istride, int pos) {
  const int lane = threadIdx.x & 31;
  if (lane != 0) return;
  StageCursor load_c;
  load_c.reset();
  uint64_t policy = 0;
  if (kEvictFirst) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  uint32_t it = 0;
  bool ok = true;
  StageDesc d;
  while (ok && load_c.next(g, my, istride, pos, d)) {
    const int slot = it % L::depth();
    if (!mbar_wait(L::empty(smem, slot), ((it / L::depth()) & 1u) ^ 1u, g.status, ST_TIMEOUT_EMPTY, 900 + d.op)) { ok = false; break; }
    const uint32_t full = L::full(smem, slot);
    const uint32_t dst = smem + L::ring() + slot * kStageBytes;
    mbar_arrive_expect_tx(full, d.bytes);
    if (d.attn) {
      tma_load_4d(dst, map_k, full, 0, d.head, d.token, d.layer);
      tma_load_4d(dst + kStageBytes / 2, map_v, full, 0, d.head, d.token, d.layer);
    } else if (kEvictFirst) {
      bulk_load_hint(dst, d.src, d.bytes, full, policy);
    } else {
      bulk_load(dst, d.src, d.bytes, full);
    }
    ++it;
  }
  if (!ok) {  // let copies in flight land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000LL) {
    }
  }
}

// The sixteen consumer warps: the interpreter proper.
template <class L>
__device__ __forceinline__ void interpret_role(const DecodeGlobals& g, uint8_t* dsm, uint32_t smem, const int* my, int istride,
                                               int pos) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ volatile int stage_failed;  // a consumer warp gave up on a stage: all leave together at the next barrier
  if (threadIdx.x == 0) stage_failed = 0;
  consumer_sync();
  uint8_t* ring = dsm + L::ring();
  float* partial = reinterpret_cast<float*>(dsm + L::partial());
  float* scratch = reinterpret_cast<float*>(dsm + L::scratch());
  // ------------------------------------------------------------------ consumers
  uint32_t it = 0;
  for (int ip = 0; ip < g.num_instructions; ++ip) {
    const int* in = my + ip * istride;
    const int op = in[0];
    if (op == 0) continue;
    const int layer = in[1], a0 = in[2], a1 = in[3], a2 = in[4];
    const int dep = in[6], sig = in[8];
    const unsigned dep_target = static_cast<unsigned>(in[7]);
    DEC_PROF_T(t_start);
    // constants of this instruction are fetched before the dependency wait
    const Plan pl = plan_of(g, in);
    const int wpr = pl.K / 1024;          // warps per row: 2 or 8
    const int sec = warp % wpr, row_in_stage = warp / wpr;
    uint4 wn[4] = {};
    float rope_c = 0.0f, rope_s = 0.0f;
    if (op == 1) {
      load_norm_w(g.attn_norm + static_cast<size_t>(layer) * kHidden, sec, lane, wn);
      const int r = a0 + 2 * static_cast<int>(threadIdx.x);   // the pair this thread finishes in block 0
      if (2 * static_cast<int>(threadIdx.x) < a1 && r < (kQHeads + kKvHeads) * kHeadDim) {
        rope_c = g.rope_cos[static_cast<size_t>(pos) * 32 + ((r & (kHeadDim - 1)) >> 1)];
        rope_s = g.rope_sin[static_cast<size_t>(pos) * 32 + ((r & (kHeadDim - 1)) >> 1)];
      }
    } else if (op == 5) {
      load_norm_w(g.mlp_norm + static_cast<size_t>(layer) * kHidden, sec, lane, wn);
    } else if (op == 7) {
      load_norm_w(g.lm_norm, sec, lane, wn);
    }
    if (dep >= 0) {
      if (!wait_counter(g.bars + dep, dep_target, g.status, op * 100 + layer)) return;
    }
    DEC_PROF_T(t_dep);
#ifdef PLB_DECODE_PROFILE
    long long t_x = t_dep, t_st = t_dep, t_sy = t_dep;
#endif

    if (pl.nmat != 0) {
      // ---- matvec ops: partial sums of every row of the block, then the op's epilogue
      const int rps = kStageBytes / (pl.K * 2), brows = block_rows_of(pl);
      float xr[32];
      load_x(op == 4 ? g.attn_out : op == 6 ? g.silu_out : g.hidden, pl.K, op != 4 && op != 6, wn, sec, lane, g.eps, scratch, xr);
      DEC_PROF_MARK(t_x);
      float best = -INFINITY;
      int best_idx = 0x7FFFFFFF;
      for (int b0 = 0; b0 < pl.rows; b0 += brows) {
        const int nb = min(brows, pl.rows - b0);
        bool ok = true;
        for (int m = 0; m < pl.nmat && ok; ++m) {
          for (int r0 = 0; r0 < nb; r0 += rps, ++it) {
            const int slot = it % L::depth();
            if (!mbar_wait(L::full(smem, slot), (it / L::depth()) & 1u, g.status, ST_TIMEOUT_FULL, 800 + op)) { ok = false; break; }
            if (r0 + row_in_stage < nb) {
              const uint4* src = reinterpret_cast<const uint4*>(ring + slot * kStageBytes + warp * kTaskBytes);
              uint4 w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) w[i] = src[lane + 32 * i];
              float acc = 0.0f;
#pragma unroll
              for (int i = 0; i < 4; ++i) acc += dot8r(w[i], xr + i * 8);
              acc = warp_sum(acc);
              if (lane == 0) partial[(m * nb + r0 + row_in_stage) * wpr + sec] = acc;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(L::empty(smem, slot));
          }
        }
        // a failed wait has set the status word, so every other warp's wait gives up too and all
        // 16 warps still meet at this barrier before leaving
        if (!ok) stage_failed = 1;
        DEC_PROF_MARK(t_st);
        consumer_sync();
        DEC_PROF_MARK(t_sy);
        if (stage_failed != 0) return;
        // ---- epilogue of rows [b0, b0 + nb) of this instruction's slice
        auto row_sum = [&](int idx) {
          float v = 0.0f;
          for (int q = 0; q < wpr; ++q) v += partial[idx * wpr + q];
          return v;
        };
        if (op == 1) {
          for (int pr = threadIdx.x; pr < nb / 2; pr += kConsumers) {
            const int r = a0 + b0 + 2 * pr;
            const float s0 = row_sum(2 * pr), s1 = row_sum(2 * pr + 1);
            const size_t cache_row = (static_cast<size_t>(layer) * g.max_seq_len + pos) * (kKvHeads * kHeadDim);
            if (r < (kQHeads + kKvHeads) * kHeadDim) {
              const int pair = (r & (kHeadDim - 1)) >> 1;
              const bool early = b0 == 0 && pr == static_cast<int>(threadIdx.x);
              const float c = early ? rope_c : g.rope_cos[static_cast<size_t>(pos) * 32 + pair];
              const float sn = early ? rope_s : g.rope_sin[static_cast<size_t>(pos) * 32 + pair];
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
        } else if (op == 4 || op == 6) {
          for (int i = threadIdx.x; i < nb; i += kConsumers) {
            const int r = a0 + b0 + i;
            g.hidden[r] = __float2bfloat16_rn(ld_bf16_coherent(g.hidden + r) + row_sum(i));
          }
        } else if (op == 5) {
          for (int i = threadIdx.x; i < nb; i += kConsumers) {
            const float sg = row_sum(i), su = row_sum(nb + i);
            g.silu_out[a0 + b0 + i] = __float2bfloat16_rn(sg / (1.0f + __expf(-sg)) * su);
          }
        } else {
          for (int i = threadIdx.x; i < nb; i += kConsumers) {
            const int r = a0 + b0 + i;
            const __nv_bfloat16 bv16 = __float2bfloat16_rn(row_sum(i));
            g.logits[r] = bv16;
            const float f = __bfloat162float(bv16);
            if (f > best || (f == best && r < best_idx)) { best = f; best_idx = r; }
          }
        }
        consumer_sync();  // partial sums are free for the next block
      }
      if (op == 7) {
        // lowest id among the maxima of this CTA's slice
        const float wbest = warp_max(best);
        int cand = best == wbest ? best_idx : 0x7FFFFFFF;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) cand = min(cand, __shfl_xor_sync(0xFFFFFFFFu, cand, d));
        float* bv = scratch;
        int* bi = reinterpret_cast<int*>(scratch + kDecWarps);
        if (lane == 0) { bv[warp] = wbest; bi[warp] = cand; }
        consumer_sync();
        if (threadIdx.x == 0) {
          float cb = bv[0];
          int ci = bi[0];
          for (int w = 1; w < kDecWarps; ++w)
            if (bv[w] > cb || (bv[w] == cb && bi[w] < ci)) { cb = bv[w]; ci = bi[w]; }
          g.argmax_val[blockIdx.x] = cb;
          g.argmax_idx[blockIdx.x] = ci;
        }
      }
    } else if (op == 2) {
      // a0 = kv head, a1 = partitions, a2 = partition index, word 5 = 1 + arrival counter of this
      // KV head when the last partition to finish also merges (op 3 folded in), else 0
      const AttnPlan ap = attn_plan_of(in, pos);
      const size_t kv_base = static_cast<size_t>(layer) * g.max_seq_len * (kKvHeads * kHeadDim) + a0 * kHeadDim;
      float* tmp_out = scratch + 256 + kDecWarps * 8 + kDecWarps * 256;
      float* tmp_lse = tmp_out + 256;
      // the token being decoded: its K/V row was written by the QKV op of this launch, so it is
      // read directly (coherent loads, issued together with the query loads) by the last warp
      const bool has_tail = pos >= ap.begin && pos < ap.end;
      uint4 tail_k[8] = {};
      uint32_t tail_v = 0;
      if (has_tail && warp == kDecWarps - 1) {
        const size_t at = kv_base + static_cast<size_t>(pos) * (kKvHeads * kHeadDim);
#pragma unroll
        for (int c = 0; c < 8; ++c) tail_k[c] = ld_coherent_v4(g.k_cache + at + c * 8);
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(tail_v) : "l"(g.v_cache + at + 2 * lane) : "memory");
      }
      attn_stage_q(g.q_post_rope + a0 * 4 * kHeadDim, g.attn_scale * 1.4426950408889634f, scratch);
      DEC_PROF_MARK(t_x);
      AttnAcc acc;
      attn_init(acc);
      if (has_tail && warp == kDecWarps - 1)
        attn_tile(acc, scratch, 1, lane, [&](int c) { return tail_k[c]; }, [&](int) { return tail_v; });
      bool ok = true;
      for (int st = 0; st < ap.stages; ++st, ++it) {
        const int slot = it % L::depth();
        if (!mbar_wait(L::full(smem, slot), (it / L::depth()) & 1u, g.status, ST_TIMEOUT_FULL, 802)) { ok = false; break; }
        if ((warp >> 2) == (st & 3)) {   // four warps per stage, rotating, so stages overlap
          const int row0 = (warp & 3) * 32;
          const int n = min(32, ap.lim - (ap.begin + st * 128 + row0));
          if (n > 0) {
            const uint8_t* kb = ring + slot * kStageBytes;
            const uint8_t* vb = kb + kStageBytes / 2;
            const int krow = row0 + lane;
            attn_tile(acc, scratch, n, lane,
                      [&](int c) { return *reinterpret_cast<const uint4*>(kb + krow * 128 + ((c ^ (krow & 7)) << 4)); },
                      [&](int j) {
                        const int r = row0 + j;
                        return *reinterpret_cast<const uint32_t*>(vb + r * 128 + (((lane >> 2) ^ (r & 7)) << 4) + (lane & 3) * 4);
                      });
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(L::empty(smem, slot));
      }
      if (!ok) stage_failed = 1;
      DEC_PROF_MARK(t_st);
      attn_merge(acc, scratch, tmp_out, tmp_lse);
      DEC_PROF_MARK(t_sy);
      if (stage_failed != 0) return;
      // partial layout: [head][part][64]; heads of this KV head are a0*4 .. a0*4+3
      if (threadIdx.x < 256) {
        const int h = threadIdx.x >> 6, d = threadIdx.x & 63;
        g.attn_out_partial[(static_cast<size_t>(a0 * 4 + h) * g.max_parts + a2) * 64 + d] = tmp_out[h * 64 + d];
        if (d == 0) g.attn_lse_partial[static_cast<size_t>(a0 * 4 + h) * g.max_parts + a2] = tmp_lse[h];
      }
      if (in[5] > 0) {
        // count this partition in; whoever completes the KV head merges its four heads and
        // signals, everyone else moves on without signalling
        __shared__ int is_last;
        consumer_sync();
        if (threadIdx.x == 0) {
          __threadfence();
          const unsigned before = atomicAdd(g.bars + (in[5] - 1), 1u);
          __threadfence();
          is_last = before + 1u == static_cast<unsigned>(a1);
        }
        consumer_sync();
        DEC_PROF_T(t_arr);
        const bool last = is_last != 0;
        if (last) merge_heads(g, a0 * 4, 4, a1);
        DEC_PROF_T(t_mrg);
        if (sig >= 0 && last) signal_counter(g.bars + sig);
        consumer_sync();
        DEC_PROF_T(t_fin);
        DEC_PROF_ADD(op, 0, t_dep - t_start);   // dependency wait
        DEC_PROF_ADD(op, 1, t_x - t_dep);       // queries (and the current token's K/V) loaded
        DEC_PROF_ADD(op, 2, t_st - t_x);        // ring stages
        DEC_PROF_ADD(op, 3, t_sy - t_st);       // merge of the warps
        DEC_PROF_ADD(op, 4, t_arr - t_sy);      // partial stored, partition counted in
        DEC_PROF_ADD(op, 5, t_mrg - t_arr);     // last arriver: merge of the KV head
        DEC_PROF_ADD(op, 6, t_fin - t_mrg);     // last arriver: signal
        DEC_PROF_ADD(op, 7, 1);
        continue;
      }
    } else if (op == 3) {
      merge_heads(g, a0, a1, a2);
    } else if (op == 8) {
      // greedy sample over the per-SM candidates (a0 = how many), next embedding row, position + 1
      __shared__ int token;
      if (warp == 0) {
        float best = -INFINITY;
        int best_idx = 0x7FFFFFFF;
        for (int i = lane; i < a0; i += 32) {
          const float v = *reinterpret_cast<const volatile float*>(g.argmax_val + i);
          const int id = *reinterpret_cast<const volatile int*>(g.argmax_idx + i);
          if (v > best || (v == best && id < best_idx)) { best = v; best_idx = id; }
        }
        const float wbest = warp_max(best);
        int cand = best == wbest ? best_idx : 0x7FFFFFFF;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) cand = min(cand, __shfl_xor_sync(0xFFFFFFFFu, cand, d));
        if (lane == 0) {
          token = cand;
          g.token_out[pos + 1] = cand;
          *g.pos_dev = pos + 1;
        }
      }
      consumer_sync();
      const __nv_bfloat16* row = g.lm_head + static_cast<size_t>(token) * kHidden;
      for (int i = threadIdx.x; i < kHidden; i += kConsumers) g.hidden[i] = row[i];
    }
    DEC_PROF_T(t_work);
    if (sig >= 0) signal_counter(g.bars + sig);
    DEC_PROF_T(t_sig);
    consumer_sync();
    DEC_PROF_T(t_end);
    DEC_PROF_ADD(op, 0, t_dep - t_start);   // dependency wait
    DEC_PROF_ADD(op, 1, t_x - t_dep);       // activations into registers
    DEC_PROF_ADD(op, 2, t_st - t_x);        // thread 0's warp through its stages (last block)
    DEC_PROF_ADD(op, 3, t_sy - t_st);       // waiting for the other warps
    DEC_PROF_ADD(op, 4, t_work - t_sy);     // epilogue
    DEC_PROF_ADD(op, 5, t_sig - t_work);    // barrier + fence + counter bump
    DEC_PROF_ADD(op, 6, t_end - t_sig);
    DEC_PROF_ADD(op, 7, 1);
  }
}

}  // namespace
}  // namespace dec
}  // namespace plb
