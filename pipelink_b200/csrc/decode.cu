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
// every matvec is HBM-bound. Weights never depend on activations, so each CTA runs one
// producer warp that walks the CTA's instruction stream ahead of the consumers and streams the
// weight rows of ops 1, 4, 5, 6, 7 into a ring of 32 KB shared-memory stages with untiled bulk
// copies (mbarrier full/empty per stage): HBM stays busy while the 16 consumer warps wait for a
// dependency counter. A stage is 16 warp tasks of 2 KB (1024 bf16 of one row); a lane keeps its
// 32 activations in registers for the whole instruction, sums four 16-byte chunks per task,
// and per-row partial sums meet in shared memory where the op's epilogue (RoPE + KV append,
// residual add, SiLU * up, logits + argmax) runs once per block of rows.
//
// Every wait is bounded (cycle budget -> status record, all other waits give up).
#include <cstring>

#include "decode_roles.cuh"

namespace plb {

using namespace dec;

namespace {

struct DecBars {
  uint64_t full[kStages];
  uint64_t empty[kStages];
};
constexpr int kOffBars = kStages * kStageBytes;

// The library kernel's shared-memory map, as constants.
struct LibLayout {
  __device__ static constexpr int depth() { return kStages; }
  __device__ static constexpr int ring() { return 0; }
  __device__ static uint32_t full(uint32_t smem, int slot) { return smem + kOffBars + 8 * slot; }
  __device__ static uint32_t empty(uint32_t smem, int slot) { return smem + kOffBars + 8 * (kStages + slot); }
  __device__ static constexpr int partial() { return kOffBars + 128; }
  __device__ static constexpr int scratch() { return kOffBars + 128 + kPartialFloats * 4; }
  __device__ static constexpr int inst() { return kOffBars + 128 + (kPartialFloats + kAttnSmemFloats) * 4; }
};

// ---------------------------------------------------------------- the interpreter
__global__ void __launch_bounds__(kDecThreads, 1)
decode_kernel(const DecodeGlobals g, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t dsm_raw[];
  const uint32_t smem = smem_u32(dsm_raw);
  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);   // warp-uniform, and said so to the compiler
  const int pos = *g.pos_dev;
  int istride;
  const int* my = stage_instructions(g, reinterpret_cast<int*>(dsm_raw + LibLayout::inst()), threadIdx.x, kDecThreads, istride);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(LibLayout::full(smem, s), 1);
      mbar_init(LibLayout::empty(smem, s), kDecWarps);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == kDecWarps) {
    stream_role<LibLayout>(g, &map_k, &map_v, smem, my, istride, pos);
    return;
  }
  interpret_role<LibLayout>(g, dsm_raw, smem, my, istride, pos);
}

// Standalone harness for op 2 with the layout of the reference's checker
// (campaigns/megakernel/host/check_cute_attention.cu:16-45): grid = 8 * partitions CTAs,
// q bf16 [32][64], k/v bf16 [length][8][64], out f32 [(head*partitions+part)*4 + h][64].
__global__ void __launch_bounds__(kConsumers, 1)
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

constexpr int kDecodeSmemBytes = kStages * kStageBytes + 128 + (kPartialFloats + kAttnSmemFloats) * 4 + kInstSmemBytes;
static_assert(sizeof(DecBars) <= 128, "barrier block");
static_assert(kDecodeSmemBytes + 1024 <= 227 * 1024, "shared memory budget (1 KB of static shared memory and alignment)");

}  // namespace

#ifdef PLB_DECODE_PROFILE
cudaError_t set_decode_profile(void* buffer) {
  long long* p = static_cast<long long*>(buffer);
  return cudaMemcpyToSymbol(g_decode_profile, &p, sizeof(p));
}
#endif

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// KV cache [layers, max_seq_len, 8, 64] bf16 as a 4-D tensor; box = 128 tokens of one KV head
// (rows of 128 bytes, 128-byte swizzle). Rows past max_seq_len read as zeros.
bool encode_kv_map(CUtensorMap* map, const void* base, int layers, int max_seq_len) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return false;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(kKvHeads),
                              static_cast<cuuint64_t>(max_seq_len), static_cast<cuuint64_t>(layers)};
  const cuuint64_t strides[3] = {kHeadDim * 2, kKvHeads * kHeadDim * 2,
                                 static_cast<cuuint64_t>(max_seq_len) * kKvHeads * kHeadDim * 2};
  const cuuint32_t box[4] = {kHeadDim, 1, 128, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The maps depend only on (cache address, layers, max_seq_len): one decode session reuses them.
struct KvMapCache {
  const void* k = nullptr;
  const void* v = nullptr;
  int layers = 0, max_seq_len = 0;
  CUtensorMap map_k, map_v;
};

}  // namespace

cudaError_t encode_decode_kv_map(void* out128, const void* base, int layers, int max_seq_len) {
  CUtensorMap map;
  if (out128 == nullptr || base == nullptr || layers < 1 || max_seq_len < 1 || !encode_kv_map(&map, base, layers, max_seq_len))
    return cudaErrorInvalidValue;
  memcpy(out128, &map, sizeof(map));
  return cudaSuccess;
}

cudaError_t launch_decode_step(const DecodeGlobals& g, int num_sms, cudaStream_t stream) {
  const int smem = kDecodeSmemBytes;
  static thread_local KvMapCache cache;
  if (cache.k != g.k_cache || cache.v != g.v_cache || cache.layers != g.layers || cache.max_seq_len != g.max_seq_len) {
    if (g.layers < 1 || g.max_seq_len < 1 || !encode_kv_map(&cache.map_k, g.k_cache, g.layers, g.max_seq_len) ||
        !encode_kv_map(&cache.map_v, g.v_cache, g.layers, g.max_seq_len)) {
      cache.k = nullptr;
      return cudaErrorInvalidValue;
    }
    cache.k = g.k_cache;
    cache.v = g.v_cache;
    cache.layers = g.layers;
    cache.max_seq_len = g.max_seq_len;
  }
  cudaError_t err = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  DecodeGlobals copy = g;
  void* args[] = {&copy, &cache.map_k, &cache.map_v};
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
  attention_partial_kernel<<<kKvHeads * partitions, kConsumers, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
      static_cast<const __nv_bfloat16*>(v), out, lse, length, partitions, scale);
  return cudaGetLastError();
}

}  // namespace plb
