// extern "C" layer: argument checks, then one launcher call per entry point.
// Declarations and their reference counterparts are in include/pipelink_b200.h.
#include "../../include/pipelink_b200.h"

#include <string.h>

#include "attention.h"
#include "decode.h"
#include "kernels.h"

namespace {

thread_local int g_last_cuda_error = 0;

float g_swiglu_limit = 0.0f;  // 0: plain SwiGLU

void* g_profile_buffer = nullptr;

cudaError_t run_gemm(plb::GroupedGemmArgs& a, cudaStream_t s) {
  a.profile = g_profile_buffer;
  a.swiglu_limit = g_swiglu_limit;
  return plb::launch_grouped_gemm_pair(a, s);
}

int from_cuda(cudaError_t err) {
  if (err == cudaSuccess) return PLB_OK;
  g_last_cuda_error = static_cast<int>(err);
  return err == cudaErrorInvalidValue ? PLB_E_ARGUMENT : PLB_E_CUDA;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return sms;
}

}  // namespace

extern "C" {

int plb_abi_version(void) { return PLB_ABI_VERSION; }

const char* plb_error_string(int code) {
  switch (code) {
    case PLB_OK: return "ok";
    case PLB_E_VERSION: return "ABI version mismatch";
    case PLB_E_CAPACITY: return "capacity exceeded";
    case PLB_E_ARGUMENT: return "bad argument";
    case PLB_E_CONTRACT: return "contract violated";
    case PLB_E_RESOURCE: return "resource unavailable";
    case PLB_E_BUILD: return "build failed";
    case PLB_E_RELEASE: return "release failed";
    case PLB_E_CUDA: return "CUDA call failed";
    default: return "unknown error";
  }
}

int plb_last_cuda_error(void) { return g_last_cuda_error; }

int plb_moe_set_swiglu_limit(float limit) {
  if (!(limit >= 0.0f) || limit > 3.0e38f) return PLB_E_ARGUMENT;
  g_swiglu_limit = limit;
  return PLB_OK;
}

float plb_moe_swiglu_limit(void) { return g_swiglu_limit; }
int plb_debug_set_profile_buffer(void* device_i64_grid_by_16) {
  g_profile_buffer = device_i64_grid_by_16;
#ifdef PLB_DECODE_PROFILE
  plb::set_decode_profile(device_i64_grid_by_16);
#endif
  return PLB_OK;
}
int plb_moe_tile_rows(void) { return 256; }

int plb_mxfp8_quantize(const void* src_bf16, int64_t rows, int64_t cols, void* dst_fp8,
                       void* dst_sc, void* dst_t_fp8, void* dst_t_sc, void* stream) {
  return plb_mxfp8_quantize_live(src_bf16, rows, cols, nullptr, dst_fp8, dst_sc, dst_t_fp8, dst_t_sc, stream);
}

int plb_mxfp8_quantize_live(const void* src_bf16, int64_t rows, int64_t cols, const int* live_rows_dev, void* dst_fp8,
                            void* dst_sc, void* dst_t_fp8, void* dst_t_sc, void* stream) {
  if (rows < 0 || cols < 0 || rows % 128 || cols % 128) return PLB_E_ARGUMENT;
  if (src_bf16 == nullptr || !aligned16(src_bf16)) return PLB_E_ARGUMENT;
  if ((dst_fp8 == nullptr) != (dst_sc == nullptr)) return PLB_E_ARGUMENT;
  if ((dst_t_fp8 == nullptr) != (dst_t_sc == nullptr)) return PLB_E_ARGUMENT;
  if (!aligned16(dst_fp8) || !aligned16(dst_sc) || !aligned16(dst_t_fp8) || !aligned16(dst_t_sc))
    return PLB_E_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dst_t_fp8 != nullptr || live_rows_dev != nullptr)   // the transposed orientation, alone or with the other: one pass
    return from_cuda(plb::launch_quantize_tile(src_bf16, rows, cols, live_rows_dev, dst_fp8, dst_sc, dst_t_fp8, dst_t_sc, s));
  if (dst_fp8 != nullptr) {
    const int rc = from_cuda(plb::launch_quantize_plain(src_bf16, rows, cols, dst_fp8, dst_sc, s));
    if (rc != PLB_OK) return rc;
  }
  if (dst_t_fp8 != nullptr) {
    const int rc =
        from_cuda(plb::launch_quantize_transposed(src_bf16, rows, cols, dst_t_fp8, dst_t_sc, s));
    if (rc != PLB_OK) return rc;
  }
  return PLB_OK;
}

int plb_mxfp8_dequantize(const void* src_fp8, const void* src_sc, int64_t rows, int64_t cols,
                         float* dst_f32, void* stream) {
  if (rows < 0 || cols < 0 || rows % 128 || cols % 128) return PLB_E_ARGUMENT;
  if (src_fp8 == nullptr || src_sc == nullptr || dst_f32 == nullptr) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_dequantize(src_fp8, src_sc, rows, cols, dst_f32,
                                          static_cast<cudaStream_t>(stream)));
}

size_t plb_moe_schedule_scratch_bytes(int world, int tokens, int topk, int num_local_experts) {
  const int64_t entries = static_cast<int64_t>(world) * tokens * topk;
  return static_cast<size_t>(plb::schedule_scratch_ints(entries, num_local_experts)) * sizeof(int);
}

int plb_moe_schedule(const int32_t* routes, int world, int tokens, int topk, int expert_base,
                     int num_local_experts, int capacity, int padding, int32_t* peer_rank,
                     int32_t* peer_token_idx, int32_t* dest_row, int32_t* num_tokens,
                     int32_t* tokens_per_expert, int32_t* expert_offsets, int32_t* block_expert,
                     void* scratch, size_t scratch_bytes, plb_status* status, void* stream) {
  if (world < 1 || tokens < 0 || topk < 1 || num_local_experts < 1 || num_local_experts > 1024)
    return PLB_E_ARGUMENT;
  if (capacity < 0 || capacity % 128 || padding < 128 || padding % 128) return PLB_E_ARGUMENT;
  if (!routes || !peer_rank || !peer_token_idx || !dest_row || !num_tokens || !tokens_per_expert ||
      !expert_offsets || !block_expert || !status)
    return PLB_E_ARGUMENT;
  const size_t need = plb_moe_schedule_scratch_bytes(world, tokens, topk, num_local_experts);
  if (need > 0 && (scratch == nullptr || scratch_bytes < need)) return PLB_E_CAPACITY;
  plb::ScheduleArgs a;
  a.routes = routes;
  a.world = world;
  a.tokens = tokens;
  a.topk = topk;
  a.expert_base = expert_base;
  a.num_local_experts = num_local_experts;
  a.capacity = capacity;
  a.padding = padding;
  a.peer_rank = peer_rank;
  a.peer_token_idx = peer_token_idx;
  a.dest_row = dest_row;
  a.num_tokens = num_tokens;
  a.tokens_per_expert = tokens_per_expert;
  a.expert_offsets = expert_offsets;
  a.block_expert = block_expert;
  a.scratch = static_cast<int*>(scratch);
  a.status = reinterpret_cast<plb::Status*>(status);
  return from_cuda(plb::launch_schedule(a, static_cast<cudaStream_t>(stream)));
}

size_t plb_moe_schedule_streams_scratch_bytes(int world, int tokens, int topk, int num_local_experts) {
  return plb_moe_schedule_scratch_bytes(world, tokens, topk, num_local_experts) +
         2u * static_cast<size_t>(world) * num_local_experts * sizeof(int);
}

int plb_moe_schedule_streams(const int32_t* routes, int world, int tokens, int topk, int expert_base,
                             int num_local_experts, int capacity, int padding, int32_t* peer_rank,
                             int32_t* peer_token_idx, int32_t* dest_row, int32_t* num_tokens,
                             int32_t* tokens_per_expert, int32_t* expert_offsets, int32_t* block_expert,
                             void* scratch, size_t scratch_bytes, int rank, int64_t stream_cap,
                             int32_t* stream_row, void* const* index_peers, plb_status* status,
                             void* stream) {
  if (world < 1 || world > 32 || tokens < 0 || topk < 1 || num_local_experts < 1 || num_local_experts > 1024)
    return PLB_E_ARGUMENT;
  if (capacity < 0 || capacity % 128 || padding < 128 || padding % 128) return PLB_E_ARGUMENT;
  if (!routes || !peer_rank || !peer_token_idx || !dest_row || !num_tokens || !tokens_per_expert ||
      !expert_offsets || !block_expert || !status || !stream_row || !index_peers)
    return PLB_E_ARGUMENT;
  if (rank < 0 || rank >= world || stream_cap < 1 || stream_cap * world > 2147483647LL) return PLB_E_ARGUMENT;
  // a counting chunk must not span two source ranks
  if ((static_cast<int64_t>(tokens) * topk) % plb::kScheduleChunk != 0) return PLB_E_ARGUMENT;
  const size_t need = plb_moe_schedule_streams_scratch_bytes(world, tokens, topk, num_local_experts);
  if (scratch == nullptr || scratch_bytes < need) return PLB_E_CAPACITY;
  plb::ScheduleArgs a;
  a.routes = routes;
  a.world = world;
  a.tokens = tokens;
  a.topk = topk;
  a.expert_base = expert_base;
  a.num_local_experts = num_local_experts;
  a.capacity = capacity;
  a.padding = padding;
  a.peer_rank = peer_rank;
  a.peer_token_idx = peer_token_idx;
  a.dest_row = dest_row;
  a.num_tokens = num_tokens;
  a.tokens_per_expert = tokens_per_expert;
  a.expert_offsets = expert_offsets;
  a.block_expert = block_expert;
  a.scratch = static_cast<int*>(scratch);
  a.status = reinterpret_cast<plb::Status*>(status);
  a.stream_row = stream_row;
  a.stream_index_peers = reinterpret_cast<int* const*>(index_peers);
  a.stream_tables = static_cast<int*>(scratch) +
                    plb_moe_schedule_scratch_bytes(world, tokens, topk, num_local_experts) / sizeof(int);
  a.rank = rank;
  a.stream_cap = stream_cap;
  return from_cuda(plb::launch_schedule(a, static_cast<cudaStream_t>(stream)));
}

size_t plb_moe_schedule_noalloc_max_scratch_bytes(void) {
  return static_cast<size_t>(plb::schedule_static_scratch_ints()) * sizeof(int);
}

int plb_moe_schedule_noalloc(const int32_t* routes, int world, int tokens, int topk,
                             int expert_base, int num_local_experts, int capacity, int padding,
                             int32_t* peer_rank, int32_t* peer_token_idx, int32_t* dest_row,
                             int32_t* num_tokens, int32_t* tokens_per_expert,
                             int32_t* expert_offsets, int32_t* block_expert, plb_status* status,
                             void* stream) {
  if (world < 1 || tokens < 0 || topk < 1 || num_local_experts < 1 || num_local_experts > 1024)
    return PLB_E_ARGUMENT;
  if (capacity < 0 || capacity % 128 || padding < 128 || padding % 128) return PLB_E_ARGUMENT;
  if (!routes || !peer_rank || !peer_token_idx || !dest_row || !num_tokens || !tokens_per_expert ||
      !expert_offsets || !block_expert || !status)
    return PLB_E_ARGUMENT;
  // the built-in scratch has a fixed size: refuse anything that would not fit
  if (plb_moe_schedule_scratch_bytes(world, tokens, topk, num_local_experts) >
      plb_moe_schedule_noalloc_max_scratch_bytes())
    return PLB_E_CAPACITY;
  plb::ScheduleArgs a;
  a.routes = routes;
  a.world = world;
  a.tokens = tokens;
  a.topk = topk;
  a.expert_base = expert_base;
  a.num_local_experts = num_local_experts;
  a.capacity = capacity;
  a.padding = padding;
  a.peer_rank = peer_rank;
  a.peer_token_idx = peer_token_idx;
  a.dest_row = dest_row;
  a.num_tokens = num_tokens;
  a.tokens_per_expert = tokens_per_expert;
  a.expert_offsets = expert_offsets;
  a.block_expert = block_expert;
  a.scratch = nullptr;
  a.status = reinterpret_cast<plb::Status*>(status);
  return from_cuda(plb::launch_schedule_static(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_dispatch(const void* const* x_peers, const int32_t* peer_rank,
                     const int32_t* peer_token_idx, const int32_t* num_tokens, int64_t capacity,
                     int64_t hidden, void* x_routed_fp8, void* x_routed_sc, void* stream) {
  if (capacity < 0 || capacity % 128 || hidden <= 0 || hidden % 128) return PLB_E_ARGUMENT;
  if (!x_peers || !peer_rank || !peer_token_idx || !num_tokens || !x_routed_fp8 || !x_routed_sc)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_fp8) || !aligned16(x_routed_sc)) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_quantize_rows(x_peers, peer_rank, peer_token_idx, num_tokens,
                                             capacity, hidden, x_routed_fp8, x_routed_sc,
                                             static_cast<cudaStream_t>(stream)));
}

int plb_moe_pack_gate_up(const void* gate_fp8, const void* gate_sc, const void* up_fp8,
                         const void* up_sc, int experts, int inter, int hidden, void* w13_fp8,
                         void* w13_sc, void* stream) {
  if (experts < 1 || inter < 128 || inter % 128 || hidden < 128 || hidden % 128)
    return PLB_E_ARGUMENT;
  if (!gate_fp8 || !gate_sc || !up_fp8 || !up_sc || !w13_fp8 || !w13_sc) return PLB_E_ARGUMENT;
  if (!aligned16(gate_fp8) || !aligned16(up_fp8) || !aligned16(w13_fp8)) return PLB_E_ARGUMENT;
  if (inter % plb_moe_tile_rows()) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_pack_gate_up(gate_fp8, gate_sc, up_fp8, up_sc, experts, inter,
                                            hidden, plb_moe_tile_rows() / 2, w13_fp8, w13_sc,
                                            static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_gate_up(const void* x_routed_fp8, const void* x_routed_sc, const void* w13_fp8,
                         const void* w13_sc, const int32_t* block_expert,
                         const int32_t* num_tokens, int64_t capacity, int experts, int inter,
                         int hidden, void* hidden_fp8, void* hidden_sc, plb_status* status,
                         void* stream) {
  if (capacity < 0 || capacity % plb_moe_tile_rows() || experts < 1 || inter < 128 || inter % 128 ||
      hidden < 128 || hidden % 128)
    return PLB_E_ARGUMENT;
  if (!x_routed_fp8 || !x_routed_sc || !w13_fp8 || !w13_sc || !block_expert || !num_tokens ||
      !hidden_fp8 || !hidden_sc || !status)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_fp8) || !aligned16(x_routed_sc) || !aligned16(w13_fp8) ||
      !aligned16(w13_sc) || !aligned16(hidden_fp8) || !aligned16(hidden_sc))
    return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.a_fp8 = x_routed_fp8;
  a.a_sc = x_routed_sc;
  a.b_fp8 = w13_fp8;
  a.b_sc = w13_sc;
  a.rows_capacity = capacity;
  a.experts = experts;
  a.n_rows = 2 * inter;
  a.K = hidden;
  a.block_expert = block_expert;
  a.num_rows_dev = num_tokens;
  a.mode = 0;
  a.out = hidden_fp8;
  a.out_sc = hidden_sc;
  a.dest_row = nullptr;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

static int gemm_down_impl(const void* hidden_fp8, const void* hidden_sc, const void* w2_fp8,
                          const void* w2_sc, const int32_t* block_expert,
                          const int32_t* num_tokens, const int32_t* dest_row, int64_t capacity,
                          int experts, int inter, int hidden, void* combine_bf16,
                          void* const* combine_peers, const int32_t* peer_rank, int tile_rotation, int tile_stride,
                          plb_status* status, void* stream) {
  if (tile_rotation < 0 || tile_stride < 1) return PLB_E_ARGUMENT;
  if (capacity < 0 || capacity % plb_moe_tile_rows() || experts < 1 || inter < 128 || inter % 128 ||
      hidden < 128 || hidden % 128)
    return PLB_E_ARGUMENT;
  if (!hidden_fp8 || !hidden_sc || !w2_fp8 || !w2_sc || !block_expert || !num_tokens ||
      !dest_row || !combine_bf16 || !status)
    return PLB_E_ARGUMENT;
  if (!aligned16(hidden_fp8) || !aligned16(hidden_sc) || !aligned16(w2_fp8) ||
      !aligned16(w2_sc) || !aligned16(combine_bf16))
    return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.a_fp8 = hidden_fp8;
  a.a_sc = hidden_sc;
  a.b_fp8 = w2_fp8;
  a.b_sc = w2_sc;
  a.rows_capacity = capacity;
  a.experts = experts;
  a.n_rows = hidden;
  a.K = inter;
  a.block_expert = block_expert;
  a.num_rows_dev = num_tokens;
  a.mode = 1;
  a.m_rotation = tile_rotation;
  a.m_stride = tile_stride;
  a.out = combine_bf16;
  a.out_sc = nullptr;
  a.dest_row = dest_row;
  a.out_peers = combine_peers;
  a.peer_rank = peer_rank;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_down(const void* hidden_fp8, const void* hidden_sc, const void* w2_fp8,
                      const void* w2_sc, const int32_t* block_expert, const int32_t* num_tokens,
                      const int32_t* dest_row, int64_t capacity, int experts, int inter, int hidden,
                      void* combine_bf16, plb_status* status, void* stream) {
  return gemm_down_impl(hidden_fp8, hidden_sc, w2_fp8, w2_sc, block_expert, num_tokens, dest_row,
                        capacity, experts, inter, hidden, combine_bf16, nullptr, nullptr, 0, 1, status,
                        stream);
}

int plb_moe_gemm_down_push(const void* hidden_fp8, const void* hidden_sc, const void* w2_fp8,
                           const void* w2_sc, const int32_t* block_expert,
                           const int32_t* num_tokens, const int32_t* dest_row,
                           const int32_t* peer_rank, int64_t capacity, int experts, int inter,
                           int hidden, int tile_rotation, int tile_stride, void* const* combine_peers,
                           plb_status* status, void* stream) {
  if (!combine_peers || !peer_rank) return PLB_E_ARGUMENT;
  // the local base is only a non-null placeholder; every row is addressed through the table
  return gemm_down_impl(hidden_fp8, hidden_sc, w2_fp8, w2_sc, block_expert, num_tokens, dest_row,
                        capacity, experts, inter, hidden, const_cast<void**>(combine_peers),
                        combine_peers, peer_rank, tile_rotation, tile_stride, status, stream);
}

int plb_ep_barrier(void* const* flags_peers, void* state, int rank, int world, plb_status* status,
                   void* stream) {
  if (!flags_peers || !state || !status || world < 1 || world > 32 || rank < 0 || rank >= world)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_barrier(reinterpret_cast<unsigned* const*>(flags_peers),
                                          static_cast<unsigned*>(state), rank, world,
                                          reinterpret_cast<plb::Status*>(status),
                                          static_cast<cudaStream_t>(stream)));
}

int plb_ep_publish(const void* src, int64_t bytes, void* const* dst_peers, int rank, int world,
                   void* stream) {
  if (!src || !dst_peers || bytes < 0 || bytes % 16 || !aligned16(src) || world < 1 || rank < 0 ||
      rank >= world)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_publish(src, bytes, dst_peers, rank, world,
                                          static_cast<cudaStream_t>(stream)));
}

int plb_ep_pull_rows(const void* const* xq_peers, const void* const* xsc_peers,
                     const int32_t* peer_rank, const int32_t* peer_token_idx,
                     const int32_t* num_tokens, int64_t capacity, int64_t hidden,
                     void* x_routed_fp8, void* x_routed_sc, void* stream) {
  if (capacity < 0 || capacity % 128 || hidden <= 0 || hidden % 128) return PLB_E_ARGUMENT;
  if (!xq_peers || !xsc_peers || !peer_rank || !peer_token_idx || !num_tokens || !x_routed_fp8 ||
      !x_routed_sc)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_fp8) || !aligned16(x_routed_sc)) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_pull_rows(xq_peers, xsc_peers, peer_rank, peer_token_idx,
                                            num_tokens, capacity, static_cast<int>(hidden),
                                            x_routed_fp8, x_routed_sc,
                                            static_cast<cudaStream_t>(stream)));
}

int plb_ep_pull_rows_bulk(const void* const* xq_peers, const void* const* xsc_peers, const int32_t* peer_rank,
                          const int32_t* peer_token_idx, const int32_t* num_tokens, int64_t capacity, int64_t hidden,
                          void* x_routed_fp8, void* x_routed_sc, int scale_rows, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 128 || hidden <= 0 || hidden % 128 || hidden > 4096) return PLB_E_ARGUMENT;
  if (!xq_peers || !xsc_peers || !peer_rank || !peer_token_idx || !num_tokens || !x_routed_fp8 || !x_routed_sc ||
      !status)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_fp8) || !aligned16(x_routed_sc)) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_pull_rows_bulk(xq_peers, xsc_peers, peer_rank, peer_token_idx, num_tokens, capacity,
                                                 static_cast<int>(hidden), x_routed_fp8, x_routed_sc, scale_rows,
                                                 reinterpret_cast<plb::Status*>(status),
                                                 static_cast<cudaStream_t>(stream)));
}

int plb_ep_scale_rows(const void* xsc, int64_t tokens, int64_t hidden, void* scale_rows_u32, void* stream) {
  if (!xsc || !scale_rows_u32 || tokens < 0 || tokens % 128 || hidden <= 0 || hidden % 128) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_scale_rows(xsc, tokens, static_cast<int>(hidden), scale_rows_u32,
                                          static_cast<cudaStream_t>(stream)));
}

int plb_ep_stream_rows(const int32_t* peer_rank, const int32_t* dest_row, const int32_t* num_tokens, int64_t capacity,
                       int rank, int world, int64_t stream_cap, int32_t* stream_row, void* const* index_peers,
                       void* stream) {
  if (!peer_rank || !dest_row || !num_tokens || !stream_row || !index_peers || capacity < 0 || world < 1 ||
      world > 32 || rank < 0 || rank >= world || stream_cap < 1 || stream_cap * world > 2147483647LL)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_stream_rows(peer_rank, dest_row, num_tokens, capacity, rank, world, stream_cap,
                                              stream_row, reinterpret_cast<int* const*>(index_peers),
                                              static_cast<cudaStream_t>(stream)));
}

int plb_moe_fwd_epilogue_indexed(const void* y_shared_bf16, const void* rows_bf16, const int32_t* row_index,
                                 const float* router_weights, int64_t tokens, int topk, int64_t hidden,
                                 void* out_bf16, void* stream) {
  if (tokens < 0 || topk < 1 || hidden <= 0 || hidden % 8) return PLB_E_ARGUMENT;
  if (!rows_bf16 || !row_index || !router_weights || !out_bf16) return PLB_E_ARGUMENT;
  if (!aligned16(rows_bf16) || !aligned16(out_bf16) || !aligned16(y_shared_bf16)) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_weighted_combine(rows_bf16, router_weights, y_shared_bf16, tokens, topk, hidden,
                                                out_bf16, static_cast<cudaStream_t>(stream), row_index));
}

int plb_sym_alloc(size_t bytes, void** out) {
  if (!out || bytes == 0) return PLB_E_ARGUMENT;
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err != cudaSuccess) return from_cuda(err);
  err = cudaMemset(p, 0, bytes);
  if (err != cudaSuccess) {
    cudaFree(p);
    return from_cuda(err);
  }
  *out = p;
  return PLB_OK;
}

int plb_sym_free(void* p) { return p ? from_cuda(cudaFree(p)) : PLB_OK; }

int plb_ipc_export(void* p, void* handle64) {
  if (!p || !handle64) return PLB_E_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  return from_cuda(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p));
}

int plb_ipc_import(const void* handle64, void** out) {
  if (!handle64 || !out) return PLB_E_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return from_cuda(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}

int plb_ipc_close(void* p) { return p ? from_cuda(cudaIpcCloseMemHandle(p)) : PLB_OK; }

// Dispatch fused into the gate/up GEMM: rows are pulled into x_routed by a warp of every CTA
// while the tensor pipe works on the tiles already complete.
int plb_moe_gemm_gate_up_dispatch(const void* const* xq_peers, const void* const* xsc_rows_peers,
                                  const int32_t* peer_rank, const int32_t* peer_token_idx, void* x_routed_fp8,
                                  void* x_routed_sc, const void* w13_fp8, const void* w13_sc,
                                  const int32_t* block_expert, const int32_t* num_tokens, int64_t capacity,
                                  int experts, int inter, int hidden, void* hidden_fp8, void* hidden_sc,
                                  void* scratch_u32, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || inter < 128 || inter % 128 || hidden < 128 || hidden % 128 ||
      hidden > 4096)
    return PLB_E_ARGUMENT;
  if (!xq_peers || !xsc_rows_peers || !peer_rank || !peer_token_idx || !x_routed_fp8 || !x_routed_sc || !w13_fp8 ||
      !w13_sc || !block_expert || !num_tokens || !hidden_fp8 || !hidden_sc || !scratch_u32 || !status)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_fp8) || !aligned16(x_routed_sc) || !aligned16(w13_fp8) || !aligned16(w13_sc) ||
      !aligned16(hidden_fp8) || !aligned16(hidden_sc))
    return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.a_fp8 = x_routed_fp8; a.a_sc = x_routed_sc; a.b_fp8 = w13_fp8; a.b_sc = w13_sc;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = 2 * inter; a.K = hidden;
  a.block_expert = block_expert; a.num_rows_dev = num_tokens; a.mode = 0;
  a.out = hidden_fp8; a.out_sc = hidden_sc; a.dest_row = nullptr;
  a.pull_xq = xq_peers; a.pull_sc_rows = xsc_rows_peers; a.pull_peer_rank = peer_rank;
  a.pull_token_idx = peer_token_idx; a.pull_scratch = scratch_u32;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

// bf16 routed precision: the same two GEMMs on bf16 operands.
int plb_moe_gemm_gate_up_bf16(const void* x_routed_bf16, const void* w13_bf16, const int32_t* block_expert,
                              const int32_t* num_tokens, int64_t capacity, int experts, int inter, int hidden,
                              void* hidden_bf16, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || inter < 128 || inter % 128 || hidden < 128 || hidden % 128)
    return PLB_E_ARGUMENT;
  if (!x_routed_bf16 || !w13_bf16 || !block_expert || !num_tokens || !hidden_bf16 || !status) return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_bf16) || !aligned16(w13_bf16) || !aligned16(hidden_bf16)) return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.bf16 = true;
  a.a_fp8 = x_routed_bf16; a.a_sc = nullptr; a.b_fp8 = w13_bf16; a.b_sc = nullptr;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = 2 * inter; a.K = hidden;
  a.block_expert = block_expert; a.num_rows_dev = num_tokens; a.mode = 0;
  a.out = hidden_bf16; a.out_sc = nullptr; a.dest_row = nullptr;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_gate_up_bf16_train(const void* x_routed_bf16, const void* w13_bf16, const int32_t* block_expert,
                                    const int32_t* num_tokens, int64_t capacity, int experts, int inter, int hidden,
                                    void* hidden_bf16, void* gate_bf16, void* up_bf16, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || inter < 128 || inter % 128 || hidden < 128 || hidden % 128)
    return PLB_E_ARGUMENT;
  if (!x_routed_bf16 || !w13_bf16 || !block_expert || !num_tokens || !hidden_bf16 || !gate_bf16 || !up_bf16 || !status)
    return PLB_E_ARGUMENT;
  if (!aligned16(x_routed_bf16) || !aligned16(w13_bf16) || !aligned16(hidden_bf16) || !aligned16(gate_bf16) ||
      !aligned16(up_bf16))
    return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.bf16 = true;
  a.a_fp8 = x_routed_bf16; a.a_sc = nullptr; a.b_fp8 = w13_bf16; a.b_sc = nullptr;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = 2 * inter; a.K = hidden;
  a.block_expert = block_expert; a.num_rows_dev = num_tokens; a.mode = 0;
  a.out = hidden_bf16; a.out_sc = nullptr; a.dest_row = nullptr;
  a.save_gate = gate_bf16; a.save_up = up_bf16;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_wgrad_bf16(const void* a_t_bf16, const void* b_t_bf16, const int32_t* expert_offsets, int64_t capacity,
                            int experts, int m_rows, int n_rows, void* d_w_bf16, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || m_rows < 256 || m_rows % 256 || n_rows < 256 || n_rows % 256)
    return PLB_E_ARGUMENT;
  if (!a_t_bf16 || !b_t_bf16 || !expert_offsets || !d_w_bf16 || !status) return PLB_E_ARGUMENT;
  if (!aligned16(a_t_bf16) || !aligned16(b_t_bf16) || !aligned16(d_w_bf16)) return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.bf16 = true;
  a.a_fp8 = a_t_bf16; a.a_sc = nullptr; a.b_fp8 = b_t_bf16; a.b_sc = nullptr;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = n_rows; a.m_rows = m_rows; a.K = 0;
  a.block_expert = nullptr; a.num_rows_dev = nullptr; a.mode = 2;
  a.out = d_w_bf16; a.out_sc = nullptr; a.dest_row = nullptr;
  a.expert_offsets = expert_offsets;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(plb::launch_grouped_gemm_pair(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_swiglu_bwd_bf16(const void* gate_bf16, const void* up_bf16, const void* d_hidden_bf16,
                            const int32_t* num_tokens, int64_t capacity, int inter, void* d_gate_up_bf16, void* stream) {
  if (!gate_bf16 || !up_bf16 || !d_hidden_bf16 || !num_tokens || !d_gate_up_bf16 || capacity < 0 || inter <= 0 || inter % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_swiglu_bwd_bf16(gate_bf16, up_bf16, d_hidden_bf16, num_tokens, capacity, inter,
                                               g_swiglu_limit, d_gate_up_bf16, static_cast<cudaStream_t>(stream)));
}

int plb_bf16_transpose(const void* src_bf16, int64_t rows, int64_t cols, void* dst_bf16, void* stream) {
  return plb_bf16_transpose_live(src_bf16, rows, cols, nullptr, dst_bf16, stream);
}

int plb_bf16_transpose_live(const void* src_bf16, int64_t rows, int64_t cols, const int* live_rows_dev, void* dst_bf16,
                            void* stream) {
  if (!src_bf16 || !dst_bf16 || rows < 0 || cols < 0 || rows % 64 || cols % 64) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_transpose_bf16(src_bf16, rows, cols, live_rows_dev, dst_bf16, static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_down_bf16(const void* hidden_bf16, const void* w2_bf16, const int32_t* block_expert,
                           const int32_t* num_tokens, const int32_t* dest_row, const int32_t* peer_rank,
                           int64_t capacity, int experts, int inter, int hidden, int tile_rotation,
                           void* combine_bf16, void* const* combine_peers, plb_status* status, void* stream) {
  if (tile_rotation < 0 || capacity < 0 || capacity % 256 || experts < 1 || inter < 128 || inter % 128 ||
      hidden < 256 || hidden % 256)
    return PLB_E_ARGUMENT;
  if (!hidden_bf16 || !w2_bf16 || !block_expert || !num_tokens || !dest_row || !status) return PLB_E_ARGUMENT;
  if ((combine_peers == nullptr) == (combine_bf16 == nullptr)) return PLB_E_ARGUMENT;  // exactly one destination form
  if (combine_peers != nullptr && peer_rank == nullptr) return PLB_E_ARGUMENT;
  if (!aligned16(hidden_bf16) || !aligned16(w2_bf16) || !aligned16(combine_bf16)) return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.bf16 = true;
  a.a_fp8 = hidden_bf16; a.a_sc = nullptr; a.b_fp8 = w2_bf16; a.b_sc = nullptr;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = hidden; a.K = inter;
  a.block_expert = block_expert; a.num_rows_dev = num_tokens; a.mode = 1; a.m_rotation = tile_rotation;
  a.out = combine_bf16; a.out_sc = nullptr; a.dest_row = dest_row;
  a.out_peers = combine_peers; a.peer_rank = peer_rank;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_fwd_epilogue(const void* y_shared_bf16, const void* combine_bf16,
                         const float* router_weights, int64_t tokens, int topk, int64_t hidden,
                         void* out_bf16, void* stream) {
  if (tokens < 0 || topk < 1 || hidden <= 0 || hidden % 8) return PLB_E_ARGUMENT;
  if (!combine_bf16 || !router_weights || !out_bf16) return PLB_E_ARGUMENT;
  if (!aligned16(combine_bf16) || !aligned16(out_bf16) || !aligned16(y_shared_bf16))
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_weighted_combine(combine_bf16, router_weights, y_shared_bf16,
                                                tokens, topk, hidden, out_bf16,
                                                static_cast<cudaStream_t>(stream)));
}

int plb_decode_step(const plb_decode_args* args, int num_sms, void* stream) {
  static_assert(sizeof(plb_decode_args) == sizeof(plb::DecodeGlobals), "decode argument blocks differ");
  if (!args || num_sms < 1) return PLB_E_ARGUMENT;
  if (!args->qkv_w || !args->hidden || !args->instructions || !args->bars || !args->pos_dev ||
      !args->status || args->num_instructions < 1 || args->num_bars < 1 || args->max_parts < 1 ||
      args->layers < 1 || !args->k_cache || !args->v_cache)
    return PLB_E_ARGUMENT;
  plb::DecodeGlobals g;
  memcpy(&g, args, sizeof(g));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemsetAsync(args->bars, 0, sizeof(uint32_t) * args->num_bars, s);
  if (err != cudaSuccess) return from_cuda(err);
  return from_cuda(plb::launch_decode_step(g, num_sms, s));
}

int plb_decode_attention_partial(const void* q, const void* k, const void* v, float* out,
                                 float* lse, int length, int partitions, float scale,
                                 void* stream) {
  if (!q || !k || !v || !out || !lse || length < 0 || partitions < 1) return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_attention_partial(q, k, v, out, lse, length, partitions, scale,
                                                 static_cast<cudaStream_t>(stream)));
}

static int gate_up_train_impl(const void* const* xq_peers, const void* const* xsc_rows_peers, const int32_t* peer_rank,
                              const int32_t* peer_token_idx, void* scratch_u32, const void* x_routed_fp8,
                              const void* x_routed_sc, const void* w13_fp8, const void* w13_sc,
                              const int32_t* block_expert, const int32_t* num_tokens, int64_t capacity, int experts,
                              int inter, int hidden, void* hidden_fp8, void* hidden_sc, void* gate_fp8, void* gate_sc,
                              void* up_fp8, void* up_sc, void* hidden_bf16, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || inter < 256 || inter % 256 || hidden < 256 || hidden % 256)
    return PLB_E_ARGUMENT;
  if (!x_routed_fp8 || !x_routed_sc || !w13_fp8 || !w13_sc || !block_expert || !num_tokens || !hidden_fp8 ||
      !hidden_sc || !gate_fp8 || !gate_sc || !up_fp8 || !up_sc || !hidden_bf16 || !status)
    return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.a_fp8 = x_routed_fp8; a.a_sc = x_routed_sc; a.b_fp8 = w13_fp8; a.b_sc = w13_sc;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = 2 * inter; a.K = hidden;
  a.block_expert = block_expert; a.num_rows_dev = num_tokens; a.mode = 0;
  a.out = hidden_fp8; a.out_sc = hidden_sc; a.dest_row = nullptr;
  a.save_gate = gate_fp8; a.save_gate_sc = gate_sc; a.save_up = up_fp8; a.save_up_sc = up_sc;
  a.save_hidden = hidden_bf16;
  if (xq_peers != nullptr) {
    if (!xsc_rows_peers || !peer_rank || !peer_token_idx || !scratch_u32 || hidden > 4096) return PLB_E_ARGUMENT;
    a.pull_xq = xq_peers; a.pull_sc_rows = xsc_rows_peers; a.pull_peer_rank = peer_rank;
    a.pull_token_idx = peer_token_idx; a.pull_scratch = scratch_u32;
  }
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_gemm_gate_up_train(const void* x_routed_fp8, const void* x_routed_sc, const void* w13_fp8,
                               const void* w13_sc, const int32_t* block_expert, const int32_t* num_tokens,
                               int64_t capacity, int experts, int inter, int hidden, void* hidden_fp8,
                               void* hidden_sc, void* gate_fp8, void* gate_sc, void* up_fp8, void* up_sc,
                               void* hidden_bf16, plb_status* status, void* stream) {
  return gate_up_train_impl(nullptr, nullptr, nullptr, nullptr, nullptr, x_routed_fp8, x_routed_sc, w13_fp8, w13_sc,
                            block_expert, num_tokens, capacity, experts, inter, hidden, hidden_fp8, hidden_sc, gate_fp8,
                            gate_sc, up_fp8, up_sc, hidden_bf16, status, stream);
}

int plb_moe_gemm_gate_up_train_dispatch(const void* const* xq_peers, const void* const* xsc_rows_peers,
                                        const int32_t* peer_rank, const int32_t* peer_token_idx, void* x_routed_fp8,
                                        void* x_routed_sc, const void* w13_fp8, const void* w13_sc,
                                        const int32_t* block_expert, const int32_t* num_tokens, int64_t capacity,
                                        int experts, int inter, int hidden, void* hidden_fp8, void* hidden_sc,
                                        void* gate_fp8, void* gate_sc, void* up_fp8, void* up_sc, void* hidden_bf16,
                                        void* scratch_u32, plb_status* status, void* stream) {
  if (!xq_peers) return PLB_E_ARGUMENT;
  return gate_up_train_impl(xq_peers, xsc_rows_peers, peer_rank, peer_token_idx, scratch_u32, x_routed_fp8, x_routed_sc,
                            w13_fp8, w13_sc, block_expert, num_tokens, capacity, experts, inter, hidden, hidden_fp8,
                            hidden_sc, gate_fp8, gate_sc, up_fp8, up_sc, hidden_bf16, status, stream);
}

int plb_moe_gemm_wgrad(const void* a_t_fp8, const void* a_t_sc, const void* b_t_fp8, const void* b_t_sc,
                       const int32_t* expert_offsets, int64_t capacity, int experts, int m_rows, int n_rows,
                       void* d_w_bf16, plb_status* status, void* stream) {
  if (capacity < 0 || capacity % 256 || experts < 1 || m_rows < 256 || m_rows % 256 || n_rows < 256 || n_rows % 256)
    return PLB_E_ARGUMENT;
  if (!a_t_fp8 || !a_t_sc || !b_t_fp8 || !b_t_sc || !expert_offsets || !d_w_bf16 || !status) return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.a_fp8 = a_t_fp8; a.a_sc = a_t_sc; a.b_fp8 = b_t_fp8; a.b_sc = b_t_sc;
  a.rows_capacity = capacity; a.experts = experts; a.n_rows = n_rows; a.m_rows = m_rows; a.K = 0;
  a.block_expert = nullptr; a.num_rows_dev = nullptr; a.mode = 2;
  a.out = d_w_bf16; a.out_sc = nullptr; a.dest_row = nullptr;
  a.expert_offsets = expert_offsets;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(plb::launch_grouped_gemm_pair(a, static_cast<cudaStream_t>(stream)));
}

int plb_moe_bwd_dy(const void* d_out_bf16, const void* combine_bf16, const float* router_weights,
                   const int32_t* peer_rank, const int32_t* peer_token_idx, const int32_t* dest_row,
                   const int32_t* num_tokens, int64_t capacity, int hidden, int topk, void* d_y_bf16,
                   float* d_router_weights, void* stream) {
  if (!d_out_bf16 || !combine_bf16 || !router_weights || !peer_rank || !peer_token_idx || !dest_row ||
      !num_tokens || !d_y_bf16 || !d_router_weights || capacity < 0 || hidden <= 0 || hidden % 8 || topk < 1)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_bwd_dy(d_out_bf16, combine_bf16, router_weights, peer_rank, peer_token_idx,
                                      dest_row, num_tokens, capacity, hidden, topk, d_y_bf16, d_router_weights,
                                      static_cast<cudaStream_t>(stream)));
}

int plb_moe_swiglu_bwd(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                       const void* d_hidden_bf16, const int32_t* num_tokens, int64_t capacity, int inter,
                       void* d_gate_up_bf16, void* stream) {
  if (!gate_fp8 || !gate_sc || !up_fp8 || !up_sc || !d_hidden_bf16 || !num_tokens || !d_gate_up_bf16 ||
      capacity < 0 || capacity % 128 || inter <= 0 || inter % 128)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_swiglu_bwd(gate_fp8, gate_sc, up_fp8, up_sc, d_hidden_bf16, num_tokens, capacity,
                                          inter, g_swiglu_limit, d_gate_up_bf16,
                                          static_cast<cudaStream_t>(stream)));
}

int plb_moe_gather_rows(const void* src_bf16, const int32_t* peer_rank, const int32_t* peer_token_idx,
                        const int32_t* num_tokens, int64_t capacity, int cols, void* dst_bf16, void* stream) {
  if (!src_bf16 || !peer_rank || !peer_token_idx || !num_tokens || !dst_bf16 || capacity < 0 || cols <= 0 || cols % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_gather_rows(src_bf16, peer_rank, peer_token_idx, num_tokens, capacity, cols,
                                           dst_bf16, static_cast<cudaStream_t>(stream)));
}

int plb_ep_bwd_dy(const void* const* d_out_peers, const float* const* router_w_peers, const int32_t* peer_rank,
                  const int32_t* peer_token_idx, const int32_t* dest_row, const int32_t* num_tokens, int64_t capacity,
                  int hidden, void* d_y_bf16, void* stream) {
  if (!d_out_peers || !router_w_peers || !peer_rank || !peer_token_idx || !dest_row || !num_tokens || !d_y_bf16 ||
      capacity < 0 || hidden <= 0 || hidden % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_bwd_dy(d_out_peers, router_w_peers, peer_rank, peer_token_idx, dest_row, num_tokens,
                                         capacity, hidden, d_y_bf16, static_cast<cudaStream_t>(stream)));
}

int plb_moe_router_grad(const void* d_out_bf16, const void* combine_bf16, int64_t tokens, int topk, int hidden,
                        float* d_router_weights, void* stream) {
  if (!d_out_bf16 || !combine_bf16 || !d_router_weights || tokens < 0 || topk < 1 || hidden <= 0 || hidden % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_router_grad(d_out_bf16, combine_bf16, tokens, topk, hidden, d_router_weights,
                                           static_cast<cudaStream_t>(stream)));
}

int plb_moe_router_grad_indexed(const void* d_out_bf16, const void* rows_bf16, const int32_t* row_index, int64_t tokens,
                                int topk, int hidden, float* d_router_weights, void* stream) {
  if (!d_out_bf16 || !rows_bf16 || !row_index || !d_router_weights || tokens < 0 || topk < 1 || hidden <= 0 ||
      hidden % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_router_grad(d_out_bf16, rows_bf16, tokens, topk, hidden, d_router_weights,
                                           static_cast<cudaStream_t>(stream), row_index));
}

int plb_ep_gather_rows(const void* const* src_peers, const int32_t* peer_rank, const int32_t* peer_token_idx,
                       const int32_t* num_tokens, int64_t capacity, int cols, void* dst_bf16, void* stream) {
  if (!src_peers || !peer_rank || !peer_token_idx || !num_tokens || !dst_bf16 || capacity < 0 || cols <= 0 || cols % 8)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_ep_gather_rows(src_peers, peer_rank, peer_token_idx, num_tokens, capacity, cols, dst_bf16,
                                              static_cast<cudaStream_t>(stream)));
}

static int attention_impl(const void* q, const void* k, const void* v, void* out, float* lse,
                          const plb_attn_work* work, int num_work, int heads_per_work, int q_heads, int kv_heads, int seq_q,
                          uint64_t q_rows, uint64_t kv_rows, float scale, int window, float softcap, const uint32_t* ready,
                          uint32_t ready_target, plb::AttnArgs& a, plb_status* status, void* stream) {
  static_assert(sizeof(plb_attn_work) == sizeof(plb::AttnWork), "work descriptor layouts differ");
  if (!q || !k || !v || !out || !lse || !work || !status || num_work < 0) return PLB_E_ARGUMENT;
  if (q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || seq_q < 128 || seq_q % 128 ||
      q_rows % 128 || kv_rows % 128)
    return PLB_E_ARGUMENT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return PLB_E_ARGUMENT;
  if (heads_per_work != 1 && !(heads_per_work == 2 && (q_heads / kv_heads) % 2 == 0)) return PLB_E_ARGUMENT;
  a.heads_per_work = heads_per_work;
  a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
  a.work = reinterpret_cast<const plb::AttnWork*>(work);
  a.num_work = num_work;
  a.q_heads = q_heads; a.kv_heads = kv_heads; a.seq_q = seq_q;
  a.q_rows = q_rows; a.kv_rows = kv_rows;
  if (window < 0 || softcap < 0.0f) return PLB_E_ARGUMENT;
  a.scale = scale;
  a.window = window;
  a.softcap = softcap;
  a.ready = ready; a.ready_target = ready_target;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(plb::launch_attention_fwd(a, static_cast<cudaStream_t>(stream)));
}

int plb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                      const plb_attn_work* work, int num_work, int heads_per_work, int q_heads, int kv_heads, int seq_q,
                      uint64_t q_rows, uint64_t kv_rows, float scale, int window, float softcap, const uint32_t* ready,
                      uint32_t ready_target, plb_status* status, void* stream) {
  plb::AttnArgs a;
  return attention_impl(q, k, v, out, lse, work, num_work, heads_per_work, q_heads, kv_heads, seq_q, q_rows, kv_rows, scale,
                        window, softcap, ready, ready_target, a, status, stream);
}

int plb_attention_fwd_cp(const void* q, const void* k_gather, const void* v_gather, void* out, float* lse,
                         const plb_attn_work* work, int num_work, int q_heads, int kv_heads, int seq_q, uint64_t q_rows,
                         uint64_t kv_rows, float scale, const uint32_t* ready, uint32_t ready_target, const void* k_local,
                         const void* v_local, int chunk_blocks, int64_t block_bytes, int parts, int rank, int world,
                         void* const* k_gather_peers, void* const* v_gather_peers, void* const* ready_peers,
                         void* ticket_u32, plb_status* status, void* stream) {
  if (!ready || !k_local || !v_local || !k_gather_peers || !v_gather_peers || !ready_peers || !ticket_u32)
    return PLB_E_ARGUMENT;
  if (chunk_blocks < 0 || block_bytes <= 0 || parts < 1 || block_bytes % (16 * parts) || world < 1 || world > 32 ||
      rank < 0 || rank >= world || (q_heads / (kv_heads > 0 ? kv_heads : 1)) % 2)
    return PLB_E_ARGUMENT;
  plb::AttnArgs a;
  a.push_k = k_local; a.push_v = v_local;
  a.push_k_peers = k_gather_peers; a.push_v_peers = v_gather_peers;
  a.push_ready_peers = reinterpret_cast<unsigned* const*>(ready_peers);
  a.push_ticket = static_cast<unsigned*>(ticket_u32);
  a.push_chunk_blocks = chunk_blocks; a.push_parts = parts; a.push_rank = rank; a.push_world = world;
  a.push_block_bytes = block_bytes;
  return attention_impl(q, k_gather, v_gather, out, lse, work, num_work, 2, q_heads, kv_heads, seq_q, q_rows, kv_rows, scale, 0,
                        0.0f, ready, ready_target, a, status, stream);
}

int plb_cp_push_kv(const void* k_local, const void* v_local, int chunk_blocks, int64_t block_bytes,
                   int rank, int world, void* const* k_gather_peers, void* const* v_gather_peers,
                   void* const* ready_peers, int ctas, void* stream) {
  if (!k_local || !v_local || !k_gather_peers || !v_gather_peers || !ready_peers) return PLB_E_ARGUMENT;
  if (chunk_blocks < 0 || block_bytes <= 0 || block_bytes % 16 || world < 1 || rank < 0 ||
      rank >= world || ctas < 1)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_cp_push_kv(k_local, v_local, chunk_blocks, block_bytes, rank, world,
                                          k_gather_peers, v_gather_peers,
                                          reinterpret_cast<unsigned* const*>(ready_peers), ctas,
                                          static_cast<cudaStream_t>(stream)));
}

// ---- tensor-parallel compositions: all-gather -> GEMM and GEMM -> reduce-scatter push
int plb_tp_push_rows(const void* src, int blocks, int64_t block_bytes, int parts, int rank, int world,
                     void* const* gather_peers, void* const* ready_peers, int ctas, void* stream) {
  if (!src || !gather_peers || !ready_peers) return PLB_E_ARGUMENT;
  if (blocks < 0 || parts < 1 || block_bytes <= 0 || block_bytes % (16 * parts) || world < 1 || rank < 0 ||
      rank >= world || ctas < 1)
    return PLB_E_ARGUMENT;
  return from_cuda(plb::launch_tp_push_rows(src, blocks, block_bytes, parts, rank, world, gather_peers,
                                            reinterpret_cast<unsigned* const*>(ready_peers), ctas,
                                            static_cast<cudaStream_t>(stream)));
}

int plb_tp_gemm_bf16(const void* a_bf16, const void* b_bf16, const int32_t* block_group, const int32_t* num_rows,
                     const int32_t* dest_row, const int32_t* peer_rank, int64_t m, int n, int k, int tile_rotation,
                     const uint32_t* ready, uint32_t ready_target, void* out_bf16, void* const* out_peers,
                     plb_status* status, void* stream) {
  if (m <= 0 || m % 256 || n < 256 || n % 256 || k < 128 || k % 128 || tile_rotation < 0) return PLB_E_ARGUMENT;
  if (!a_bf16 || !b_bf16 || !block_group || !num_rows || !dest_row || !status) return PLB_E_ARGUMENT;
  if ((out_peers == nullptr) == (out_bf16 == nullptr)) return PLB_E_ARGUMENT;
  if (out_peers != nullptr && peer_rank == nullptr) return PLB_E_ARGUMENT;
  if (!aligned16(a_bf16) || !aligned16(b_bf16) || !aligned16(out_bf16)) return PLB_E_ARGUMENT;
  plb::GroupedGemmArgs a;
  a.bf16 = true;
  a.a_fp8 = a_bf16; a.a_sc = nullptr; a.b_fp8 = b_bf16; a.b_sc = nullptr;
  a.rows_capacity = m; a.experts = 1; a.n_rows = n; a.K = k;
  a.block_expert = block_group; a.num_rows_dev = num_rows; a.mode = 1; a.m_rotation = tile_rotation;
  a.ready = ready; a.ready_target = ready_target;
  a.out = out_bf16; a.out_sc = nullptr; a.dest_row = dest_row;
  a.out_peers = out_peers; a.peer_rank = peer_rank;
  a.num_sms = sm_count();
  a.status = reinterpret_cast<plb::Status*>(status);
  if (a.num_sms <= 0) return PLB_E_CUDA;
  return from_cuda(run_gemm(a, static_cast<cudaStream_t>(stream)));
}

// ---- linked-image launcher (cudaLibrary API) and tensor-map helper for stage providers
int plb_image_load(const void* image, const char* symbol, int dyn_smem_bytes, void** library,
                   void** kernel) {
  if (!image || !symbol || !library || !kernel) return PLB_E_ARGUMENT;
  cudaLibrary_t lib = nullptr;
  cudaError_t err = cudaLibraryLoadData(&lib, image, nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (err != cudaSuccess) return from_cuda(err);
  cudaKernel_t k = nullptr;
  err = cudaLibraryGetKernel(&k, lib, symbol);
  if (err == cudaSuccess && dyn_smem_bytes > 0)
    err = cudaFuncSetAttribute(reinterpret_cast<const void*>(k),
                               cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem_bytes);
  if (err != cudaSuccess) {
    cudaLibraryUnload(lib);
    return from_cuda(err);
  }
  *library = lib;
  *kernel = k;
  return PLB_OK;
}

int plb_image_launch(void* kernel, int grid_x, int grid_y, int grid_z, int threads,
                     int dyn_smem_bytes, const void* params_image, void* stream) {
  if (!kernel || !params_image || grid_x < 1 || grid_y < 1 || grid_z < 1 || threads < 32)
    return PLB_E_ARGUMENT;
  void* args[] = {const_cast<void*>(params_image)};
  return from_cuda(cudaLaunchKernel(kernel, dim3(grid_x, grid_y, grid_z), dim3(threads), args,
                                    dyn_smem_bytes, static_cast<cudaStream_t>(stream)));
}

int plb_image_launch_cooperative(void* kernel, int grid_x, int threads, int dyn_smem_bytes, const void* params_image,
                                 void* stream) {
  if (!kernel || !params_image || grid_x < 1 || threads < 32) return PLB_E_ARGUMENT;
  void* args[] = {const_cast<void*>(params_image)};
  // every CTA of the grid is resident at once: images whose CTAs wait on one another's counters need it
  return from_cuda(cudaLaunchCooperativeKernel(kernel, dim3(grid_x), dim3(threads), args, dyn_smem_bytes,
                                               static_cast<cudaStream_t>(stream)));
}

int plb_decode_kv_map(void* out128, const void* cache_bf16, int layers, int max_seq_len) {
  return from_cuda(plb::encode_decode_kv_map(out128, cache_bf16, layers, max_seq_len));
}

int plb_image_unload(void* library) {
  return library ? from_cuda(cudaLibraryUnload(static_cast<cudaLibrary_t>(library))) : PLB_OK;
}

int plb_tensor_map_2d_u8(void* out128, const void* base, uint64_t rows, uint64_t row_bytes,
                         uint32_t box_rows, uint32_t box_bytes, int swizzle128) {
  if (!out128 || !base || rows == 0 || row_bytes == 0 || row_bytes % 16 || box_bytes > 256 ||
      box_rows > 256)
    return PLB_E_ARGUMENT;
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                         CUtensorMapFloatOOBfill);
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return PLB_E_RESOURCE;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = reinterpret_cast<Fn>(sym)(
      &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return PLB_E_BUILD;
  memcpy(out128, &map, sizeof(map));
  return PLB_OK;
}

int plb_tensor_map_2d_bf16(void* out128, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                           uint32_t box_cols, int swizzle128) {
  if (!out128 || !base || rows == 0 || cols == 0 || cols % 8 || box_cols > 256 || box_rows > 256 || box_cols == 0 ||
      box_rows == 0 || (swizzle128 && box_cols != 64))
    return PLB_E_ARGUMENT;
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                         CUtensorMapFloatOOBfill);
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return PLB_E_RESOURCE;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = reinterpret_cast<Fn>(sym)(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return PLB_E_BUILD;
  memcpy(out128, &map, sizeof(map));
  return PLB_OK;
}

int plb_tensor_map_2d_u32(void* out128, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                          uint32_t box_cols) {
  if (!out128 || !base || rows == 0 || cols == 0 || cols % 4 || box_cols > 256 || box_rows > 256 || box_cols == 0 ||
      box_rows == 0)
    return PLB_E_ARGUMENT;
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                         CUtensorMapFloatOOBfill);
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return PLB_E_RESOURCE;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = reinterpret_cast<Fn>(sym)(
      &map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return PLB_E_BUILD;
  memcpy(out128, &map, sizeof(map));
  return PLB_OK;
}

}  // extern "C"
