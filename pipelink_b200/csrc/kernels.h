// Internal launcher declarations shared by the kernel translation units and the
// C-ABI layer. Every launcher enqueues work on `stream` and returns a cudaError_t
// from the launch; none synchronises or allocates.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace plb {

// ---- MXFP8 quantisation (quant.cu)
cudaError_t launch_quantize_rows(const void* const* src_peers, const int* peer_rank,
                                 const int* peer_token_idx, const int* num_rows_dev,
                                 int64_t rows, int64_t cols, void* dst_fp8, void* dst_sc,
                                 cudaStream_t stream);
cudaError_t launch_quantize_plain(const void* src_bf16, int64_t rows, int64_t cols, void* dst_fp8,
                                  void* dst_sc, cudaStream_t stream);
cudaError_t launch_quantize_tile(const void* src_bf16, int64_t rows, int64_t cols, const int* live_rows_dev, void* dst_fp8,
                                 void* dst_sc, void* dst_t_fp8, void* dst_t_sc, cudaStream_t stream);
cudaError_t launch_quantize_transposed(const void* src_bf16, int64_t rows, int64_t cols,
                                       void* dst_t_fp8, void* dst_t_sc, cudaStream_t stream);
cudaError_t launch_dequantize(const void* src_fp8, const void* src_sc, int64_t rows, int64_t cols,
                              float* dst, cudaStream_t stream);
cudaError_t launch_pack_gate_up(const void* gate_fp8, const void* gate_sc, const void* up_fp8,
                                const void* up_sc, int experts, int inter, int hidden, int block,
                                void* w13_fp8, void* w13_sc, cudaStream_t stream);
cudaError_t launch_weighted_combine(const void* combine_bf16, const float* router_weights,
                                    const void* y_shared_bf16, int64_t tokens, int topk,
                                    int64_t hidden, void* out_bf16, cudaStream_t stream, const int* index = nullptr);

// ---- routing schedule (schedule.cu)
struct ScheduleArgs {
  const int* routes;      // [world * tokens * topk] global expert ids
  int world, tokens, topk;
  int expert_base;        // first global expert id owned by this rank
  int num_local_experts;
  int capacity;           // rows available in the schedule arrays (multiple of 128)
  int padding;            // every expert segment is padded to a multiple of this (multiple of 128)
  int* peer_rank;         // [capacity] source rank, -1 on padding rows
  int* peer_token_idx;    // [capacity] token index on the source rank
  int* dest_row;          // [capacity] token * topk + slot on the source rank, -1 on padding
  int* num_tokens;        // [1] padded rows in use
  int* tokens_per_expert; // [num_local_experts] unpadded counts
  int* expert_offsets;    // [num_local_experts + 1] first row of each segment
  int* block_expert;      // [capacity / 128] local expert of each 128-row block, -1 if unused
  int* scratch;           // [schedule_scratch_ints(...)]
  Status* status;
  // Receive-stream positions of the combine push, written by the same three launches when
  // stream_row is set (needs tokens * topk % kScheduleChunk == 0, so that no chunk spans two ranks):
  // stream_row[p] = rank * stream_cap + (earlier rows of this schedule with the same home rank), and
  // that position is also stored at stream_index_peers[home][dest_row[p]], where the home rank's
  // epilogue looks its (token, slot) rows up.
  int* stream_row = nullptr;                // [capacity], -1 on padding rows
  int* const* stream_index_peers = nullptr; // per home rank: i32 [tokens * topk]
  int* stream_tables = nullptr;             // scratch, [2 * world * num_local_experts]
  int rank = 0;
  int64_t stream_cap = 0;
};
constexpr int kScheduleChunk = 1024;
inline int64_t schedule_scratch_ints(int64_t entries, int num_local_experts) {
  return ((entries + kScheduleChunk - 1) / kScheduleChunk) * num_local_experts;
}
cudaError_t launch_schedule(const ScheduleArgs& a, cudaStream_t stream);
// Same schedule with the chunk counts kept in a library-owned static device array
// (a.scratch is ignored). cudaErrorInvalidValue if the problem needs more than
// schedule_static_scratch_ints() ints.
cudaError_t launch_schedule_static(const ScheduleArgs& a, cudaStream_t stream);
int64_t schedule_static_scratch_ints();

// ---- grouped MXFP8 GEMM (grouped_gemm2.cu)
struct GroupedGemmArgs {
  const void* a_fp8;      // [rows_capacity, K]
  const void* a_sc;       // [rows_capacity/128, K/128, 32, 16]
  const void* b_fp8;      // [experts * n_rows, K]
  const void* b_sc;       // [experts * n_rows/128, K/128, 32, 16]
  int64_t rows_capacity;  // multiple of 256
  int experts;
  int n_rows;             // weight rows per expert (multiple of 256)
  int K;                  // multiple of 128
  const int* block_expert;
  const int* num_rows_dev;
  // mode 0: tile columns [0,128) are gate, [128,256) are up -> hidden (fp8 + scales), [rows, n_rows/2]
  // mode 1: tile columns are output columns -> bf16 rows scattered through dest_row, [*, n_rows]
  int mode;
  void* out;
  void* out_sc;
  const int* dest_row;
  void* const* out_peers = nullptr;  // mode 1: per-source-rank output bases (device array), or null
  const int* peer_rank = nullptr;    // mode 1 with out_peers
  const unsigned* ready = nullptr;   // mode 1: readiness counter per 256-row tile of A
  unsigned ready_target = 0;
  bool bf16 = false;                 // modes 0/1: a_fp8 / b_fp8 hold bf16, no scales, mode 0 writes bf16
  float swiglu_limit = 0.0f;         // mode 0: > 0 bounds gate from above and up from both sides
  // mode 0: dispatch inside the GEMM kernel (all null = A is already in place)
  const void* const* pull_xq = nullptr;        // per rank: u8 [tokens, K]
  const void* const* pull_sc_rows = nullptr;   // per rank: u32 [tokens, K / 128]
  const int* pull_peer_rank = nullptr;
  const int* pull_token_idx = nullptr;
  void* pull_scratch = nullptr;                // u32 [rows_capacity / 256 + 1], zeroed by the launcher
  int m_stride = 1;                  // row-tile distance between consecutive loop steps
  int m_rotation = 0;                // 256-row tiles are visited starting this many tiles in
  int num_sms;
  Status* status;
  void* profile = nullptr;  // cycle counters [grid, 16] i64, written only by profiling builds
  // mode 0, training: MXFP8 gate / up and bf16 hidden kept for the backward pass
  void* save_gate = nullptr;
  void* save_gate_sc = nullptr;
  void* save_up = nullptr;
  void* save_up_sc = nullptr;
  void* save_hidden = nullptr;
  // mode 2: weight gradients, contraction over each expert's schedule rows
  const int* expert_offsets = nullptr;
  int m_rows = 0;
};
// CTA pairs on 256x256 tiles: rows_capacity, every expert segment and n_rows are multiples of 256;
// mode 0 weights are interleaved per 128 rows.
cudaError_t launch_grouped_gemm_pair(const GroupedGemmArgs& a, cudaStream_t stream);

// ---- backward-pass stages (backward.cu)
cudaError_t launch_bwd_dy(const void* d_out, const void* y, const float* router_w, const int* peer_rank,
                          const int* peer_token_idx, const int* dest_row, const int* num_rows_dev,
                          int64_t capacity, int hidden, int topk, void* dy, float* d_router_w,
                          cudaStream_t stream);
cudaError_t launch_swiglu_bwd(const void* gate, const void* gate_sc, const void* up, const void* up_sc,
                              const void* d_hidden, const int* num_rows_dev, int64_t capacity, int inter,
                              float limit, void* dgu, cudaStream_t stream);
cudaError_t launch_swiglu_bwd_bf16(const void* gate, const void* up, const void* d_hidden, const int* num_rows_dev,
                                   int64_t capacity, int inter, float limit, void* dgu, cudaStream_t stream);
cudaError_t launch_transpose_bf16(const void* in, int64_t rows, int64_t cols, const int* live_rows_dev, void* out,
                                  cudaStream_t stream);
cudaError_t launch_ep_pull_rows_bulk(const void* const* xq_peers, const void* const* xsc_peers, const int* peer_rank,
                                     const int* peer_token_idx, const int* num_rows_dev, int64_t capacity, int hidden,
                                     void* x_routed_fp8, void* x_routed_sc, int scale_rows, Status* status,
                                     cudaStream_t stream);
cudaError_t launch_scale_rows(const void* xsc, int64_t tokens, int hidden, void* out, cudaStream_t stream);
cudaError_t launch_ep_stream_rows(const int* peer_rank, const int* dest_row, const int* num_rows_dev, int64_t capacity,
                                  int rank, int world, int64_t stream_cap, int* stream_row, int* const* index_peers,
                                  cudaStream_t stream);
cudaError_t launch_tp_push_rows(const void* src, int blocks, int64_t block_bytes, int parts, int rank, int world,
                                void* const* gather_peers, unsigned* const* ready_peers, int ctas,
                                cudaStream_t stream);
cudaError_t launch_ep_bwd_dy(const void* const* d_out_peers, const float* const* router_w_peers, const int* peer_rank,
                             const int* peer_token_idx, const int* dest_row, const int* num_rows_dev, int64_t capacity,
                             int hidden, void* dy, cudaStream_t stream);
cudaError_t launch_router_grad(const void* d_out, const void* combine, int64_t tokens, int topk, int hidden,
                               float* d_router_w, cudaStream_t stream, const int* row_index = nullptr);
cudaError_t launch_ep_gather_rows(const void* const* src_peers, const int* peer_rank, const int* peer_token_idx,
                                  const int* num_rows_dev, int64_t capacity, int cols, void* dst, cudaStream_t stream);
cudaError_t launch_gather_rows(const void* src, const int* peer_rank, const int* peer_token_idx,
                               const int* num_rows_dev, int64_t capacity, int cols, void* dst,
                               cudaStream_t stream);

// ---- expert-parallel plumbing (ep.cu)
cudaError_t launch_ep_barrier(unsigned* const* flags_peers, unsigned* state, int rank, int world,
                              Status* status, cudaStream_t stream);
cudaError_t launch_ep_publish(const void* src, int64_t bytes, void* const* dst_peers, int rank,
                              int world, cudaStream_t stream);
cudaError_t launch_cp_push_kv(const void* k_local, const void* v_local, int chunk_blocks,
                              int64_t block_bytes, int rank, int world, void* const* k_peers,
                              void* const* v_peers, unsigned* const* ready_peers, int ctas,
                              cudaStream_t stream);
cudaError_t launch_ep_pull_rows(const void* const* xq_peers, const void* const* xsc_peers,
                                const int* peer_rank, const int* peer_token_idx,
                                const int* num_rows_dev, int64_t capacity, int hidden,
                                void* x_routed_fp8, void* x_routed_sc, cudaStream_t stream);

}  // namespace plb
