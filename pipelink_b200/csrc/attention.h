// Work descriptors and arguments of the prefill attention kernel (attention.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace plb {

// One 128-query tile of one head. Mirrored by plb_attn_work in include/pipelink_b200.h.
struct AttnWork {
  int q_row0;     // first row of the tile in the [batch*seq_q, q_heads*128] view of Q / O
  int q_pos0;     // global sequence position of that row (differs from the row under context parallelism)
  int kv_row0;    // row of key block 0 in the [kv_rows, kv_heads*128] view of K / V
  int kv_pos0;    // global sequence position of that key
  int kv_blocks;  // 128-key blocks to visit (causal: q_pos0 / 128 + 1 when kv_pos0 = 0)
  int head;       // query head (the first of two when records cover head pairs)
  int batch;
  int reserved;
};

struct AttnParams {
  const AttnWork* work;
  int num_work;
  int q_heads;
  int q_per_kv;
  int seq_q;
  __nv_bfloat16* out;
  float* lse;
  float scale_log2;
  float cap_in, cap_out;  // soft cap: score = cap_out * tanh(s * cap_in) in the base-2 domain (unused without a cap)
  int window;             // sliding window: keys with kv_pos > q_pos - window are visible; 0 = none
  unsigned ready_target;
  const unsigned* ready;  // per 128-key block readiness counters (context parallel), or null
  Status* status;
  // context parallel, K/V exchange inside this launch (null push_k: the blocks are pushed by a launch
  // in front of this one, or are local). Warps 2 and 3 of every CTA take tickets; a ticket is one of
  // push_parts pieces of one 128-token K/V block for one consumer rank, copied with 16-byte stores
  // and counted into that rank's ready[block] with a system-scope release.
  const uint4* push_k;
  const uint4* push_v;
  uint4* const* push_k_peers;
  uint4* const* push_v_peers;
  unsigned* const* push_ready_peers;
  unsigned* push_ticket;      // zeroed before the launch
  int push_chunk_blocks, push_vec_per_part, push_parts, push_rank, push_world;
};

struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  const AttnWork* work;
  int num_work;
  int heads_per_work;  // 1: one head per record; 2: records cover heads (head, head + 1) of one KV group
  int q_heads, kv_heads;
  int seq_q;
  uint64_t q_rows, kv_rows;
  float scale;
  float softcap;          // 0 = none
  int window;             // 0 = none
  const unsigned* ready;
  unsigned ready_target;
  int num_sms;
  Status* status;
  // in-kernel K/V push (all null / 0 = off); see AttnParams
  const void* push_k = nullptr;
  const void* push_v = nullptr;
  void* const* push_k_peers = nullptr;
  void* const* push_v_peers = nullptr;
  unsigned* const* push_ready_peers = nullptr;
  unsigned* push_ticket = nullptr;
  int push_chunk_blocks = 0, push_parts = 0, push_rank = 0, push_world = 0;
  int64_t push_block_bytes = 0;
};

cudaError_t launch_attention_fwd(const AttnArgs& a, cudaStream_t stream);

}  // namespace plb
