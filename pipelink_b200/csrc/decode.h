// Argument block of the decode interpreter kernel; mirrored by plb_decode_args in
// include/pipelink_b200.h (same field order) and filled by the C-ABI layer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace plb {

struct DecodeGlobals {
  const __nv_bfloat16* qkv_w;      // [layers, 3072, 2048]
  const __nv_bfloat16* o_w;        // [layers, 2048, 2048]
  const __nv_bfloat16* up_w;       // [layers, 8192, 2048]
  const __nv_bfloat16* gate_w;     // [layers, 8192, 2048]
  const __nv_bfloat16* down_w;     // [layers, 2048, 8192]
  const __nv_bfloat16* attn_norm;  // [layers, 2048]
  const __nv_bfloat16* mlp_norm;   // [layers, 2048]
  const __nv_bfloat16* lm_norm;    // [2048]
  const __nv_bfloat16* lm_head;    // [vocab, 2048], also the embedding table (tied)
  __nv_bfloat16* k_cache;          // [layers, max_seq_len, 8, 64]
  __nv_bfloat16* v_cache;
  const float* rope_cos;           // [rope_rows, 32] one entry per rotated pair
  const float* rope_sin;
  __nv_bfloat16* hidden;           // [2048] residual stream
  __nv_bfloat16* q_post_rope;      // [2048]
  __nv_bfloat16* attn_out;         // [2048]
  __nv_bfloat16* silu_out;         // [8192]
  __nv_bfloat16* logits;           // [vocab]
  float* attn_out_partial;         // [32, max_parts, 64]
  float* attn_lse_partial;         // [32, max_parts]
  float* argmax_val;               // [num_sms]
  int* argmax_idx;                 // [num_sms]
  unsigned* bars;                  // dependency counters, zeroed before every launch
  const int* instructions;         // [num_sms, num_instructions, 32]
  int* pos_dev;                    // [1] position of the token being decoded
  int* token_out;                  // [max_seq_len] token_out[pos + 1] = greedy choice
  Status* status;
  int num_instructions;
  int max_seq_len;
  int max_parts;
  int vocab;
  float attn_scale;
  float eps;
  int num_bars;
  int layers;
};

#ifdef PLB_DECODE_PROFILE
cudaError_t set_decode_profile(void* buffer);  // profiling builds only: [grid][9][8] i64 cycle sums
#endif
cudaError_t launch_decode_step(const DecodeGlobals& g, int num_sms, cudaStream_t stream);
// The tensor map the decode kernel reads a KV cache through ([layers, max_seq_len, 8, 64] bf16, box = 128
// tokens of one head, 128-byte swizzle), for hosts that launch the linked decode image themselves.
cudaError_t encode_decode_kv_map(void* out128, const void* base, int layers, int max_seq_len);
cudaError_t launch_attention_partial(const void* q, const void* k, const void* v, float* out,
                                     float* lse, int length, int partitions, float scale,
                                     cudaStream_t stream);

}  // namespace plb
