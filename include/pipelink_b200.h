/* pipelink_b200 — C ABI of the sm_100a stage kernels.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the
 * given CUDA stream (a cudaStream_t passed as void*; NULL = the legacy default
 * stream), and returns 0 (PLB_OK) or a PLB_E_* code. No entry point synchronises,
 * allocates device memory, or throws. Device-side failures (a bounded wait that ran
 * out, a schedule that does not fit its capacity) are written to the caller's
 * plb_status record, which the caller zeroes before a sequence of calls and reads
 * after synchronising the stream.
 *
 * Each declaration names the reference interface it stands in for, by path inside
 * the PipeLink tree.
 */
#ifndef PIPELINK_B200_H
#define PIPELINK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLB_ABI_VERSION 1

/* Return codes. 1..7 mirror PLK_E_* of the provider ABI
 * (pipec/src/pipec2/host/include/pipelink_host_abi_v2.h:21-28). */
enum {
  PLB_OK = 0,
  PLB_E_VERSION = 1,
  PLB_E_CAPACITY = 2,
  PLB_E_ARGUMENT = 3,
  PLB_E_CONTRACT = 4,
  PLB_E_RESOURCE = 5,
  PLB_E_BUILD = 6,
  PLB_E_RELEASE = 7,
  PLB_E_CUDA = 8 /* a CUDA runtime/driver call failed; see plb_last_cuda_error() */
};

/* Device-written status record (32 bytes, device memory, 4-byte aligned).
 * code: 0 healthy; 1 full-barrier timeout; 2 empty-barrier timeout; 3/4 accumulator
 * barrier timeouts; 5 readiness-counter timeout; 6 bad argument found on the device
 * (e.g. schedule larger than capacity); 7 drain timeout. */
typedef struct plb_status {
  int32_t code;
  int32_t who;      /* CTA that recorded the failure */
  int32_t what;     /* kernel-specific location */
  uint32_t observed;
  uint32_t expected;
  int32_t reserved[3];
} plb_status;

int plb_abi_version(void);
const char* plb_error_string(int code);
int plb_last_cuda_error(void);

/* Row granularity of the grouped GEMMs: CTA pairs on 256x256 tiles (cta_group::2, the reference's
 * geometry, campaigns/mok/port/gemm/gemm.cu:26-36). `padding` of the schedule, `capacity`, `inter`
 * and `hidden` must be multiples of it, and plb_moe_pack_gate_up interleaves in blocks of half of
 * it. A GEMM entry point refuses a capacity that is not a multiple (PLB_E_ARGUMENT), and a row tile
 * whose two 128-row blocks belong to different experts, or a row count that is not a multiple, is
 * reported on the device (status code 6) instead of being multiplied by the wrong weights. */
int plb_moe_tile_rows(void);
/* Clamped SwiGLU, process-wide (the reference selects it per link through
 * the variant handle pipelink_mok_clamp, campaigns/mok/port/act/act.cu:9,246-249, and carries the
 * bound as the scalar mok.clamp, act.cu:294): limit > 0 makes the gate/up epilogue compute
 * silu(min(gate, limit)) * clamp(up, -limit, limit) and plb_moe_swiglu_bwd pass no gradient
 * through a bound that is reached (campaigns/mok/port/act_gptoss/swiglu.cuh:13-37); 0 (default)
 * is the plain activation. Forward, recompute and backward calls must run under the same value. */
int plb_moe_set_swiglu_limit(float limit);
float plb_moe_swiglu_limit(void);
/* Diagnostics: a device buffer of [grid, 16] int64 that profiling builds of the library
 * (-DPLB_GEMM_PROFILE) fill with per-role cycle counters; ignored by regular builds. */
int plb_debug_set_profile_buffer(void* device_i64_grid_by_16);

/* ------------------------------------------------------------------ MXFP8
 * ops.mxfp8_quantize(tensor, normal, transposed) as used at
 * campaigns/mok/host/mok_port_host.py:122. src is bf16 [rows, cols], rows and cols
 * multiples of 128. dst_fp8 is u8 [rows, cols]; dst_sc is u8
 * [rows/128, cols/128, 32, 16] (campaigns/mok/host/resources.py:62-68). The
 * transposed outputs are [cols, rows] with blocks of 32 along the source rows.
 * Either pair of outputs may be NULL. */
int plb_mxfp8_quantize(const void* src_bf16, int64_t rows, int64_t cols, void* dst_fp8,
                       void* dst_sc, void* dst_t_fp8, void* dst_t_sc, void* stream);
/* The same for a routed buffer sized for the worst case: only the 128-row tiles below
 * *live_rows_dev (a device scalar, e.g. the schedule's num_tokens) are read and written; the
 * tensors keep `rows` as their leading dimension, the rest of them is left as it was. With
 * live_rows_dev NULL this is plb_mxfp8_quantize. */
int plb_mxfp8_quantize_live(const void* src_bf16, int64_t rows, int64_t cols, const int32_t* live_rows_dev,
                            void* dst_fp8, void* dst_sc, void* dst_t_fp8, void* dst_t_sc, void* stream);

/* Inverse of the above for checking: fp32 [rows, cols]. (No reference counterpart on
 * the host; mirrors mxfp8::dequantize_single_block,
 * campaigns/mok/port/act_gptoss/swiglu.cuh:395-396.) */
int plb_mxfp8_dequantize(const void* src_fp8, const void* src_sc, int64_t rows, int64_t cols,
                         float* dst_f32, void* stream);

/* ------------------------------------------------------------------ MoE routing schedule
 * ops.schedule_out (campaigns/mok/host/mok_port_host.py:59-69). routes is i32
 * [world, tokens, topk] (the all-gathered top-k ids); this rank owns experts
 * [expert_base, expert_base + num_local_experts). Every expert segment is padded to a
 * multiple of `padding` rows (a multiple of 128; the reference's EXPERT_PADDING,
 * campaigns/mok/port/framework/interp_fwd.cu:324). Outputs: peer_rank / peer_token_idx /
 * dest_row i32 [capacity]; num_tokens i32 [1] (padded rows in use); tokens_per_expert
 * i32 [num_local_experts]; expert_offsets i32 [num_local_experts + 1]; block_expert
 * i32 [capacity/128]. scratch holds plb_moe_schedule_scratch_bytes() bytes. */
size_t plb_moe_schedule_scratch_bytes(int world, int tokens, int topk, int num_local_experts);
int plb_moe_schedule(const int32_t* routes, int world, int tokens, int topk, int expert_base,
                     int num_local_experts, int capacity, int padding, int32_t* peer_rank,
                     int32_t* peer_token_idx, int32_t* dest_row, int32_t* num_tokens,
                     int32_t* tokens_per_expert, int32_t* expert_offsets, int32_t* block_expert,
                     void* scratch, size_t scratch_bytes, plb_status* status, void* stream);

/* The same schedule for callers that cannot provide scratch memory and cannot call
 * cudaMalloc themselves: a plugin that is handed only input and output pointers, a
 * stage built behind a broker that owns every workspace (the provider ABI gives a
 * stage no allocator), or a serving loop where an allocation would stall the whole
 * device. It has no counterpart in the reference. The chunk counts live in a 1 MiB
 * static device array inside the library (held by every GPU that loads the library
 * until the process exits), so:
 *   - problems whose plb_moe_schedule_scratch_bytes() exceeds
 *     plb_moe_schedule_noalloc_max_scratch_bytes() are refused with PLB_E_CAPACITY;
 *   - the first call on each device looks up the array's device address (no
 *     allocation); make that first call outside any stream capture;
 *   - all calls on a device share the array: two calls whose kernels can overlap on
 *     the GPU (different streams) race. Calls ordered on one stream are safe, and
 *     nothing in the array needs clearing between calls, because every count a call
 *     reads is first written by that call.
 * It never calls cudaMalloc, cudaFree or any allocating routine. Results are
 * identical to plb_moe_schedule. */
size_t plb_moe_schedule_noalloc_max_scratch_bytes(void);
int plb_moe_schedule_noalloc(const int32_t* routes, int world, int tokens, int topk,
                             int expert_base, int num_local_experts, int capacity, int padding,
                             int32_t* peer_rank, int32_t* peer_token_idx, int32_t* dest_row,
                             int32_t* num_tokens, int32_t* tokens_per_expert,
                             int32_t* expert_offsets, int32_t* block_expert, plb_status* status,
                             void* stream);

/* ------------------------------------------------------------------ MoE dispatch
 * dispatch_kernel (campaigns/mok/port/comm/comm.cu:105-123): for every scheduled row p,
 * x_routed[p] = quantise(x_peers[peer_rank[p]][peer_token_idx[p]]); padding rows become
 * zeros. x_peers is a device array of `world` device pointers to bf16 [tokens, hidden]
 * buffers (peer-mapped for other ranks). Rows at or beyond *num_tokens are not written. */
int plb_moe_dispatch(const void* const* x_peers, const int32_t* peer_rank,
                     const int32_t* peer_token_idx, const int32_t* num_tokens, int64_t capacity,
                     int64_t hidden, void* x_routed_fp8, void* x_routed_sc, void* stream);

/* Interleave reference-layout gate and up weights ([experts, inter, hidden] fp8 +
 * scales, campaigns/mok/host/resources.py:69) into the [experts, 2*inter, hidden]
 * operand of plb_moe_gemm_gate_up: per expert, B gate rows then the B up rows of the
 * same hidden indices, repeated, with B = plb_moe_tile_rows() / 2. Pure data movement. */
int plb_moe_pack_gate_up(const void* gate_fp8, const void* gate_sc, const void* up_fp8,
                         const void* up_sc, int experts, int inter, int hidden, void* w13_fp8,
                         void* w13_sc, void* stream);

/* FWD_ROUTED_GATE + FWD_ROUTED_UP (campaigns/mok/port/gemm/gemm.cu:150-157) fused with
 * mok_act_fwd (campaigns/mok/port/act/act.cu:100-178): hidden = silu(gate) * up,
 * rounded to bf16, quantised to MXFP8 along the intermediate dimension. */
int plb_moe_gemm_gate_up(const void* x_routed_fp8, const void* x_routed_sc, const void* w13_fp8,
                         const void* w13_sc, const int32_t* block_expert,
                         const int32_t* num_tokens, int64_t capacity, int experts, int inter,
                         int hidden, void* hidden_fp8, void* hidden_sc, plb_status* status,
                         void* stream);

/* FWD_ROUTED_DOWN (gemm.cu:158-162) with the combine stage's row placement
 * (combine_kernel, campaigns/mok/port/comm/comm.cu:124-129): row p of the product is
 * written as bf16 to combine[dest_row[p]], skipped where dest_row[p] < 0. */
int plb_moe_gemm_down(const void* hidden_fp8, const void* hidden_sc, const void* w2_fp8,
                      const void* w2_sc, const int32_t* block_expert, const int32_t* num_tokens,
                      const int32_t* dest_row, int64_t capacity, int experts, int inter, int hidden,
                      void* combine_bf16, plb_status* status, void* stream);

/* ------------------------------------------------------------------ MoE backward
 * plb_moe_gemm_gate_up_train: plb_moe_gemm_gate_up that also keeps what the backward pass reads,
 * as the reference's forward does (gemm.cu:150-157 emits gate/up in bf16 and MXFP8; the act stage
 * writes hidden in both orientations, act.cu:310-313): MXFP8 gate and up [capacity, inter] and the
 * bf16 hidden that was quantised (its transposed quantisation is a plb_mxfp8_quantize call).
 * plb_moe_bwd_dy: backward of the weighted combine for every scheduled row p = (t, slot):
 *   d_y[p] = bf16(w[t, slot] * d_out[t]), d_w[t, slot] = <d_out[t], combine[t*k+slot]>; padding rows
 *   become zeros. Rows at and beyond *num_tokens are not written: nothing downstream reads them
 *   (plb_mxfp8_quantize_live, the grouped GEMMs and the weight gradients stop at the rows in use).
 * plb_moe_swiglu_bwd: swiglu_bwd_kernel (campaigns/mok/port/act_gptoss/swiglu.cuh:219-558, default
 *   silu(g)*u math): d_gate_up bf16 [capacity, 2*inter] = [d_gate | d_up] from the saved MXFP8
 *   gate / up and bf16 d_hidden.
 * plb_moe_gather_rows: bf16 rows in schedule order (operand of the gate/up weight gradient).
 * plb_moe_gemm_wgrad: the wgrad cases of expert_grouped_gemm_kernel (gemm.cu:166-243): for every
 *   expert e, d_w[e] = A_t[:, rows of e] . B_t[:, rows of e]^T with both operands quantised along
 *   the schedule-row dimension ([m_rows, capacity] and [n_rows, capacity]); an expert without rows
 *   gets zeros (zero_empty_routed_wgrads, mok_port_host.py:218-220). d_w is bf16 [experts, m_rows, n_rows].
 * The data gradients are plb_moe_gemm_down calls on transposed-quantised weights
 * (d_hidden = d_y . W_down: inter := hidden, hidden := inter; d_x = d_gate_up . [W_gate; W_up]). */
int plb_moe_gemm_gate_up_train(const void* x_routed_fp8, const void* x_routed_sc, const void* w13_fp8,
                               const void* w13_sc, const int32_t* block_expert, const int32_t* num_tokens,
                               int64_t capacity, int experts, int inter, int hidden, void* hidden_fp8,
                               void* hidden_sc, void* gate_fp8, void* gate_sc, void* up_fp8, void* up_sc,
                               void* hidden_bf16, plb_status* status, void* stream);
/* plb_moe_gemm_gate_up_train with the dispatch inside the kernel, as plb_moe_gemm_gate_up_dispatch
 * does it for the inference forward: x_routed_* are filled by the kernel's dispatch warps while the
 * tensor pipe works on the row tiles already complete. scratch_u32: capacity / 256 + 1 words. */
int plb_moe_gemm_gate_up_train_dispatch(const void* const* xq_peers, const void* const* xsc_rows_peers,
                                        const int32_t* peer_rank, const int32_t* peer_token_idx, void* x_routed_fp8,
                                        void* x_routed_sc, const void* w13_fp8, const void* w13_sc,
                                        const int32_t* block_expert, const int32_t* num_tokens, int64_t capacity,
                                        int experts, int inter, int hidden, void* hidden_fp8, void* hidden_sc,
                                        void* gate_fp8, void* gate_sc, void* up_fp8, void* up_sc, void* hidden_bf16,
                                        void* scratch_u32, plb_status* status, void* stream);
int plb_moe_bwd_dy(const void* d_out_bf16, const void* combine_bf16, const float* router_weights,
                   const int32_t* peer_rank, const int32_t* peer_token_idx, const int32_t* dest_row,
                   const int32_t* num_tokens, int64_t capacity, int hidden, int topk, void* d_y_bf16,
                   float* d_router_weights, void* stream);
int plb_moe_swiglu_bwd(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                       const void* d_hidden_bf16, const int32_t* num_tokens, int64_t capacity, int inter,
                       void* d_gate_up_bf16, void* stream);
int plb_moe_gather_rows(const void* src_bf16, const int32_t* peer_rank, const int32_t* peer_token_idx,
                        const int32_t* num_tokens, int64_t capacity, int cols, void* dst_bf16, void* stream);
int plb_moe_gemm_wgrad(const void* a_t_fp8, const void* a_t_sc, const void* b_t_fp8, const void* b_t_sc,
                       const int32_t* expert_offsets, int64_t capacity, int experts, int m_rows, int n_rows,
                       void* d_w_bf16, plb_status* status, void* stream);

/* ------------------------------------------------------------------ expert parallelism
 * One process per GPU; every rank owns tokens [tokens, hidden] and experts/world experts.
 * Peer-visible buffers are plain device allocations shared through CUDA IPC; "*_peers"
 * arguments are device arrays of `world` device pointers (entry `rank` = the local
 * buffer), the counterpart of the provider ABI's peer_addresses[world]
 * (pipec/src/pipec2/host/include/pipelink_host_abi_v2.h:162-180). */

/* Set-up helpers (these DO allocate / map memory and synchronise; not for the hot loop).
 * plb_sym_alloc: zero-filled device allocation that can be exported.
 * plb_ipc_export / import: 64-byte cudaIpcMemHandle_t out / in; import enables peer access. */
int plb_sym_alloc(size_t bytes, void** out);
int plb_sym_free(void* p);
int plb_ipc_export(void* p, void* handle64);
int plb_ipc_import(const void* handle64, void** out);
int plb_ipc_close(void* p);

/* Flag barrier over the group, the stand-in for ops.barrier_all
 * (campaigns/mok/host/mok_port_host.py:178-180): every rank adds 1 to flags[rank] on every
 * peer (fence.acq_rel.sys + red.release.sys) and waits (ld.acquire.sys, bounded) until its
 * own flags[i] reach the generation kept in state[0], which the kernel then advances.
 * flags: u32 [world] per rank, zero at start, never reset. state: u32 [1] local, zero at start.
 * All ranks must launch it in the same order; one CTA, so it cannot starve its peers. */
int plb_ep_barrier(void* const* flags_peers, void* state, int rank, int world, plb_status* status,
                   void* stream);

/* ops.all_gather_top_experts (mok_port_host.py:59-62): copy `bytes` (multiple of 16) from src
 * into slot `rank` of every peer's gather buffer (dst_peers[p] + rank * bytes). Follow with
 * plb_ep_barrier before reading the gathered buffer. */
int plb_ep_publish(const void* src, int64_t bytes, void* const* dst_peers, int rank, int world,
                   void* stream);

/* dispatch_kernel over NVLink (campaigns/mok/port/comm/comm.cu:105-123) on pre-quantised
 * tokens: x_routed[p] = xq_peers[peer_rank[p]][peer_token_idx[p]] (E4M3 bytes and the row's
 * scale words); padding rows become zeros. xq is u8 [tokens, hidden], xsc its
 * [tokens/128, hidden/128, 32, 16] scales, both produced by plb_mxfp8_quantize at home. */
int plb_ep_pull_rows(const void* const* xq_peers, const void* const* xsc_peers,
                     const int32_t* peer_rank, const int32_t* peer_token_idx,
                     const int32_t* num_tokens, int64_t capacity, int64_t hidden,
                     void* x_routed_fp8, void* x_routed_sc, void* stream);
/* The same dispatch on the bulk-copy engine (cp.async.bulk peer -> shared -> local, one request
 * per row and direction; scale words through registers). hidden <= 4096; every xq_peers[r] is
 * 16-byte aligned. scale_rows != 0: xsc_peers point at plb_ep_scale_rows' output instead of the
 * tensor-core layout, so a row's scale words cross NVLink as one 128-byte request instead of one
 * 32-byte sector per word. A load that never completes is reported in `status` (code 1).
 * plb_ep_scale_rows: u32 [tokens, hidden / 128] from xsc (tokens a multiple of 128), at home. */
int plb_ep_pull_rows_bulk(const void* const* xq_peers, const void* const* xsc_peers, const int32_t* peer_rank,
                          const int32_t* peer_token_idx, const int32_t* num_tokens, int64_t capacity, int64_t hidden,
                          void* x_routed_fp8, void* x_routed_sc, int scale_rows, plb_status* status, void* stream);
int plb_ep_scale_rows(const void* xsc, int64_t tokens, int64_t hidden, void* scale_rows_u32, void* stream);

/* Expert-parallel backward, the mirror of dispatch and combine (mok_comm_bwd,
 * campaigns/mok/port/comm/comm.cu:226-262): gradients of routed rows are pulled from the token's
 * home rank and the input gradient rows are pushed back to it.
 * plb_ep_bwd_dy: d_y[p] = router_w_peers[r][dest_row[p]] * d_out_peers[r][peer_token_idx[p]] with
 *   r = peer_rank[p]; padding rows and rows past *num_tokens become zeros.
 * plb_moe_router_grad: at the home rank, d_router_weights[t, j] = <d_out[t], combine[t * topk + j]>
 *   (the same reduction order as plb_moe_bwd_dy, so both give the same bits).
 * plb_ep_gather_rows: plb_moe_gather_rows with the source picked by peer_rank[p] (bf16 rows of x
 *   for the gate/up weight gradient).
 * The input gradient d_x is plb_moe_gemm_down_push on the transposed-quantised gate/up weights into
 * every home rank's [tokens * topk, hidden] buffer, summed over the slots with plb_moe_fwd_epilogue. */
int plb_ep_bwd_dy(const void* const* d_out_peers, const float* const* router_w_peers, const int32_t* peer_rank,
                  const int32_t* peer_token_idx, const int32_t* dest_row, const int32_t* num_tokens, int64_t capacity,
                  int hidden, void* d_y_bf16, void* stream);
int plb_moe_router_grad(const void* d_out_bf16, const void* combine_bf16, int64_t tokens, int topk, int hidden,
                        float* d_router_weights, void* stream);
/* plb_moe_router_grad for a forward pass whose combine rows were pushed into receive streams:
 * slot t * topk + j is read from rows_bf16[row_index[t * topk + j]] (the receive buffer and the
 * index plb_moe_schedule_streams / plb_ep_stream_rows wrote). Same arithmetic, same result. */
int plb_moe_router_grad_indexed(const void* d_out_bf16, const void* rows_bf16, const int32_t* row_index, int64_t tokens,
                                int topk, int hidden, float* d_router_weights, void* stream);
int plb_ep_gather_rows(const void* const* src_peers, const int32_t* peer_rank, const int32_t* peer_token_idx,
                       const int32_t* num_tokens, int64_t capacity, int cols, void* dst_bf16, void* stream);

/* plb_moe_gemm_down with the combine push (combine_kernel, comm.cu:124-129,327): row p is
 * stored to combine_peers[peer_rank[p]][dest_row[p]] from the GEMM epilogue. Rows are ordered by
 * (expert, source rank), so ranks that walked their tiles in the same order would all write to
 * the same home rank at the same time; tile_rotation (>= 0, in 256-row tiles)
 * makes this rank start that many tiles in and wrap around, and tile_stride (>= 1) makes
 * consecutive steps of the tile loop that many row tiles apart (rounded up to the next value
 * coprime to the live tile count), so that the tiles in flight at any moment go to different home
 * ranks. Pass rank * tiles per (expert, source rank) block and those tiles + 1, or 0 and 1. The
 * result does not depend on either. */
int plb_moe_gemm_down_push(const void* hidden_fp8, const void* hidden_sc, const void* w2_fp8,
                           const void* w2_sc, const int32_t* block_expert,
                           const int32_t* num_tokens, const int32_t* dest_row,
                           const int32_t* peer_rank, int64_t capacity, int experts, int inter,
                           int hidden, int tile_rotation, int tile_stride, void* const* combine_peers,
                           plb_status* status, void* stream);

/* plb_ep_pull_rows_bulk + plb_moe_gemm_gate_up in one kernel, the shape of the reference's
 * megakernel, whose comm CTAs dispatch rows while its GEMM CTAs compute
 * (campaigns/mok/port/comm/comm.cu:105-123, campaigns/mok/port/framework/interp_fwd.cu): one warp
 * of every CTA takes row tickets, copies the row peer -> shared -> x_routed with bulk copies (scale
 * words from plb_ep_scale_rows' layout through registers) and counts it into its 256-row tile; the
 * TMA lane acquires a tile's count (256) before its first read of the tile. x_routed_fp8 /
 * x_routed_sc are written exactly as plb_ep_pull_rows writes them. scratch_u32: capacity / 256 + 1
 * words, zeroed on the stream by this call. hidden <= 4096, capacity % 256 == 0.
 * A row that never arrives is reported as status code 1 (its copy) or 5 (the tile's count). */
int plb_moe_gemm_gate_up_dispatch(const void* const* xq_peers, const void* const* xsc_rows_peers,
                                  const int32_t* peer_rank, const int32_t* peer_token_idx, void* x_routed_fp8,
                                  void* x_routed_sc, const void* w13_fp8, const void* w13_sc,
                                  const int32_t* block_expert, const int32_t* num_tokens, int64_t capacity,
                                  int experts, int inter, int hidden, void* hidden_fp8, void* hidden_sc,
                                  void* scratch_u32, plb_status* status, void* stream);

/* bf16 routed precision (the reference's second value of the variant handle
 * pipelink_mok_precision, campaigns/mok/port/act/act.cu:246-249; gemm stage precision variants,
 * campaigns/mok/README.md:99-104): the gate/up and down grouped GEMMs on bf16 operands with fp32
 * accumulation, no quantisation anywhere on the routed path. x_routed_bf16 [capacity, hidden] are
 * the rows in schedule order (plb_moe_gather_rows / plb_ep_gather_rows); w13_bf16
 * [experts, 2*inter, hidden] interleaves, per 256 rows, 128 gate rows then the 128 up rows of the
 * same hidden columns; hidden_bf16 [capacity, inter] = bf16(act(bf16 gate, bf16 up)) under the
 * current plb_moe_set_swiglu_limit. plb_moe_gemm_down_bf16 places rows like plb_moe_gemm_down
 * (combine_bf16 set, combine_peers NULL) or pushes them like plb_moe_gemm_down_push (combine_peers
 * and peer_rank set, combine_bf16 NULL);
 * capacity multiple of 256, inter of 128, hidden of 256. Forward pass only. */
int plb_moe_gemm_gate_up_bf16(const void* x_routed_bf16, const void* w13_bf16, const int32_t* block_expert,
                              const int32_t* num_tokens, int64_t capacity, int experts, int inter, int hidden,
                              void* hidden_bf16, plb_status* status, void* stream);
int plb_moe_gemm_down_bf16(const void* hidden_bf16, const void* w2_bf16, const int32_t* block_expert,
                           const int32_t* num_tokens, const int32_t* dest_row, const int32_t* peer_rank,
                           int64_t capacity, int experts, int inter, int hidden, int tile_rotation,
                           void* combine_bf16, void* const* combine_peers, plb_status* status, void* stream);

/* The backward and recompute cells of the bf16 routed precision (campaigns/mok/README.md:86-104: the
 * bf16 value of pipelink_mok_precision under the bwd and rec passes; same pass structure as the
 * MXFP8 cells, campaigns/mok/port/gemm/gemm.cu:166-243, with no quantisation anywhere).
 * plb_moe_gemm_gate_up_bf16_train: plb_moe_gemm_gate_up_bf16 that also keeps the bf16 gate and up
 *   rows [capacity, inter] the activation backward differentiates through.
 * plb_moe_gemm_wgrad_bf16: plb_moe_gemm_wgrad on bf16 operands: a_t [m_rows, capacity] and b_t
 *   [n_rows, capacity] are the TRANSPOSES of the row-major activations (plb_bf16_transpose), the
 *   contraction runs over each expert's rows of the schedule, out is bf16 [experts, m_rows, n_rows].
 * plb_moe_swiglu_bwd_bf16: plb_moe_swiglu_bwd with bf16 gate / up inputs.
 * The data gradients are plb_moe_gemm_down_bf16 calls on the transposed weights (a reshape on the
 * host at weight load). */
int plb_moe_gemm_gate_up_bf16_train(const void* x_routed_bf16, const void* w13_bf16, const int32_t* block_expert,
                                    const int32_t* num_tokens, int64_t capacity, int experts, int inter, int hidden,
                                    void* hidden_bf16, void* gate_bf16, void* up_bf16, plb_status* status, void* stream);
int plb_moe_gemm_wgrad_bf16(const void* a_t_bf16, const void* b_t_bf16, const int32_t* expert_offsets, int64_t capacity,
                            int experts, int m_rows, int n_rows, void* d_w_bf16, plb_status* status, void* stream);
int plb_moe_swiglu_bwd_bf16(const void* gate_bf16, const void* up_bf16, const void* d_hidden_bf16,
                            const int32_t* num_tokens, int64_t capacity, int inter, void* d_gate_up_bf16, void* stream);
/* dst [cols, rows] = src [rows, cols]^T, bf16, rows and cols multiples of 64. */
int plb_bf16_transpose(const void* src_bf16, int64_t rows, int64_t cols, void* dst_bf16, void* stream);
/* plb_bf16_transpose for a routed buffer sized for the worst case: only the 64-row tiles below *live_rows_dev move. */
int plb_bf16_transpose_live(const void* src_bf16, int64_t rows, int64_t cols, const int32_t* live_rows_dev, void* dst_bf16,
                            void* stream);

/* ops.fwd_epilogue (campaigns/mok/host/mok_port_host.py:204):
 * out[t] = y_shared[t] + sum_j router_weights[t, j] * combine[t * topk + j], j ascending,
 * fp32, every operation rounded separately. y_shared may be NULL. */
int plb_moe_fwd_epilogue(const void* y_shared_bf16, const void* combine_bf16,
                         const float* router_weights, int64_t tokens, int topk, int64_t hidden,
                         void* out_bf16, void* stream);

/* ------------------------------------------------------------------ batch-1 decode
 * One launch decodes one token of a Llama-shaped model (hidden 2048, 32 query / 8 KV heads,
 * head_dim 64, FFN 8192) as a persistent interpreter over per-SM instruction streams: the
 * stand-in for the reference's decode megakernel and its provider arguments
 * (campaigns/megakernel/host/mk_host_abi.h:35-85, MkProviderArgs). All pointers are device
 * addresses. Tensor layouts follow that header: qkv_w [layers,3072,2048], o_w
 * [layers,2048,2048], up_w / gate_w [layers,8192,2048], down_w [layers,2048,8192], norms
 * [layers,2048], lm_head [vocab,2048] (tied embedding table), k_cache / v_cache
 * [layers,max_seq_len,8,64], instructions i32 [num_sms,num_instructions,32]; rope tables are
 * f32 [rows,32] (one entry per rotated pair, interleaved-pair RoPE,
 * campaigns/megakernel/host/export_inputs.py:229-240). Instruction words: 0 opcode, 1 layer,
 * 2-5 operands, 6 counter to wait on (-1 none), 7 its target, 8 counter to bump (-1 none).
 * Opcodes 1-7 as campaigns/megakernel/host/export_inputs.py:49-58; for opcode 2 a non-zero word
 * 5 is 1 + the index of a counter on which the partitions of one KV head count themselves in:
 * the last one to arrive also merges that head's partials (the work of opcode 3) and only it
 * bumps the counter of word 8. 8 = greedy sample
 * (argmax with ties to the lower id, token_out[pos+1], next embedding row into hidden,
 * *pos_dev += 1). The call zeroes `bars` (num_bars counters) on the stream, then launches
 * cooperatively with num_sms CTAs. */
typedef struct plb_decode_args {
  const void *qkv_w, *o_w, *up_w, *gate_w, *down_w, *attn_norm, *mlp_norm, *lm_norm, *lm_head;
  void *k_cache, *v_cache;
  const float *rope_cos, *rope_sin;
  void *hidden, *q_post_rope, *attn_out, *silu_out, *logits;
  float *attn_out_partial, *attn_lse_partial, *argmax_val;
  int32_t* argmax_idx;
  uint32_t* bars;
  const int32_t* instructions;
  int32_t* pos_dev;
  int32_t* token_out;
  plb_status* status;
  int32_t num_instructions, max_seq_len, max_parts, vocab;
  float attn_scale, eps;
  int32_t num_bars, layers;
} plb_decode_args;
int plb_decode_step(const plb_decode_args* args, int num_sms, void* stream);

/* The partial-attention op alone, in the harness layout of the reference's checker
 * (campaigns/megakernel/host/check_cute_attention.cu:16-45): q bf16 [32,64], k / v bf16
 * [length,8,64], out f32 [(kv_head*partitions+part)*4+h, 64] normalised, lse f32 (base 2);
 * an empty partition yields zeros and -inf. */
int plb_decode_attention_partial(const void* q, const void* k, const void* v, float* out,
                                 float* lse, int length, int partitions, float scale,
                                 void* stream);

/* ------------------------------------------------------------------ prefill attention
 * Causal flash-attention forward, bf16, head_dim 128 (the reference's sm90 core,
 * campaigns/attention/src/sm90/role_core.cuh + role_load.cuh + role_epilogue.cuh). Q / O are
 * [q_rows, q_heads, 128], K / V [kv_rows, kv_heads, 128], LSE f32 [batch * q_heads, seq_q]
 * (natural log of the sum of exp of the scaled scores, campaigns/attention/src/slot/family.cuh:156-229).
 * The caller supplies the work list, one record per 128-query tile and head, the counterpart of
 * WorkDesc (campaigns/attention/src/sm90/README.md:107-122); heavy tiles first balances a causal
 * mask. `ready` (optional) holds one counter per 128-key block of K / V: a block is read only once
 * (int32)(ready[block] - ready_target) >= 0, the context-parallel acquire of
 * campaigns/attention/src/sm90/cp_load.cuh:124-137. */
typedef struct plb_attn_work {
  int32_t q_row0;    /* first row of the tile in Q / O */
  int32_t q_pos0;    /* global sequence position of that query */
  int32_t kv_row0;   /* row of key block 0 in K / V */
  int32_t kv_pos0;   /* global sequence position of that key */
  int32_t kv_blocks; /* 128-key blocks to visit */
  int32_t head;      /* query head; the first of two when heads_per_work is 2 */
  int32_t batch;
  int32_t reserved;
} plb_attn_work;
/* heads_per_work: 1 = one record per head; 2 = one record per pair of heads (head, head + 1) that
 * share a KV head (q_heads / kv_heads must be even, head even): K / V are fetched once for both.
 * window > 0: sliding-window mask on top of the causal one, key visible iff kv_pos > q_pos - window
 * (campaigns/attention/src/sm90/stage_mask_window.cu:8-11); the work list should then start each
 * tile at the first block that holds a visible key. softcap > 0: the scaled score becomes
 * softcap * tanh(score * scale / softcap) (campaigns/attention/src/sm90/stage_score_softcap.cu:10-13,
 * family_params.cuh:112-113). 0 switches either off. */
int plb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                      const plb_attn_work* work, int num_work, int heads_per_work, int q_heads, int kv_heads, int seq_q,
                      uint64_t q_rows, uint64_t kv_rows, float scale, int window, float softcap, const uint32_t* ready,
                      uint32_t ready_target, plb_status* status, void* stream);

/* Context-parallel K/V exchange (kv_gather_role_gather, campaigns/attention/src/sm90/stage_kv_gather.cu:16-78):
 * rank r holds chunks r and 2*world-1-r of the sequence (zigzag) as k_local / v_local
 * [2 * chunk_blocks * 128, kv_heads * 128]; every 128-token block (block_bytes bytes of K, same of
 * V) is stored into the gathered global-order buffers of each rank that needs it (early chunk:
 * all ranks; late chunk: ranks <= r), then that rank's ready[global block] is bumped by 1 with
 * fence.acq_rel.sys + red.release.sys. Counters are never reset: launch n makes them n. */
int plb_cp_push_kv(const void* k_local, const void* v_local, int chunk_blocks, int64_t block_bytes,
                   int rank, int world, void* const* k_gather_peers, void* const* v_gather_peers,
                   void* const* ready_peers, int ctas, void* stream);

/* Context-parallel attention with the K/V exchange INSIDE the attention launch
 * (kv_gather_role_gather in the attention CTA, campaigns/attention/src/sm90/stage_kv_gather.cu:16-78;
 * ticket queue and publish of examples/comm-overlap/comm/push_gather.cuh:80-150): two warps of every
 * CTA copy this rank's 128-token K/V blocks, in `parts` pieces each, into the gathered buffers of
 * the ranks that need them and add 1 per piece to that rank's ready[block]; the load lanes wait
 * for ready_target = (launches so far) * parts. k_local / v_local as for plb_cp_push_kv; the
 * gathered buffers, counters and peers tables are the same slab regions; ticket_u32 is one word
 * of scratch, zeroed on the stream by this call. Head pairs only (q_heads / kv_heads even), no
 * window or soft cap. Every CTA of the launch must be resident at once (the grid is one CTA per
 * SM at most), so do not share the GPU with other work while it runs. */
int plb_attention_fwd_cp(const void* q, const void* k_gather, const void* v_gather, void* out, float* lse,
                         const plb_attn_work* work, int num_work, int q_heads, int kv_heads, int seq_q, uint64_t q_rows,
                         uint64_t kv_rows, float scale, const uint32_t* ready, uint32_t ready_target, const void* k_local,
                         const void* v_local, int chunk_blocks, int64_t block_bytes, int parts, int rank, int world,
                         void* const* k_gather_peers, void* const* v_gather_peers, void* const* ready_peers,
                         void* ticket_u32, plb_status* status, void* stream);

/* Receive streams for the combine push. plb_moe_gemm_down_push writes row p to
 * `token * topk + slot` of its home rank: 8 KB rows scattered over every peer's combine buffer,
 * which on eight GPUs costs almost twice the time of the same bytes written in order. With
 * streams, row p goes to position rank * stream_cap + (earlier rows of this rank with the same
 * home) of the home rank's receive buffer [world * stream_cap, hidden], and the home rank reads
 * its (token, slot) rows through an index.
 * plb_ep_stream_rows (after the schedule): stream_row[p] = that position (-1 for padding rows), to
 * be passed to plb_moe_gemm_down_push as dest_row with the receive buffers as combine_peers; and
 * index_peers[peer_rank[p]][dest_row[p]] = stream_row[p], a 4-byte write to the home rank.
 * stream_cap >= rows any one rank can send to any one home (tokens * topk is always enough).
 * plb_moe_fwd_epilogue_indexed (after the group barrier): plb_moe_fwd_epilogue with slot
 * t * topk + j read from rows_bf16[row_index[t * topk + j]]. Same arithmetic, same result. */
int plb_ep_stream_rows(const int32_t* peer_rank, const int32_t* dest_row, const int32_t* num_tokens, int64_t capacity,
                       int rank, int world, int64_t stream_cap, int32_t* stream_row, void* const* index_peers,
                       void* stream);
/* plb_moe_schedule with the receive-stream positions written by the same launches (no separate
 * plb_ep_stream_rows pass): stream_row and the home ranks' index come out exactly as that pass
 * writes them, because inside an expert segment the rows of one source rank form one run and the
 * counts the schedule already keeps give every run's place in its stream. Needs
 * tokens * topk % 1024 == 0 (PLB_E_ARGUMENT otherwise; use the two-call form then) and scratch of
 * plb_moe_schedule_streams_scratch_bytes(). The reference builds its schedule on the host before
 * the kernel (campaigns/mok/host/mok_port_host.py:59-69); the stream positions have no counterpart
 * there (its combine writes token * topk + slot, campaigns/mok/port/comm/comm.cu:124-129). */
size_t plb_moe_schedule_streams_scratch_bytes(int world, int tokens, int topk, int num_local_experts);
int plb_moe_schedule_streams(const int32_t* routes, int world, int tokens, int topk, int expert_base,
                             int num_local_experts, int capacity, int padding, int32_t* peer_rank,
                             int32_t* peer_token_idx, int32_t* dest_row, int32_t* num_tokens,
                             int32_t* tokens_per_expert, int32_t* expert_offsets, int32_t* block_expert,
                             void* scratch, size_t scratch_bytes, int rank, int64_t stream_cap,
                             int32_t* stream_row, void* const* index_peers, plb_status* status,
                             void* stream);
int plb_moe_fwd_epilogue_indexed(const void* y_shared_bf16, const void* rows_bf16, const int32_t* row_index,
                                 const float* router_weights, int64_t tokens, int topk, int64_t hidden,
                                 void* out_bf16, void* stream);

/* Tensor-parallel GEMM compositions (examples/comm-overlap: `ag` = C_r = gather(A_q) @ B_r^T,
 * `rs` = rows [r*M/W, (r+1)*M/W) of sum_q A_q @ B_q^T; README "AllGather protocol" and
 * "ReduceScatter protocol"), bf16 operands, fp32 accumulation, bf16 results.
 *
 * plb_tp_push_rows: the all-gather side. `src` is this rank's shard, `blocks` row blocks of
 * block_bytes each (a block = 256 rows, the GEMM's tile height); every block is copied, in `parts`
 * pieces, into gather_peers[c] at the shard's place for every c != rank, and each piece adds 1 to
 * ready_peers[c][rank * blocks + block] with release semantics at system scope (the rank's own
 * counters advance too; its shard must already sit in its gathered buffer). After step g (1-based)
 * a complete block's counter reads g * parts.
 *
 * plb_tp_gemm_bf16: out[dest_row[i]] = A[i, :] @ B^T for the m rows of A ([m, k] bf16; B [n, k]),
 * CTA pairs on 256 x 256 tiles starting `tile_rotation` row tiles in. `ready` (nullable): the
 * loads of row tile t wait, bounded, for ready[t] >= ready_target (status code 5 if it never
 * comes). Exactly one of out_bf16 (local placement) and out_peers (row i goes to
 * out_peers[peer_rank[i]], the reduce-scatter push into the owner's receive slots; the owner then
 * sums its slots in rank order with plb_moe_fwd_epilogue on unit weights) is given.
 * block_group: m / 128 zeros; num_rows: device int32 holding m. The pushing kernel of a step must
 * be launched before that step's GEMM on the same stream, and a group barrier (plb_ep_barrier)
 * separates the steps: a GEMM never waits for a kernel that is queued behind it on its own GPU. */
int plb_tp_push_rows(const void* src, int blocks, int64_t block_bytes, int parts, int rank, int world,
                     void* const* gather_peers, void* const* ready_peers, int ctas, void* stream);
int plb_tp_gemm_bf16(const void* a_bf16, const void* b_bf16, const int32_t* block_group, const int32_t* num_rows,
                     const int32_t* dest_row, const int32_t* peer_rank, int64_t m, int n, int k, int tile_rotation,
                     const uint32_t* ready, uint32_t ready_target, void* out_bf16, void* const* out_peers,
                     plb_status* status, void* stream);

/* ------------------------------------------------------------------ linked images
 * Load and launch a linked pipeline image (`pipeline.cubin` + `link.json` of the link driver):
 * the roles of CudaBackend in the reference (pipec/src/pipec2/host/cuda.py:123-286: module load,
 * one launch with the block size, dynamic shared memory and params image the link recorded;
 * stream-only work, so a launch can be captured into a CUDA graph). params_image points to host
 * memory holding link.json's params.total_bytes bytes (stage blobs at their recorded offsets). */
int plb_image_load(const void* image, const char* symbol, int dyn_smem_bytes, void** library,
                   void** kernel);
int plb_image_launch(void* kernel, int grid_x, int grid_y, int grid_z, int threads,
                     int dyn_smem_bytes, const void* params_image, void* stream);
/* plb_image_launch for an image whose CTAs wait on one another (dependency counters between SMs, as the
 * decode interpreter's): a cooperative launch, so that every CTA of the grid is resident. */
int plb_image_launch_cooperative(void* kernel, int grid_x, int threads, int dyn_smem_bytes, const void* params_image,
                                 void* stream);
/* The 128-byte tensor map the decode interpreter reads a KV cache through (bf16 [layers, max_seq_len, 8, 64];
 * box = 128 tokens of one KV head, 128-byte swizzle): plb_decode_step builds it internally, a host that launches
 * the linked decode image (stages/decode) places two of them in the stream owner's parameter block. */
int plb_decode_kv_map(void* out128, const void* cache_bf16, int layers, int max_seq_len);
int plb_image_unload(void* library);

/* Encode a 2-D byte tensor map (what an owner's provider writes into its residue,
 * examples/hopper-gemm-split/host/owner/provider.cpp:13-48): [rows, row_bytes] row-major, box
 * box_rows x box_bytes, optional 128-byte swizzle; out128 receives the 128-byte CUtensorMap. */
int plb_tensor_map_2d_u8(void* out128, const void* base, uint64_t rows, uint64_t row_bytes,
                         uint32_t box_rows, uint32_t box_bytes, int swizzle128);
/* The same for a row-major [rows, cols] tensor of 32-bit words without swizzle (the scale tensors
 * seen as one 128-word row per 512-byte scale block). */
/* The same for a bf16 [rows, cols] tensor: coordinates and box in elements (with the 128-byte swizzle a box row is
 * 64 elements). The prefill attention image's Q / K / V maps: box 128 rows x 64 columns. */
int plb_tensor_map_2d_bf16(void* out128, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                           uint32_t box_cols, int swizzle128);
int plb_tensor_map_2d_u32(void* out128, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                          uint32_t box_cols);

#ifdef __cplusplus
}
#endif
#endif /* PIPELINK_B200_H */
