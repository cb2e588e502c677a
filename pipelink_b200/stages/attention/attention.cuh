// Shared vocabulary of the prefill attention kernel's stage owners: parameter blocks, link-time
// handles, the layout policy that reads them, and the contracts the owners state.
//
// The linked image is the two-heads-per-CTA causal prefill kernel of csrc/attention.cu cut along
// its warp roles, the way the reference composes its attention kernel from stage packages (load,
// mma, softmax, mask and score variants, the K/V gather of context parallelism:
// campaigns/attention/src/sm90/stage_*.cu):
//   attn.load / attn.load.counters     1 warp   TMA: both Q tiles per record, K and V blocks through two rings;
//                                               the counters form acquires a key block's readiness counter first
//   attn.mma                           1 warp   S_t = Q_t K^T and O_t += P_t V on tcgen05, S / P / O in tensor memory
//   attn.gather.none / attn.gather.push 2 warps nothing, or the context-parallel K/V exchange by ticket
//   attn.softmax / attn.softmax.softcap 8 warps online softmax with deferred rescale, final O / l and LSE;
//                                               the softcap form applies c * tanh(s / c) to the scaled scores
// joined by `q_tiles` (depth 1), `k_tiles` and `v_tiles` (depth bound at link time) in shared memory
// and `scores` / `output` in tensor memory (one slot per head of the pair; the softmax warps of a head
// arrive 128 strong). The device bodies are the library kernel's own (csrc/attention_roles.cuh).
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <pipelink/stage.hpp>

#ifndef PIPELINK_EMIT
#include "../../csrc/attention_roles.cuh"
#endif

// plb::AttnParams (csrc/attention.h), field for field, in plain types so that the manifest pass sees it.
struct AttnParamsImage {
  const void* work;
  int num_work, q_heads, q_per_kv, seq_q;
  void* out;
  float* lse;
  float scale_log2, cap_in, cap_out;
  int window;
  unsigned ready_target;
  const unsigned* ready;
  void* status;
  const void* push_k;
  const void* push_v;
  void* const* push_k_peers;
  void* const* push_v_peers;
  unsigned* const* push_ready_peers;
  unsigned* push_ticket;
  int push_chunk_blocks, push_vec_per_part, push_parts, push_rank, push_world;
};
struct alignas(64) AttnLoadParams {
  CUtensorMap map_q, map_k, map_v;   // [rows, heads * 128] bf16, box 128 rows x 64 columns, 128-byte swizzle
  AttnParamsImage p;
};
struct alignas(16) AttnRoleParams {
  AttnParamsImage p;
};

namespace attnstage {
constexpr int TileBytes = 128 * 128 * 2;     // 128 x 128 bf16
}

extern "C" __device__ int pipelink_attn_kv_depth();
extern "C" __device__ int pipelink_attn_q();        // smem byte offsets
extern "C" __device__ int pipelink_attn_k();
extern "C" __device__ int pipelink_attn_v();
extern "C" __device__ int pipelink_attn_q_full();   // mbarrier slots (16 bytes each)
extern "C" __device__ int pipelink_attn_q_empty();
extern "C" __device__ int pipelink_attn_k_full();
extern "C" __device__ int pipelink_attn_k_empty();
extern "C" __device__ int pipelink_attn_v_full();
extern "C" __device__ int pipelink_attn_v_empty();
extern "C" __device__ int pipelink_attn_s_full();
extern "C" __device__ int pipelink_attn_p_full();
extern "C" __device__ int pipelink_attn_o_full();
extern "C" __device__ int pipelink_attn_o_free();
extern "C" __device__ int pipelink_attn_drain();
extern "C" __device__ int pipelink_attn_s();        // first tensor-memory column of S / P (two tiles)
extern "C" __device__ int pipelink_attn_o();        // first tensor-memory column of O (two tiles)
extern "C" __device__ int pipelink_attn_warp_softmax();
extern "C" __device__ int pipelink_tmem_slot();     // smem byte offset where dispatch put the TMEM base

#ifndef PIPELINK_EMIT
static_assert(sizeof(AttnParamsImage) == sizeof(plb::AttnParams) && offsetof(AttnParamsImage, status) == offsetof(plb::AttnParams, status) &&
              offsetof(AttnParamsImage, push_world) == offsetof(plb::AttnParams, push_world) &&
              offsetof(AttnParamsImage, cap_out) == offsetof(plb::AttnParams, cap_out), "parameter image and plb::AttnParams differ");
static_assert(attnstage::TileBytes == plb::attn::kTileBytes, "the claims state the sizes the roles use");

namespace attnstage {
#define ATTN_BAR(name) \
  __device__ static uint32_t name(uint32_t sb, int i = 0) { return sb + 16u * static_cast<uint32_t>(pipelink_attn_##name() + i); }
struct LinkedLayout {
  __device__ static int kv_depth() { return pipelink_attn_kv_depth(); }
  __device__ static int q() { return pipelink_attn_q(); }
  __device__ static int k() { return pipelink_attn_k(); }
  __device__ static int v() { return pipelink_attn_v(); }
  __device__ static int s_col() { return pipelink_attn_s(); }
  __device__ static int o_col() { return pipelink_attn_o(); }
  __device__ static int warp_softmax() { return pipelink_attn_warp_softmax(); }
  ATTN_BAR(q_full) ATTN_BAR(q_empty) ATTN_BAR(k_full) ATTN_BAR(k_empty) ATTN_BAR(v_full) ATTN_BAR(v_empty)
  ATTN_BAR(s_full) ATTN_BAR(p_full) ATTN_BAR(o_full) ATTN_BAR(o_free) ATTN_BAR(drain)
};
#undef ATTN_BAR
__device__ __forceinline__ const plb::AttnParams& params_of(const AttnParamsImage& image) {
  return reinterpret_cast<const plb::AttnParams&>(image);
}
__device__ __forceinline__ uint32_t tmem_base(const unsigned char* smem) {
  return *reinterpret_cast<const volatile uint32_t*>(smem + pipelink_tmem_slot());
}
}  // namespace attnstage
#endif

// ---- the contracts the owners share
#ifdef PIPELINK_EMIT
namespace attnstage {
inline pl::endpoint tiles(const char* direction, const char* role, int heads, const pl::depth& d, const char* base, const char* full,
                          const char* empty) {
  return pl::endpoint(direction, role).space("smem").scope("cta").proxy("async")
      .tile("bf16", {heads, 128, 128})
      .layout_smem(16, {heads, 2, 128, 64}, {TileBytes / 2, 128 * 64, 64, 1}, 3, 4, 3)
      .ring(d, heads * TileBytes)
      .mbarrier(pl::arrivals(full, 1, "load", heads * TileBytes), pl::arrivals(empty, 1, "mma"), "load")
      .bind("base", base).bind("full", full).bind("empty", empty);
}
inline pl::endpoint q_tiles(const char* direction, const char* role) {
  return tiles(direction, role, 2, pl::depth::fixed(1), "pipelink_attn_q", "pipelink_attn_q_full", "pipelink_attn_q_empty");
}
inline pl::endpoint k_tiles(const char* direction, const char* role) {
  return tiles(direction, role, 1, pl::depth::handle("pipelink_attn_kv_depth"), "pipelink_attn_k", "pipelink_attn_k_full",
               "pipelink_attn_k_empty");
}
inline pl::endpoint v_tiles(const char* direction, const char* role) {
  return tiles(direction, role, 1, pl::depth::handle("pipelink_attn_kv_depth"), "pipelink_attn_v", "pipelink_attn_v_full",
               "pipelink_attn_v_empty");
}
// Tensor memory, one slot per head of the pair (128 lanes x 128 fp32 columns each): the MMA owner
// commits a slot's full barrier, the four softmax warps of that head give it back with 128 arrivals.
inline pl::endpoint accum(const char* direction, const char* role, const char* base, const char* full, const char* empty) {
  return pl::endpoint(direction, role).space("tmem").scope("cta").proxy("async")
      .tile("f32", {128, 128})
      .layout_tmem(32, 0, 128, 128)
      .ring(pl::depth::fixed(2), 128 * 128 * 4)
      .mbarrier(pl::arrivals(full, 1, "mma"), pl::arrivals(empty, 128, "softmax"), "mma")
      .bind("base", base).bind("full", full).bind("empty", empty);
}
inline pl::endpoint scores(const char* direction, const char* role) {
  return accum(direction, role, "pipelink_attn_s", "pipelink_attn_s_full", "pipelink_attn_p_full");
}
inline pl::endpoint output(const char* direction, const char* role) {
  return accum(direction, role, "pipelink_attn_o", "pipelink_attn_o_full", "pipelink_attn_o_free");
}
}  // namespace attnstage
#endif

#define ATTN_TOPOLOGY() PL_TOPOLOGY(pl::topology().cta_group(1).cluster(1, 1, 1).persistent().scheduler("static"))
#define ATTN_CLAIM_TILES()                                                                              \
  PL_CLAIM(smem, pipelink_attn_q, pl::units(2 * attnstage::TileBytes), 1024);                           \
  PL_CLAIM(smem, pipelink_attn_k, pl::per("pipelink_attn_kv_depth", attnstage::TileBytes), 1024);       \
  PL_CLAIM(smem, pipelink_attn_v, pl::per("pipelink_attn_kv_depth", attnstage::TileBytes), 1024);       \
  PL_CLAIM(mbarrier, pipelink_attn_q_full, pl::units(1), 1);                                            \
  PL_CLAIM(mbarrier, pipelink_attn_q_empty, pl::units(1), 1);                                           \
  PL_CLAIM(mbarrier, pipelink_attn_k_full, pl::per("pipelink_attn_kv_depth", 1), 1);                    \
  PL_CLAIM(mbarrier, pipelink_attn_k_empty, pl::per("pipelink_attn_kv_depth", 1), 1);                   \
  PL_CLAIM(mbarrier, pipelink_attn_v_full, pl::per("pipelink_attn_kv_depth", 1), 1);                    \
  PL_CLAIM(mbarrier, pipelink_attn_v_empty, pl::per("pipelink_attn_kv_depth", 1), 1)
#define ATTN_CLAIM_ACCUM()                                         \
  PL_CLAIM(tmem, pipelink_attn_s, pl::units(256), 32);             \
  PL_CLAIM(tmem, pipelink_attn_o, pl::units(256), 32);             \
  PL_CLAIM(mbarrier, pipelink_attn_s_full, pl::units(2), 1);       \
  PL_CLAIM(mbarrier, pipelink_attn_p_full, pl::units(2), 1);       \
  PL_CLAIM(mbarrier, pipelink_attn_o_full, pl::units(2), 1);       \
  PL_CLAIM(mbarrier, pipelink_attn_o_free, pl::units(2), 1)

// One load owner per form (keys local / key blocks behind readiness counters): stage id and entry differ.
#define ATTN_LOAD_STAGE(ID, ENTRY)                                                                              \
  extern "C" __device__ void ENTRY(const void* params, unsigned variant);                                       \
  PL_STAGE(ID, "1.0.0");                                                                                        \
  PL_PARAMS(AttnLoadParams, map_q, map_k, map_v, p);                                                            \
  PL_ROLE(load, ENTRY, 1);                                                                                      \
  ATTN_TOPOLOGY();                                                                                              \
  PL_ENDPOINT(q_tiles, attnstage::q_tiles(pl::produce, "load"));                                                \
  PL_ENDPOINT(k_tiles, attnstage::k_tiles(pl::produce, "load"));                                                \
  PL_ENDPOINT(v_tiles, attnstage::v_tiles(pl::produce, "load"));                                                \
  PL_CLAIM_WARPS(pipelink_attn_warp_load, load, 1, 1);                                                          \
  ATTN_CLAIM_TILES()
#define ATTN_SOFTMAX_STAGE(ID, ENTRY)                                                                           \
  extern "C" __device__ void ENTRY(const void* params, unsigned variant);                                       \
  PL_STAGE(ID, "1.0.0");                                                                                        \
  PL_PARAMS(AttnRoleParams, p);                                                                                 \
  PL_ROLE(softmax, ENTRY, 8);                                                                                   \
  ATTN_TOPOLOGY();                                                                                              \
  PL_ENDPOINT(scores, attnstage::scores(pl::consume, "softmax"));                                               \
  PL_ENDPOINT(output, attnstage::output(pl::consume, "softmax"));                                               \
  PL_CLAIM_WARPS(pipelink_attn_warp_softmax, softmax, 8, 4);                                                    \
  ATTN_CLAIM_ACCUM()
#define ATTN_GATHER_STAGE(ID, ENTRY)                                                                            \
  extern "C" __device__ void ENTRY(const void* params, unsigned variant);                                       \
  PL_STAGE(ID, "1.0.0");                                                                                        \
  PL_PARAMS(AttnRoleParams, p);                                                                                 \
  PL_ROLE(gather, ENTRY, 2);                                                                                    \
  ATTN_TOPOLOGY();                                                                                              \
  PL_CLAIM_WARPS(pipelink_attn_warp_gather, gather, 2, 1)
