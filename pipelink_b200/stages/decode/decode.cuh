// Shared vocabulary of the decode interpreter's two stage owners: parameter blocks, link-time
// handles, the layout policy that reads them, and the contracts both owners state.
//
// The linked image is the persistent decode interpreter of csrc/decode.cu cut along its warp
// roles (the reference links its decode megakernel from separately packed owners the same way and
// gates the linked build within 1 % of the single-unit build, campaigns/megakernel/README.md):
//   decode.stream     1 warp    walks the CTA's instruction stream ahead of the interpreter and
//                               streams weight rows and K/V tiles into the ring (bulk copies, TMA)
//   decode.interpret  16 warps  the opcode interpreter: matvec partial sums from the ring, the
//                               ops' epilogues, partial attention, dependency counters
// joined by a `weights` ring in shared memory whose depth is bound at link time (32 KB stages,
// full: one arrival + transaction bytes, empty: one arrival per interpreter warp) and an
// `instructions` hand-off (the interpreter copies the CTA's instruction words to shared memory
// once, the stream owner waits for them). Both device bodies are the library kernel's own
// (csrc/decode_roles.cuh), so a linked launch computes what the library launch computes.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <pipelink/stage.hpp>

#include "../../../include/pipelink_b200.h"

#ifndef PIPELINK_EMIT
#include "../../csrc/decode_roles.cuh"
#endif

struct alignas(16) DecInterpretParams {
  plb_decode_args args;          // the argument block of plb_decode_step, as the library kernel takes it
};
struct alignas(64) DecStreamParams {
  CUtensorMap map_k, map_v;      // KV cache [layers, max_seq_len, 8, 64] bf16, box = 128 tokens of one head
  plb_decode_args args;
};

namespace decstage {
constexpr int StageBytes = 32768;
constexpr int InterpretWarps = 16;
constexpr int PartialBytes = 2048 * 4;
constexpr int ScratchBytes = (256 + 16 * 8 + 16 * 256 + 256 + 8) * 4;
constexpr int InstBytes = 6144;
}  // namespace decstage

extern "C" __device__ int pipelink_dec_depth();
extern "C" __device__ int pipelink_dec_ring();        // smem byte offset of the ring
extern "C" __device__ int pipelink_dec_full();        // first mbarrier slot (16 bytes each)
extern "C" __device__ int pipelink_dec_empty();
extern "C" __device__ int pipelink_dec_inst_ready();  // mbarrier slot: instruction words are in shared memory
extern "C" __device__ int pipelink_dec_partial();     // smem byte offset: per-row partial sums
extern "C" __device__ int pipelink_dec_scratch();     // smem byte offset: attention workspace / argmax
extern "C" __device__ int pipelink_dec_inst();        // smem byte offset: copy of the instruction stream

#ifndef PIPELINK_EMIT
static_assert(sizeof(plb_decode_args) == sizeof(plb::DecodeGlobals), "decode argument blocks differ");
static_assert(decstage::StageBytes == plb::dec::kStageBytes && decstage::PartialBytes == plb::dec::kPartialFloats * 4 &&
              decstage::ScratchBytes == plb::dec::kAttnSmemFloats * 4 && decstage::InstBytes == plb::dec::kInstSmemBytes &&
              decstage::InterpretWarps == plb::dec::kDecWarps, "the claims state the sizes the roles use");

namespace decstage {
// The image's shared-memory map, from the link.
struct LinkedLayout {
  __device__ static int depth() { return pipelink_dec_depth(); }
  __device__ static int ring() { return pipelink_dec_ring(); }
  __device__ static uint32_t full(uint32_t smem, int slot) { return smem + 16u * static_cast<uint32_t>(pipelink_dec_full() + slot); }
  __device__ static uint32_t empty(uint32_t smem, int slot) { return smem + 16u * static_cast<uint32_t>(pipelink_dec_empty() + slot); }
  __device__ static int partial() { return pipelink_dec_partial(); }
  __device__ static int scratch() { return pipelink_dec_scratch(); }
  __device__ static int inst() { return pipelink_dec_inst(); }
};
}  // namespace decstage
#endif

// ---- the contracts the two owners share
#ifdef PIPELINK_EMIT
namespace decstage {
// 32 KB stages: sixteen 2 KB warp tasks of one weight matrix, or 128 tokens of K then V of one KV
// head. The stream owner states per stage how many bytes its barrier expects (a block's last stage
// may be short); an interpreter warp releases a stage with one arrival.
inline pl::endpoint weights(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("smem").scope("cta").proxy("async")
      .tile("u8", {StageBytes})
      .layout_smem(8, {StageBytes}, {1})
      .ring(pl::depth::handle("pipelink_dec_depth"), StageBytes)
      .mbarrier(pl::arrivals("pipelink_dec_full", 1, "stream", StageBytes),
                pl::arrivals("pipelink_dec_empty", InterpretWarps, "interpret"), "stream")
      .bind("base", "pipelink_dec_ring").bind("full", "pipelink_dec_full").bind("empty", "pipelink_dec_empty");
}
// The CTA's instruction words, copied to shared memory once per launch by the interpreter's
// threads; one arrival tells the stream owner they are there.
inline pl::endpoint instructions(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("smem").scope("cta").proxy("generic")
      .tile("s32", {InstBytes / 4})
      .layout_smem(32, {InstBytes / 4}, {1})
      .ring(pl::depth::fixed(1), InstBytes)
      .mbarrier_full_only(pl::arrivals("pipelink_dec_inst_ready", 1, "interpret"), "interpret")
      .bind("base", "pipelink_dec_inst").bind("full", "pipelink_dec_inst_ready");
}
}  // namespace decstage
#endif

#define DEC_TOPOLOGY() PL_TOPOLOGY(pl::topology().cta_group(1).cluster(1, 1, 1).persistent().scheduler("static"))
#define DEC_CLAIM_RING()                                                                              \
  PL_CLAIM(smem, pipelink_dec_ring, pl::per("pipelink_dec_depth", decstage::StageBytes), 1024);       \
  PL_CLAIM(mbarrier, pipelink_dec_full, pl::per("pipelink_dec_depth", 1), 1);                         \
  PL_CLAIM(mbarrier, pipelink_dec_empty, pl::per("pipelink_dec_depth", 1), 1)
#define DEC_CLAIM_INSTRUCTIONS()                                                  \
  PL_CLAIM(smem, pipelink_dec_inst, pl::units(decstage::InstBytes), 16);          \
  PL_CLAIM(mbarrier, pipelink_dec_inst_ready, pl::units(1), 1)
