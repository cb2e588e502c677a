// Shared vocabulary of the three-stage MXFP8 GEMM (TMA load -> tcgen05 MMA -> epilogue):
// parameter blocks, tile constants and the link-time handles the stages read.
//
// sm_100a counterpart of the reference's teaching pipeline
// examples/hopper-gemm-split/src/{channels.cuh,load.cu,mma.cu,epilogue.cuh}: same split into
// a load owner, an MMA owner and an epilogue owner joined by an `operands` ring (depth bound
// at link time) and a depth-one `accumulator` channel, with E4M3 operands + UE8M0 scales, the
// accumulator kept in tensor memory, and bias + SiLU -> bf16 as the epilogue.
//
// Every pipelink_* function below is resolved by the linker-generated binding stub; after LTO
// each call folds to a constant.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <pipelink/stage.hpp>

#ifndef PIPELINK_EMIT
#include "../../csrc/common.cuh"
#endif

namespace gemm3 {
constexpr int TileM = 128, TileN = 128, TileK = 128;          // TileK in bytes = E4M3 elements
constexpr int OperandBytes = TileM * TileK;                   // 16 KiB each for A and B
constexpr int ScaleBytes = 512;                               // one 128-row x 4-group scale block
constexpr int SlotBytes = 2 * OperandBytes + 2 * ScaleBytes;  // 33,792
constexpr int ScaleColsPerSlot = 8;                           // TMEM columns: 4 (A) + 4 (B)
constexpr int AccCols = TileN;
}  // namespace gemm3

struct alignas(64) Gemm3LoadParams {
  CUtensorMap a;          // [M, K] u8, box 128 x 128, 128-byte swizzle
  CUtensorMap b;          // [N, K] u8
  const uint8_t* a_sc;    // [M/128, K/128, 32, 16]
  const uint8_t* b_sc;    // [N/128, K/128, 32, 16]
  int K;
  int pad;
};
struct alignas(16) Gemm3MmaParams {
  int K;
  int pad[3];
};
struct alignas(16) Gemm3EpilogueParams {
  const void* bias;  // bf16 [N]
  void* out;         // bf16 [M, N]
  int N;
  int pad;
};

extern "C" __device__ int pipelink_gemm_depth();
extern "C" __device__ int pipelink_gemm_operands();    // smem byte offset of the ring
extern "C" __device__ int pipelink_gemm_full();        // first mbarrier slot (16 bytes each)
extern "C" __device__ int pipelink_gemm_empty();
extern "C" __device__ int pipelink_gemm_acc_ready();   // mbarrier slot: accumulator complete
extern "C" __device__ int pipelink_gemm_acc_empty();   // mbarrier slot: accumulator drained (one arrival per epilogue warp)
extern "C" __device__ int pipelink_gemm_acc();         // first TMEM column of the accumulator
extern "C" __device__ int pipelink_gemm_sf();          // first TMEM column of the scale slots
extern "C" __device__ int pipelink_tmem_slot();        // smem byte offset where dispatch put the TMEM base
extern "C" __device__ int pipelink_gemm_warp_epilogue();

#ifndef PIPELINK_EMIT
namespace gemm3 {
__device__ __forceinline__ uint32_t barrier_addr(uint32_t smem_base, int base, int slot = 0) {
  return smem_base + 16u * static_cast<uint32_t>(base + slot);
}
// Bounded parity wait without a status record: returns false when the budget runs out.
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!plb::mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > plb::kWaitBudgetCycles) return false;
  }
  return true;
}
}  // namespace gemm3
#endif  // !PIPELINK_EMIT

// ---- the contracts the three owners share (annotations: <pipelink/stage.hpp>) ----
#ifdef PIPELINK_EMIT
namespace gemm3 {
inline pl::endpoint operands(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("smem").scope("cta").proxy("async")
      .tile("e4m3+ue8m0", {2, 128, 128})
      .layout_smem(8, {2, 128, 128}, {OperandBytes, 128, 1}, 3, 4, 3)
      .ring(pl::depth::handle("pipelink_gemm_depth"), SlotBytes)
      .mbarrier(pl::arrivals("pipelink_gemm_full", 1, "load", SlotBytes), pl::arrivals("pipelink_gemm_empty", 1, "mma"), "load")
      .bind("base", "pipelink_gemm_operands").bind("full", "pipelink_gemm_full").bind("empty", "pipelink_gemm_empty");
}
inline pl::endpoint accumulator(const char* direction, const char* role) {
  return pl::endpoint(direction, role).space("tmem").scope("cta").proxy("async")
      .tile("f32", {128, AccCols})
      .layout_tmem(32, 0, 128, AccCols)
      .ring(pl::depth::fixed(1), 128 * AccCols * 4)
      .mbarrier(pl::arrivals("pipelink_gemm_acc_ready", 1, "mma"), pl::arrivals("pipelink_gemm_acc_empty", 4, "epilogue"), "mma")
      .bind("base", "pipelink_gemm_acc").bind("full", "pipelink_gemm_acc_ready").bind("empty", "pipelink_gemm_acc_empty");
}
}  // namespace gemm3
#endif

#define GEMM3_TOPOLOGY() PL_TOPOLOGY(pl::topology().cta_group(1).cluster(1, 1, 1))
#define GEMM3_CLAIM_OPERANDS()                                                                     \
  PL_CLAIM(smem, pipelink_gemm_operands, pl::per("pipelink_gemm_depth", gemm3::SlotBytes), 1024);  \
  PL_CLAIM(mbarrier, pipelink_gemm_full, pl::per("pipelink_gemm_depth", 1), 1);                    \
  PL_CLAIM(mbarrier, pipelink_gemm_empty, pl::per("pipelink_gemm_depth", 1), 1)
#define GEMM3_CLAIM_ACCUMULATOR()                                      \
  PL_CLAIM(tmem, pipelink_gemm_acc, pl::units(gemm3::AccCols), 32);    \
  PL_CLAIM(mbarrier, pipelink_gemm_acc_ready, pl::units(1), 1);        \
  PL_CLAIM(mbarrier, pipelink_gemm_acc_empty, pl::units(1), 1)
