// Shared by the tensor-import stages: the argument record the consumer hands to a provider's
// `produce` callable, the consumer's params block, and the handle functions the link binds.
#pragma once
#include <stdint.h>
#include <pipelink/stage.hpp>
#include <pipelink/tensor_source.h>

constexpr int kTiTile = 128;   // the exported tile is 128 x 128 f32

struct TiTileArgs {
  const float* input;   // row-major [128][ld]
  int ld;
};
struct TiConsumerParams {
  const float* input;   // [tiles * 128][ld]
  const float* bias;    // [128]
  float* output;        // [tiles * 128][128]
  int ld;
  float scale;
};

PL_TYPE(TiTileArgs);

#ifdef __CUDACC__
extern "C" __device__ int pipelink_tmem_slot();     // shared-memory byte offset of the published TMEM base
extern "C" __device__ int pipelink_ti_acc();        // provider: first TMEM column of the exported tile
extern "C" __device__ int pipelink_ti_tile();       // provider: shared-memory byte offset of the exported tile
extern "C" __device__ int pipelink_ti_scratch();    // consumer: shared-memory byte offset of the lent scratch
extern "C" __device__ int pipelink_ti_barrier();    // consumer: named barrier lent to the import
#endif
