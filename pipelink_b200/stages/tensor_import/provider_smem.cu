// Stage ti.provider.smem: a role-less provider that exports the same 128 x 128 f32 tile in shared
// memory, rows 512 bytes apart and the words of a row XOR-swizzled by the row (the layout a
// bank-conflict-free transposed read wants): element (m, n) at byte 512 m + 4 (n xor (m mod 32)).
// The consumer never sees that layout; the adapter the link generates composes it with the demand.
#include "ti.cuh"

extern "C" __device__ pipelink_tensor_source ti_smem_produce(const TiTileArgs* args, void* frame);
extern "C" __device__ void ti_smem_release(const TiTileArgs* args);
PL_STAGE("ti.provider.smem", "1.0.0");
PL_NO_PARAMS();
PL_EXPORT(produce, ti_smem_produce);
PL_EXPORT(release, ti_smem_release);
PL_CALL(tensor_produce, ti_smem_produce, pl::consume, "produce");
PL_CALL(tensor_release, ti_smem_release, pl::consume, "release");
PL_CLAIM(smem, pipelink_ti_tile, pl::units(kTiTile * kTiTile * 4), 128);

#ifndef PIPELINK_EMIT
extern "C" __device__ pipelink_tensor_source ti_smem_produce(const TiTileArgs* args, void*) {
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  unsigned char* tile = pl_smem + pipelink_ti_tile();
  const int t = static_cast<int>(threadIdx.x & 127);
  // coalesced: the four warps walk the rows, a lane takes a column of each 32-wide group
  for (int m = t >> 5; m < kTiTile; m += 4)
    for (int n = t & 31; n < kTiTile; n += 32)
      *reinterpret_cast<float*>(tile + 512 * m + 4 * (n ^ (m & 31))) = args->input[static_cast<size_t>(m) * args->ld + n];
  return pl::source_of(tile);      // the import's ready rendezvous publishes the stores
}
extern "C" __device__ void ti_smem_release(const TiTileArgs*) {}
#endif
