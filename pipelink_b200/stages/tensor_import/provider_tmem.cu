// Stage ti.provider.tmem (and, with -DTI_TRANSPOSED, ti.provider.tmem-transposed): a role-less
// provider that exports a 128 x 128 f32 tile in tensor memory. `produce` runs on the four warps
// of its caller: thread L owns TMEM lane L and stores the 128 words of that lane. Natural
// placement: element (m, n) at lane m, column n. Transposed: lane n, column m, which no consumer
// thread can read in place, so the link stages it through the consumer's scratch.
// The reference's tensor-memory provider of its many-producers example has the same shape of
// interface (examples/one-epilogue-many-producers/providers/accumulator/producer_m128.cu).
#include "ti.cuh"

extern "C" __device__ pipelink_tensor_source ti_tmem_produce(const TiTileArgs* args, void* frame);
extern "C" __device__ void ti_tmem_release(const TiTileArgs* args);
#ifdef TI_TRANSPOSED
PL_STAGE("ti.provider.tmem-transposed", "1.0.0");
#else
PL_STAGE("ti.provider.tmem", "1.0.0");
#endif
PL_NO_PARAMS();
PL_EXPORT(produce, ti_tmem_produce);
PL_EXPORT(release, ti_tmem_release);
PL_CALL(tensor_produce, ti_tmem_produce, pl::consume, "produce");
PL_CALL(tensor_release, ti_tmem_release, pl::consume, "release");
PL_CLAIM(tmem, pipelink_ti_acc, pl::units(kTiTile), 32);

#ifndef PIPELINK_EMIT
extern "C" __device__ pipelink_tensor_source ti_tmem_produce(const TiTileArgs* args, void*) {
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(pl_smem + pipelink_tmem_slot()) +
                        static_cast<uint32_t>(pipelink_ti_acc());
  const int lane = static_cast<int>(threadIdx.x & 127);            // the caller's role starts on a warpgroup
  const uint32_t taddr = base + (static_cast<uint32_t>(lane & ~31) << 16);
#pragma unroll
  for (int c0 = 0; c0 < kTiTile; c0 += 8) {
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#ifdef TI_TRANSPOSED
      w[k] = __float_as_uint(args->input[static_cast<size_t>(c0 + k) * args->ld + lane]);   // lane n, column m
#else
      w[k] = __float_as_uint(args->input[static_cast<size_t>(lane) * args->ld + c0 + k]);   // lane m, column n
#endif
    }
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr + c0), "r"(w[0]),
                 "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  return pl::source_of_tmem(base);
}
extern "C" __device__ void ti_tmem_release(const TiTileArgs*) {}
#endif
