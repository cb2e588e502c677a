// Stage ti.consumer (and, with -DTI_BY_COLUMN, ti.consumer.by-column): one four-warp role asks a
// provider it does not know for a 128 x 128 f32 tile, imports it through the adapter the link
// generated for the connection, and writes out[m][n] = max(tile[m][n] * scale + bias[m], 0).
// Its demand: thread t holds row t, position p = column p (by-column: thread t holds COLUMN t,
// position p = row p). The source is the same for a tensor-memory provider, a transposed one and a
// shared-memory one; only the link's plan differs. The reference's hand-written consumer of its
// many-producers example follows the same schedule, produce -> ready -> import -> arithmetic ->
// done -> release (examples/one-epilogue-many-producers/consumer/epilogue.cu).
#include "ti.cuh"

extern "C" __device__ pipelink_tensor_source pipelink_call_tensor_produce(const TiTileArgs* args, void* frame);
extern "C" __device__ void pipelink_call_tensor_release(const TiTileArgs* args);
extern "C" __device__ void ti_import_acc(pipelink_tensor_source source, float* dest, void* scratch);
extern "C" __device__ void ti_import_acc_ready();
extern "C" __device__ void ti_import_acc_done();
extern "C" __device__ void ti_epilogue(const void* params, unsigned variant);
#ifdef TI_BY_COLUMN
PL_STAGE("ti.consumer.by-column", "1.0.0");
#else
PL_STAGE("ti.consumer", "1.0.0");
#endif
PL_PARAMS(TiConsumerParams, input, bias, output, ld, scale);
PL_ROLE(epilogue, ti_epilogue, 4);
PL_CLAIM_WARPS(pipelink_ti_warp_epilogue, epilogue, 4, 4);     // a warpgroup: thread t may read TMEM lane t
PL_CALL(tensor_produce, pipelink_call_tensor_produce, pl::produce, "epilogue", "produce");
PL_CALL(tensor_release, pipelink_call_tensor_release, pl::produce, "epilogue", "release");

#ifndef PIPELINK_EMIT
extern "C" __device__ void ti_epilogue(const void* raw_params, unsigned) {
  const TiConsumerParams& p = *static_cast<const TiConsumerParams*>(raw_params);
  extern __shared__ __align__(1024) unsigned char pl_smem[];
  // one tile per CTA: tile b is rows [128 b, 128 b + 128) of the input and of the output
  TiTileArgs args{p.input + static_cast<size_t>(blockIdx.x) * kTiTile * p.ld, p.ld};
  float* out = p.output + static_cast<size_t>(blockIdx.x) * kTiTile * kTiTile;
  const pipelink_tensor_source source = pipelink_call_tensor_produce(&args, nullptr);
  ti_import_acc_ready();
  float acc[kTiTile];
  ti_import_acc(source, acc, pl_smem + pipelink_ti_scratch());
  const int t = static_cast<int>(threadIdx.x & 127);
#ifdef TI_BY_COLUMN
#pragma unroll
  for (int m = 0; m < kTiTile; ++m) {
    const float v = acc[m] * p.scale + p.bias[m];
    out[m * kTiTile + t] = v > 0.0f ? v : 0.0f;
  }
#else
  const float bias = p.bias[t];
#pragma unroll
  for (int n = 0; n < kTiTile; n += 4) {
    float4 v;
    float* lanes = reinterpret_cast<float*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x = acc[n + i] * p.scale + bias;
      lanes[i] = x > 0.0f ? x : 0.0f;
    }
    *reinterpret_cast<float4*>(out + t * kTiTile + n) = v;
  }
#endif
  ti_import_acc_done();
  pipelink_call_tensor_release(&args);
}
#endif
